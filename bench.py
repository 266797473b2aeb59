#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of the 8B-shape INT8 decoder (32 layers, d_model 4096, 32 query /
8 KV heads, head_dim 128, d_ff 14336 SwiGLU, vocab 128256), batch 128, prompt lengths U[256, 2048],
paged bf16 KV cache (block 16), on N B200s of one box (tensor parallel for N > 1).

    python bench.py --gpus N --steps K --warmup W            # this project's CUDA path
    python bench.py --impl reference --steps K --warmup W    # CPU path (the oracle port) on the host cores

A step is one decode step of the whole batch (one new token per sequence).  Weights and the KV cache
contents are synthetic (seeded, generated on the device; the caches are random fills, not a prefill); token
ids are the model's own greedy samples.  The timed block of K steps is repeated (up to five times inside the
256 decode steps the workload names); `value` is the median block, Q1 / Q3 go to `repeats`.  One JSON line
is printed by rank 0.  At N = 1 the line also carries `extra`: the quantized GEMM (T(FL)OPS, fraction of
peak) and the paged decode attention of the kernel configurations (GB/s), timed the same way, and the same decode
workload in the FP8 x FP8 form of the decoder (`decode_fp8`, one block of K steps).  At N > 1 a
small tensor-parallel decoder is first checked against the CPU decoder on both collective paths
(`tp_parity`); a failure ends the run with a non-zero exit code.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CONFIGS = {
    # the configuration the metric is quoted on
    "llama8b": dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336, vocab=128256,
                    batch=128, prompt_lo=256, prompt_hi=2048),
    # the same layer shape with 4 layers, half the batch and a small vocabulary: small enough for a profiler
    # capture (about 1 GB of weights, 0.3 GB of KV per layer, both above the L2 size)
    "capture": dict(n_layers=4, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336, vocab=32000, batch=64,
                    prompt_lo=256, prompt_hi=2048),
    # the per-rank shapes of the 8B model under 8-way tensor parallelism (GEMM widths, heads) as one GPU sees them,
    # for a per-kernel launch list of what a rank of the 8-GPU run executes (without the cross-GPU waits)
    "tp8rank": dict(n_layers=8, d_model=4096, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1792, vocab=16032, batch=128,
                    prompt_lo=256, prompt_hi=2048),
}
DECODE_STEPS = 256      # decode steps of the workload: every timed step lies inside them

# dram__bytes_read.sum + dram__bytes_write.sum of the decode-attention kernel divided by its algorithmic bytes, from the
# ncu capture summarised in profiles/paged_attention_decode_config3_ncu.md: (1171.3 MB + 22.0 MB) / 1162.8 MB.
ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0263


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None
        self.mark = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def begin_region(self):
        """Samples taken before this call (start-up, warm-up) are dropped unless the region turns out shorter than
        the sampling period, in which case the last samples under the same load are kept."""
        self.mark = len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        lines = self.lines[self.mark:] if len(self.lines) - self.mark >= 3 else self.lines[-6:]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def prompt_lengths(cfg: dict, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return rng.integers(cfg["prompt_lo"], cfg["prompt_hi"] + 1, cfg["batch"]).astype(np.int32)


def quartiles(values):
    v = np.asarray(values, dtype=np.float64)
    return float(np.percentile(v, 25)), float(np.median(v)), float(np.percentile(v, 75))


# --------------------------------------------------------------------------------------- CPU baseline
class CpuSample:
    """The CPU port (oracle) on a bounded sample of the same decode step: `layers` full-size layers over the
    whole batch with the workload's context lengths, plus the lm_head on a slice of the vocabulary.  One
    call of step() is one timed sample; its two parts are scaled separately to the full model."""

    def __init__(self, cfg: dict, layers: int, vocab_rows: int, threads: int, seed: int = 0):
        from oracle import oracle as O
        from oracle.decoder_ref import DecoderRef

        O.set_num_threads(threads)
        self.O = O
        self.cfg, self.layers, self.vocab_rows = cfg, layers, vocab_rows
        rng = np.random.default_rng(seed)
        d, dh, hq, hkv, f = cfg["d_model"], cfg["head_dim"], cfg["n_heads"], cfg["n_kv_heads"], cfg["d_ff"]
        batch = cfg["batch"]
        lens = prompt_lengths(cfg, seed)
        max_len = int(lens.max()) + 256

        def qw(rows, cols):
            q = rng.integers(-127, 128, (rows, cols), dtype=np.int8)
            s = (np.abs(rng.standard_normal(rows)) * 1e-3 + 1e-4).astype(np.float32)
            return q, s

        sample_cfg = dict(n_layers=layers, d_model=d, n_heads=hq, n_kv_heads=hkv, head_dim=dh, d_ff=f,
                          vocab=vocab_rows, max_seq_len=max_len, block_size=16)
        ref = DecoderRef.__new__(DecoderRef)
        ref.cfg, ref.tp, ref.exact, ref.blas = sample_cfg, 1, False, None
        ref.fp8, ref._qrow, ref.sm_count = False, O.quantize_i8_per_row, 148
        ref.w = {"embed": (rng.standard_normal((vocab_rows, d)) * 0.02).astype(np.float32),
                 "final_norm": np.ones(d, np.float32),
                 "layers": [{"attn_norm": np.ones(d, np.float32), "mlp_norm": np.ones(d, np.float32)}
                            for _ in range(layers)]}
        ref.q = {"lm_head": qw(vocab_rows, d),
                 "layers": [{"wqkv": qw((hq + 2 * hkv) * dh, d), "wo": qw(d, hq * dh), "wgu": qw(2 * f, d),
                             "wdown": qw(d, f)} for _ in range(layers)]}
        ref.cos, ref.sin = O.rope_table(max_len, dh, 10000.0)
        ref.begin(batch)
        tile = O.f32_to_bf16(rng.standard_normal(1 << 20, dtype=np.float32))   # synthetic cache contents
        for l in range(layers):
            for pool in (ref.k[l], ref.v[l]):
                flat = pool.reshape(-1)
                reps = -(-flat.size // tile.size)
                flat[:] = np.tile(tile, reps)[: flat.size]
        ref.seq[:] = lens
        self.ref = ref
        self.ids = rng.integers(0, vocab_rows, batch)
        self.xn = rng.standard_normal((batch, d)).astype(np.float32)

    def step(self):
        """Returns (tokens/s of the full model extrapolated from this sample, seconds spent)."""
        cfg, ref, O = self.cfg, self.ref, self.O
        t0 = time.perf_counter()
        _, nxt = ref.step(self.ids)
        t_total = time.perf_counter() - t0
        t0 = time.perf_counter()
        O.linear_w8a8(self.xn, *ref.q["lm_head"])
        t_lm = time.perf_counter() - t0
        self.ids = nxt
        t_layers = max(t_total - t_lm, 1e-9)
        full = t_layers * cfg["n_layers"] / self.layers + t_lm * cfg["vocab"] / self.vocab_rows
        self.last = (t_layers, t_lm)
        return cfg["batch"] / full, t_total + t_lm

    def describe(self) -> str:
        cfg = self.cfg
        return (f"one decode step of batch {cfg['batch']} on the CPU port: {self.layers} of {cfg['n_layers']} layers at "
                f"full size ({self.last[0]:.2f} s) and the lm_head on {self.vocab_rows} of {cfg['vocab']} rows "
                f"({self.last[1]:.2f} s), each scaled to the full model (extrapolated)")

    @property
    def threads(self) -> int:
        return self.O.num_threads()


def cpu_threads(args) -> int:
    """All host threads unless told otherwise; never what a launcher exported as OMP_NUM_THREADS."""
    if args.cpu_threads > 0:
        return args.cpu_threads
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, cfg, rank, world):
    """The CPU arm: the oracle port of the same decode step on the host cores (the reference itself is Rust
    and cannot be built here).  Each step is a bounded sample of the decode step, extrapolated to the full model
    and labelled so; `ms_per_step` is the time the sample itself took."""
    if rank != 0:
        return
    sample = CpuSample(cfg, args.cpu_layers, args.cpu_vocab, cpu_threads(args))
    results = [sample.step() for _ in range(args.warmup + args.steps)]
    timed = results[args.warmup:] or results
    q1, val, q3 = quartiles([v for v, _ in timed])
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * float(np.median([dt for _, dt in timed])),
        "ms_per_full_step_extrapolated": 1000.0 * cfg["batch"] / val,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(args, cfg, world),
        "repeats": {"n": len(timed), "q1": q1, "median": val, "q3": q3},
        "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": sample.threads, "kind": "port",
                         "sample": sample.describe()},
        "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, world):
    return {"workload": f"{args.config}: decode step, batch {cfg['batch']}, prompt lengths U[{cfg['prompt_lo']},"
                        f"{cfg['prompt_hi']}], {cfg['n_layers']} layers d_model {cfg['d_model']} "
                        f"{cfg['n_heads']}q/{cfg['n_kv_heads']}kv heads d_ff {cfg['d_ff']} vocab {cfg['vocab']}, "
                        f"INT8 weights, per-token INT8 activations, bf16 paged KV (block 16)",
            "global_batch": cfg["batch"], "parallelism": f"tp{world}",
            "kv_contents": "random fill, no prefill",
            "l2": "inputs larger than L2: every step streams all weights and the whole KV cache"}


# --------------------------------------------------------------------------------------- tensor-parallel parity
def tp_parity(be, dist, rank, world):
    """A small tensor-parallel decoder on the ranks of this run against the CPU decoder with the same rank count
    (per-rank activation scales at the row-parallel projections), on both collective paths: the finish kernel over
    the mapped peer blocks and ncclAllReduce.  Returns the list of results on rank 0 (None elsewhere) and whether
    every path passed."""
    from fandhe_ai_b200.decoder import Decoder, DecoderConfig, nccl_unique_id

    cfg = dict(n_layers=2, d_model=1024, n_heads=16, n_kv_heads=8, head_dim=128, d_ff=2048, vocab=2048, max_seq_len=32)
    batch, steps = 8, 8
    rng = np.random.default_rng(17)
    ids = rng.integers(0, cfg["vocab"], (steps, batch)).astype(np.int32)
    weights = want = None
    from oracle.decoder_ref import DecoderRef, make_weights      # the checker

    weights = make_weights(cfg, seed=6)
    if rank == 0:
        ref = DecoderRef(cfg, weights, tp=world)
        ref.begin(batch)
        want = [ref.step(ids[t])[0] for t in range(steps)]
    results, all_ok = [], True
    saved = os.environ.get("B200_TP_EXCHANGE")
    for path in ("exchange", "nccl"):
        os.environ["B200_TP_EXCHANGE"] = "1" if path == "exchange" else "0"
        dc = DecoderConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                           cfg["vocab"], max_batch=batch, max_seq_len=cfg["max_seq_len"], tp_rank=rank, tp_size=world)
        dec = Decoder(be, dc)
        obj = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        dec.init_tp(obj[0])
        used = "exchange" if dec.tp_exchange else "nccl"
        dec.load_weights(weights)
        dec.begin(batch, [steps + 1] * batch)
        worst, finite = 0.0, True
        for t in range(steps):
            dec.step(ids[t])
            got = dec.logits()
            if rank == 0:
                finite = finite and bool(np.all(np.isfinite(got)))
                worst = max(worst, float(np.abs(got - want[t]).max() / np.abs(want[t]).max()))
        dec.close()
        dist.barrier()
        if rank == 0:
            # the ranks' f32 partials may be added in another order than the CPU decoder's, and a last-bit difference
            # can flip an int8 code downstream (1/127 of a row maximum): the bound is quantisation noise
            ok = finite and worst <= 2e-2
            all_ok = all_ok and ok
            results.append({"tp": world, "path": used, "asked_for": path, "worst": worst, "bound": 2e-2, "ok": ok})
    if saved is None:
        os.environ.pop("B200_TP_EXCHANGE", None)
    else:
        os.environ["B200_TP_EXCHANGE"] = saved
    flag = [all_ok]
    dist.broadcast_object_list(flag, src=0)
    return results, flag[0]


# --------------------------------------------------------------------------------------- GPU arm
def run_gpu(args, cfg, rank, world, local_rank):
    from fandhe_ai_b200 import Backend
    from fandhe_ai_b200.decoder import Decoder, DecoderConfig, nccl_unique_id

    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("gloo", rank=rank, world_size=world)

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch

        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local_rank)
    sampler.start()
    be = Backend(local_rank)
    parity = None
    if world > 1 and not args.no_tp_parity:
        parity, ok = tp_parity(be, dist, rank, world)
        if not ok:
            if rank == 0:
                print(json.dumps({"error": "tensor-parallel parity failed", "tp_parity": parity}), flush=True)
            be.close()
            dist.destroy_process_group()
            sys.exit(3)

    warmup = max(args.warmup, 3)
    repeats = max(1, min(5, (DECODE_STEPS - warmup) // max(args.steps, 1)))
    lens = prompt_lengths(cfg, 0)
    total_steps = warmup + repeats * args.steps + 1
    max_seq = int(lens.max()) + total_steps + 1
    blocks_per_seq = -(-max_seq // 16)
    dc = DecoderConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                       cfg["vocab"], max_batch=cfg["batch"], max_seq_len=max_seq, block_size=16,
                       num_blocks=cfg["batch"] * blocks_per_seq, tp_rank=rank, tp_size=world, use_graph=1)
    dec = Decoder(be, dc)
    if world > 1:
        obj = [nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=0)
        dec.init_tp(obj[0])
    dec.init_random(seed=0, std=0.02)
    dec.fill_cache_random(seed=1, std=1.0)
    batch = cfg["batch"]
    first_ids = np.random.default_rng(3).integers(0, cfg["vocab"], batch).astype(np.int32)
    ids = first_ids.copy()
    nxt = np.empty(batch, np.int32)
    ids_p, nxt_p = ids.ctypes.data_as(C.c_void_p), nxt.ctypes.data_as(C.c_void_p)

    # ---- device-resident loop: ids never leave the GPU; `repeats` blocks of K steps, each timed with CUDA events
    dec.begin(batch, (lens + total_steps).tolist(), start_lens=lens.tolist())
    dec.step_raw(ids_p, None)
    for _ in range(warmup - 1):
        dec.step_raw(None, None)
    be.synchronize_device()
    sampler.begin_region()
    block_ms = []
    for _ in range(repeats):
        barrier()
        be.timer_start()
        for _ in range(args.steps):
            dec.step_raw(None, None)
        ms = be.timer_stop()
        barrier()
        block_ms.append(max_over_ranks(ms))
    clocks = sampler.stop()
    q1_ms, ms, q3_ms = quartiles(block_ms)
    value = batch * args.steps / (ms / 1e3)

    # ---- end to end through the public step call over the same steps of the generation: ids from the host every
    #      step (pinned staging inside the call), samples back every step
    dec.begin(batch, (lens + total_steps).tolist(), start_lens=lens.tolist())
    ids[:] = first_ids
    dec.step_raw(ids_p, nxt_p)
    for _ in range(warmup - 1):
        ids[:] = nxt
        dec.step_raw(ids_p, nxt_p)
    block_s = []
    for _ in range(repeats):
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ids[:] = nxt
            dec.step_raw(ids_p, nxt_p)
        dt = time.perf_counter() - t0
        barrier()
        block_s.append(max_over_ranks(dt))
    e2e_q3, e2e_med, e2e_q1 = (batch * args.steps / s for s in quartiles(block_s))

    # ---- roofline of the dominant kernel: the split-K paged attention, timed alone on the same caches
    attn_ms, attn_bytes = dec.time_attention(iters=64)
    peak, peak_kind = read_peaks()
    achieved = attn_bytes / (attn_ms / 1e3) / 1e9
    plan = dec.plan_info()
    launches = dec.launches_per_step * args.steps
    weight_bytes = dec.weight_bytes
    exchange = dec.tp_exchange_mode
    dec.close()

    if rank == 0:
        extra = None
        if world == 1 and not args.no_extra:
            # the other two parts of the metric, timed on this GPU in the same run (CUDA events, rotating operand sets)
            from fandhe_ai_b200 import ACT_NONE, ACT_SILU_GATE, FP8_E4M3, I8
            from fandhe_ai_b200 import bench_kernels as bk

            gemms = []
            for op in (I8, FP8_E4M3):
                for m, n, k, act in ((4096, 4096, 4096, ACT_NONE), (8192, 8192, 8192, ACT_NONE),
                                     (8192, 2 * 14336, 4096, ACT_SILU_GATE), (128, 4096, 4096, ACT_NONE)):
                    gemms.append(bk.measure_gemm(be, op, m, n, k, act, iters=20, warmup=5))
            extra = {"gemm": gemms,
                     "gemm_note": "frac_of_2x_bf16_peak: against twice the measured bf16 burst peak of MEASURED_PEAKS.json "
                                  "(the dense int8 / fp8 rate is twice the bf16 rate); frac_of_4500_nominal: against the "
                                  "vendor's dense figure",
                     "attention_c3": bk.measure_attention_config3(be, iters=20, warmup=5, host_call=False)}
            # the same decode workload in the FP8 x FP8 form (E4M3 weights and activations, f32 accumulation): one block
            # of K steps after the warm-up, device-resident loop
            dc8 = DecoderConfig(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                                cfg["vocab"], max_batch=cfg["batch"], max_seq_len=max_seq, block_size=16,
                                num_blocks=cfg["batch"] * blocks_per_seq, use_graph=1, act_fp8=1)
            dec8 = Decoder(be, dc8)
            dec8.init_random(seed=0, std=0.02)
            dec8.fill_cache_random(seed=1, std=1.0)
            dec8.begin(batch, (lens + total_steps).tolist(), start_lens=lens.tolist())
            ids[:] = first_ids
            dec8.step_raw(ids_p, None)
            for _ in range(warmup - 1):
                dec8.step_raw(None, None)
            be.synchronize_device()
            be.timer_start()
            for _ in range(args.steps):
                dec8.step_raw(None, None)
            ms8 = be.timer_stop()
            dec8.close()
            extra["decode_fp8"] = {"value": batch * args.steps / (ms8 / 1e3), "unit": "tokens/s", "ms_per_step": ms8 / args.steps,
                                   "steps": args.steps, "dtype": "fp8_e4m3 x fp8_e4m3, f32 accumulation",
                                   "note": "same workload and caches as the headline line; weights re-encoded to E4M3 with "
                                           "per-row scales, per-token E4M3 activations"}
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample = CpuSample(cfg, args.cpu_layers, args.cpu_vocab, cpu_threads(args))
            vals, spent = [], 0.0
            while spent < 10.0 and len(vals) < 8:          # about 10 s of CPU work
                v, dt = sample.step()
                vals.append(v)
                spent += dt
            cpu = {"value": float(np.median(vals)), "unit": "tokens/s", "cores": sample.threads, "kind": "port",
                   "sample": sample.describe() + f"; median of {len(vals)} samples"}
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(args, cfg, world),
            "repeats": {"n": repeats, "steps_each": args.steps, "ms_per_step_q1": q1_ms / args.steps,
                        "ms_per_step_median": ms / args.steps, "ms_per_step_q3": q3_ms / args.steps,
                        "e2e_q1": e2e_q1, "e2e_median": e2e_med, "e2e_q3": e2e_q3},
            "collective": ("none" if world == 1 else
                           "row-parallel GEMMs store their partial rows into the owner rank's CUDA-IPC mapped block; one kernel "
                           "per output sums them in rank order, residual + RMSNorm + int8, rows delivered to every rank"
                           if exchange == 2 else
                           "row-parallel outputs finished over CUDA-IPC mapped peer blocks (one kernel: peer loads, "
                           "residual + RMSNorm + int8, rows delivered to every rank)" if exchange else
                           "ncclAllReduce of f32 partials"),
            "e2e": {"value": e2e_med, "unit": "tokens/s", "h2d_bytes_per_step": batch * 4, "d2h_bytes_per_step": batch * 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": "paged_attention_decode_kernel (+ combine_quant)", "bound": "hbm",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": attn_bytes * ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_note": "DRAM read + write bytes of one ncu capture of the same kernel on a smaller case "
                                         "(batch 64, 1.16 GB of KV), scaled by the algorithmic bytes of this launch",
                         "peak_kind": peak_kind, "ms_per_launch": attn_ms,
                         "algorithmic_bytes_per_launch": attn_bytes,
                         "frac_of_8000_nominal": achieved / 8000.0},
            "cpu_baseline": cpu,
            "plan": plan,
            "step_bytes": {"weights_per_rank": weight_bytes, "kv_per_rank_per_layer": attn_bytes},
        }
        if parity is not None:
            line["tp_parity"] = parity
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    be.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="llama8b", choices=sorted(CONFIGS),
                    help="llama8b is the benchmark; the others are small cases for profiler captures")
    ap.add_argument("--cpu-layers", type=int, default=2, help="full-size layers in the CPU sample")
    ap.add_argument("--cpu-vocab", type=int, default=8016, help="lm_head rows in the CPU sample")
    ap.add_argument("--cpu-threads", type=int, default=0, help="threads of the CPU arm (0: every core this process may use)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the GEMM / attention kernel measurements at N = 1")
    ap.add_argument("--no-tp-parity", action="store_true", help="skip the tensor-parallel parity check at N > 1")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): the named batch at every rank count; weak: batch x ranks")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, cfg, rank, world)
        return
    if cfg["n_kv_heads"] % world != 0:
        raise SystemExit(f"{world} ranks do not divide {cfg['n_kv_heads']} KV heads")
    if args.scaling == "weak" and world > 1:
        # the batch grows with the rank count (each rank keeps the KV bytes of one rank of the 1-GPU run)
        cfg = dict(cfg, batch=cfg["batch"] * world)
    run_gpu(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
