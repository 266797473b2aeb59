#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of the 8B-shape INT8 decoder (32 layers, d_model 4096, 32 query /
8 KV heads, head_dim 128, d_ff 14336 SwiGLU, vocab 128256), batch 128, prompt lengths U[256, 2048],
paged bf16 KV cache (block 16), on N B200s of one box (tensor parallel for N > 1).

    python bench.py --gpus N --steps K --warmup W            # this project's CUDA path
    python bench.py --impl reference --steps K --warmup W    # CPU path (the oracle port) on the host cores

A step is one decode step of the whole batch (one new token per sequence).  Weights and the KV cache
contents are synthetic (seeded, generated on the device); token ids are the model's own greedy samples.
One JSON line is printed by rank 0.
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
    # the same layer shape with 4 layers, half the batch and a small vocabulary: small enough for an ncu
    # capture (about 1 GB of weights, 0.3 GB of KV per layer, both above the L2 size)
    "mid": dict(n_layers=4, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=14336, vocab=32000, batch=64,
                prompt_lo=256, prompt_hi=2048),
    # one KV head per GPU (what each rank of an 8-way tensor-parallel run sees): token rows of the pools are
    # 256 bytes, so every KV block is one contiguous 4 KB piece; same KV bytes per layer as llama8b
    "kv1": dict(n_layers=2, d_model=512, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1024, vocab=2048, batch=1024,
                prompt_lo=256, prompt_hi=2048),
    # the attention shape of one rank of the 8B model under 8-way tensor parallelism at batch 128
    "kv1s": dict(n_layers=2, d_model=512, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1024, vocab=2048, batch=128,
                 prompt_lo=256, prompt_hi=2048),
    # the per-rank shapes of the 8B model under 8-way tensor parallelism (GEMM widths, heads), as one GPU sees them
    "tp8rank": dict(n_layers=8, d_model=4096, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1792, vocab=16032, batch=128,
                    prompt_lo=256, prompt_hi=2048),
    # the same with the batch of the weak-scaling run at 8 GPUs (128 sequences per rank)
    "tp8rank1024": dict(n_layers=8, d_model=4096, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1792, vocab=16032,
                        batch=1024, prompt_lo=256, prompt_hi=2048),
    # a small shape for quick functional runs of this script
    "tiny": dict(n_layers=2, d_model=512, n_heads=8, n_kv_heads=8, head_dim=128, d_ff=1024, vocab=2048, batch=16,
                 prompt_lo=32, prompt_hi=128),
}


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

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
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


# --------------------------------------------------------------------------------------- CPU baseline
class CpuSample:
    """The CPU port (oracle) on a bounded sample of the same decode step: `layers` full-size layers over the
    whole batch with the workload's context lengths, plus the lm_head on a slice of the vocabulary.  One
    call of step() is one timed sample; its two parts are scaled separately to the full model."""

    def __init__(self, cfg: dict, layers: int, vocab_rows: int, seed: int = 0):
        from oracle import oracle as O
        from oracle.decoder_ref import DecoderRef

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
        ref.cfg, ref.tp = sample_cfg, 1
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


def run_reference(args, cfg, rank, world):
    """The CPU arm: the oracle port of the same decode step on the host cores (the reference itself is Rust
    and cannot be built here)."""
    if rank != 0:
        return
    sample = CpuSample(cfg, args.cpu_layers, args.cpu_vocab)
    values = [sample.step()[0] for _ in range(args.warmup + args.steps)]
    timed = values[args.warmup:] or values
    val = float(np.median(timed))
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * cfg["batch"] / val,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(args, cfg, world),
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
            "l2": "inputs larger than L2: every step streams all weights and the whole KV cache"}


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

    be = Backend(local_rank)
    lens = prompt_lengths(cfg, 0)
    total_steps = 2 * (args.warmup + args.steps) + 8
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
    if args.attn_chunk_blocks:
        from fandhe_ai_b200 import paged_kv as _pk

        _pk.paged_attention_tuning(be, args.attn_chunk_blocks)
    if args.gemm_splits or args.gemm_tile:
        be.gemm_tuning(args.gemm_tile, args.gemm_splits)
    dec.begin(batch, (lens + total_steps).tolist(), start_lens=lens.tolist())
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], batch).astype(np.int32)
    nxt = np.empty(batch, np.int32)
    ids_p, nxt_p = ids.ctypes.data_as(C.c_void_p), nxt.ctypes.data_as(C.c_void_p)

    # ---- device-resident loop: ids never leave the GPU
    dec.step_raw(ids_p, None)
    for _ in range(max(args.warmup, 3) - 1):
        dec.step_raw(None, None)
    be.synchronize_device()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    be.timer_start()
    for _ in range(args.steps):
        dec.step_raw(None, None)
    ms = be.timer_stop()
    barrier()
    clocks = sampler.stop()
    ms = max_over_ranks(ms)
    value = batch * args.steps / (ms / 1e3)

    # ---- end to end through the public step call: ids from the host every step, samples back every step
    dec.step_raw(ids_p, nxt_p)
    for _ in range(2):
        ids[:] = nxt
        dec.step_raw(ids_p, nxt_p)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ids[:] = nxt
        dec.step_raw(ids_p, nxt_p)
    e2e_s = time.perf_counter() - t0
    barrier()
    e2e_s = max_over_ranks(e2e_s)
    e2e = batch * args.steps / e2e_s

    # ---- roofline of the dominant kernel: the split-K paged attention, timed alone on the same caches
    attn_ms, attn_bytes = dec.time_attention(iters=64)
    peak, peak_kind = read_peaks()
    achieved = attn_bytes / (attn_ms / 1e3) / 1e9
    plan = dec.plan_info()
    launches = dec.launches_per_step * args.steps

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            sample = CpuSample(cfg, args.cpu_layers, args.cpu_vocab)
            vals, spent = [], 0.0
            while spent < 10.0 and len(vals) < 8:          # about 10 s of CPU work
                v, dt = sample.step()
                vals.append(v)
                spent += dt
            cpu = {"value": float(np.median(vals)), "unit": "tokens/s", "cores": sample.threads, "kind": "port",
                   "sample": sample.describe() + f"; median of {len(vals)} samples"}
        line = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": dict(workload_config(args, cfg, world),
                           collective=("none" if world == 1 else
                                       "row-parallel outputs finished over CUDA-IPC mapped peer blocks (one kernel: peer loads, "
                                       "residual + RMSNorm + int8, rows delivered to every rank)" if dec.tp_exchange else
                                       "ncclAllReduce of f32 partials")),
            "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": batch * 4, "d2h_bytes_per_step": batch * 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": {"kernel": "paged_attention_decode_kernel (+ combine_quant)", "bound": "hbm",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": attn_bytes * ATTN_TRAFFIC_PER_ALGORITHMIC_BYTE,
                         "traffic_note": "DRAM read + write bytes of one ncu capture of the same kernel on a smaller case "
                                         "(batch 64, 1.16 GB of KV), scaled by the algorithmic bytes of this launch",
                         "peak_kind": peak_kind, "ms_per_launch": attn_ms,
                         "algorithmic_bytes_per_launch": attn_bytes},
            "cpu_baseline": cpu,
            "plan": plan,
            "step_bytes": {"weights_per_rank": dec.weight_bytes, "kv_per_rank_per_layer": attn_bytes},
        }
        print(json.dumps(line), flush=True)
    dec.close()
    be.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="llama8b", choices=sorted(CONFIGS))
    ap.add_argument("--cpu-layers", type=int, default=2, help="full-size layers in the CPU sample")
    ap.add_argument("--cpu-vocab", type=int, default=8016, help="lm_head rows in the CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): the named batch at every rank count; weak: batch x ranks")
    ap.add_argument("--attn-chunk-blocks", type=int, default=0, help="KV blocks per attention split (0: default)")
    ap.add_argument("--gemm-splits", type=int, default=0, help="force the split-K count of the layer GEMMs (0: heuristic)")
    ap.add_argument("--gemm-tile", type=int, default=0, help="force the GEMM tile width (0: heuristic)")
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
