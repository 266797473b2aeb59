"""Kernel-level benchmarks of the two hot kernels, through the C ABI, on one GPU:

    python -m fandhe_ai_b200.bench_kernels gemm        # FP8 / INT8 GEMM sweep (T(FL)OPS, fraction of peak)
    python -m fandhe_ai_b200.bench_kernels attention   # paged decode attention at the benchmark shape (GB/s)

Operands are synthetic and resident on the device; each measurement is CUDA-event time on the context's
stream over `iters` launches after `warmup` launches, cycling over several operand sets so that the inputs
of consecutive launches do not sit in L2.  One JSON line per shape.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from fandhe_ai_b200 import ACT_NONE, ACT_SILU_GATE, BF16, FP8_E4M3, I8, Backend  # noqa: E402
from fandhe_ai_b200 import paged_kv as P  # noqa: E402


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def bench_gemm(be: Backend, op: int, m: int, n: int, k: int, act: int, iters: int, warmup: int, tile: int, splits: int):
    rng = np.random.default_rng(0)
    # enough operand sets to exceed the L2 (126 MB) between reuses
    per_set = m * k + n * k
    sets = max(2, min(8, int(300e6 // per_set) + 1))
    a_bufs, w_bufs = [], []
    for s in range(sets):
        a_bufs.append(be.upload(rng.integers(-100 if op == I8 else 0, 100 if op == I8 else 120, (m, k)).astype(np.int8 if op == I8 else np.uint8)))
        w_bufs.append(be.upload(rng.integers(-100 if op == I8 else 0, 100 if op == I8 else 120, (n, k)).astype(np.int8 if op == I8 else np.uint8)))
    sa = be.upload(np.full(m, 0.01, np.float32))
    sw = be.upload(np.full(n, 0.01, np.float32))
    be.gemm_tuning(tile, splits)
    from fandhe_ai_b200._lib import check, lib

    n_out = n // 2 if act == ACT_SILU_GATE else n
    out = be.alloc_zeroed((m, n_out), np.uint16)

    def one(i):      # the output buffer is allocated once, outside the timed region
        check(lib().b200_gemm_q8_scaled(be._ctx, op, a_bufs[i % sets].handle, 0, sa.handle, 0, 1, w_bufs[i % sets].handle, 0,
                                        sw.handle, 0, 1, None, 0, act, None, 0, m, n, k, BF16, out.handle, 0))

    for i in range(warmup):
        one(i)
    be.synchronize_device()
    be.timer_start()
    for i in range(iters):
        one(i)
    ms = be.timer_stop() / iters
    for o in [out] + a_bufs + w_bufs + [sa, sw]:
        o.release()
    be.gemm_tuning(0, 0)
    return ms


def run_gemm(args):
    be = Backend(0)
    shapes = []
    for nk in (4096, 8192, 14336):
        for m in (1, 16, 128, 1024, 4096, 8192):
            shapes.append((m, nk, nk, ACT_NONE))
    shapes.append((1024, 2 * 14336, 4096, ACT_SILU_GATE))
    shapes.append((8192, 2 * 14336, 4096, ACT_SILU_GATE))
    if args.shape:
        m, n, k = (int(v) for v in args.shape.split(","))
        shapes = [(m, n, k, ACT_SILU_GATE if args.gate else ACT_NONE)]
    elif args.quick:
        shapes = [(128, 4096, 4096, ACT_NONE), (4096, 4096, 4096, ACT_NONE), (8192, 8192, 8192, ACT_NONE)]
    for op, name in ((FP8_E4M3, "fp8_e4m3"), (I8, "int8")):
        if args.operands and not name.startswith(args.operands):
            continue
        for m, n, k, act in shapes:
            print(json.dumps(measure_gemm(be, op, m, n, k, act, args.iters, args.warmup, args.tile, args.splits)), flush=True)
    be.close()


def measure_attention_config3(be: Backend, iters: int, warmup: int, chunk_blocks: int = 0, host_call: bool = True) -> dict:
    """Config 3: batch 64, 32 query / 8 KV heads, head_dim 128, bf16 KV, block 16, contexts U[512, 8192], block
    tables = consecutive slices of a seeded permutation of a 200k-block pool."""
    hbm, _, kind = peaks()
    rng = np.random.default_rng(0)
    batch, hq, hkv, dh, bs, nblk = 64, 32, 8, 128, 16, 200_000
    ctx = rng.integers(512, 8193, batch).astype(np.uint32)
    mbps = 512
    perm = rng.permutation(nblk).astype(np.uint32)
    tables = np.full((batch, mbps), P.SENTINEL, np.uint32)
    at = 0
    for b in range(batch):
        used = -(-int(ctx[b]) // bs)
        tables[b, :used] = perm[at:at + used]
        at += used
    layout = P.PagedKvLayout(nblk, bs, hkv * dh, BF16)
    a = P.PagedAttentionArgs(layout, batch, 1, hq, mbps, float(1.0 / np.sqrt(dh)), hkv)
    # pools: 200k blocks x 16 x 1024 x 2 B = 6.5 GB each; fill with a tiled random pattern
    tile = (rng.standard_normal(1 << 22).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    k_pool = be.alloc_zeroed((nblk * bs, hkv * dh), np.uint16)
    v_pool = be.alloc_zeroed((nblk * bs, hkv * dh), np.uint16)
    total = nblk * bs * hkv * dh
    for off in range(0, total, tile.size):
        nn = min(tile.size, total - off)
        be.upload_into(tile[:nn], k_pool, off * 2)
        be.upload_into(tile[:nn], v_pool, off * 2)
    q = be.upload(rng.standard_normal((batch, 1, hq * dh)).astype(np.float32))
    out = be.alloc_zeroed((batch, 1, hq * dh), np.float32)
    tdev, sdev = be.upload(tables), be.upload(ctx)
    if chunk_blocks:
        P.paged_attention_tuning(be, chunk_blocks)
    algo = int(ctx.astype(np.int64).sum()) * hkv * dh * 2 * 2 + 2 * batch * hq * dh * 4 + int(sum(-(-int(c) // bs) for c in ctx)) * 4
    for _ in range(warmup):
        P.paged_attention_forward_resident(be, q, k_pool, v_pool, tdev, sdev, int(ctx.max()), a, out)
    be.synchronize_device()
    be.timer_start()
    for _ in range(iters):
        P.paged_attention_forward_resident(be, q, k_pool, v_pool, tdev, sdev, int(ctx.max()), a, out)
    ms = be.timer_stop() / iters
    gbs = algo / (ms * 1e-3) / 1e9
    res = {"kernel": "paged_attention_decode (+combine)", "batch": batch, "sum_ctx": int(ctx.sum()),
           "algorithmic_bytes": algo, "ms": round(ms, 5), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4),
           "frac_of_8000_nominal": round(gbs / 8000.0, 4), "peak_kind": kind,
           "note": "the KV read per launch (1.1 GB) is far above the L2 size"}
    if host_call:
        # through the reference-shaped call: host block tables and seq_lens validated and uploaded per call
        import time
        be.synchronize_device()
        t0 = time.perf_counter()
        for _ in range(iters):
            P.paged_attention_forward(be, q, k_pool, v_pool, tables, ctx, a, out)
        be.synchronize_device()
        res["ms_host_tables_call"] = round((time.perf_counter() - t0) * 1e3 / iters, 5)
    for b_ in (k_pool, v_pool, q, out, tdev, sdev):
        b_.release()
    if chunk_blocks:
        P.paged_attention_tuning(be, 0)
    return res


def measure_gemm(be: Backend, op: int, m: int, n: int, k: int, act: int, iters: int, warmup: int, tile: int = 0,
                 splits: int = 0) -> dict:
    """One GEMM shape: T(FL)OPS and the two fractions (of 2 x the measured bf16 burst peak, of the 4500 nominal)."""
    hbm, bf16, kind = peaks()
    ms = bench_gemm(be, op, m, n, k, act, iters, warmup, tile, splits)
    tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    n_out = n // 2 if act == ACT_SILU_GATE else n
    gbs = (m * k + n * k + 2 * m * n_out) / (ms * 1e-3) / 1e9
    return {"kernel": "gemm_tc5", "operands": "int8" if op == I8 else "fp8_e4m3", "m": m, "n": n, "k": k,
            "epilogue": "silu_gate" if act == ACT_SILU_GATE else "dequant", "out": "bf16", "ms": round(ms, 5),
            "tops": round(tops, 1), "frac_of_2x_bf16_peak": round(tops / (2 * bf16), 4),
            "frac_of_4500_nominal": round(tops / 4500, 4), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / hbm, 4),
            "peak_kind": kind}


def run_attention(args):
    be = Backend(0)
    print(json.dumps(measure_attention_config3(be, args.iters, args.warmup, args.chunk_blocks)), flush=True)
    be.close()


def run_gemm_phases(args):
    """Where the time of a decode-shaped GEMM launch goes: the M = 1 / 16 / 128 shapes of the weight sweep (or --shape),
    raw accumulators and the dequantising epilogue, %globaltimer stamps of the launch's first CTA."""
    be = Backend(0)
    if args.tile or args.splits:
        be.gemm_tuning(args.tile, args.splits)
    if args.shape:
        shapes = [tuple(int(x) for x in args.shape.split(","))]
    else:
        shapes = [(m, n, n) for n in (4096, 8192, 14336) for m in (1, 16, 128)]
    for m, n, k in shapes:
        for fused in (False, True):
            try:
                print(json.dumps(be.gemm_phase_stamps(m, n, k, fused=fused, iters=max(args.iters, 20))), flush=True)
            except Exception as exc:            # a shape without that form: say so and go on
                print(json.dumps({"m": m, "n": n, "k": k, "fused": fused, "skipped": str(exc)[:120]}), flush=True)
    be.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention", "gemm-phases"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--shape", default="", help="m,n,k: only this GEMM shape")
    ap.add_argument("--gate", action="store_true", help="with --shape: the SiLU-gated epilogue (n counts gate + up rows)")
    ap.add_argument("--operands", default="", help="fp8 or int8: only this operand type")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--chunk-blocks", type=int, default=0)
    args = ap.parse_args()
    if args.what == "gemm":
        run_gemm(args)
    elif args.what == "gemm-phases":
        run_gemm_phases(args)
    else:
        run_attention(args)


if __name__ == "__main__":
    main()
