"""Worker of the CPU (gloo) tensor-parallel test: two ranks, no GPU.

Each rank takes the shard the library's shard plan gives it, computes its part of one decoder layer's
row-parallel projection with the CPU oracle (per-rank activation scale, exact int32 product, dequantised
partial), and the partials are summed with an all-reduce over gloo - the host-side shape of the exchange the
GPU ranks do with NCCL.  Rank 0 checks the sum against the oracle's own tensor-parallel formula and checks
that the shards of all ranks tile every full matrix exactly once."""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def main():
    import torch
    import torch.distributed as dist

    from fandhe_ai_b200.decoder import W_DOWN, W_GATE_UP, W_O, W_QKV, DecoderConfig, shard_plan
    from oracle import oracle as O

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = DecoderConfig(2, 256, 8, 4, 32, 512, 1024, tp_rank=rank, tp_size=world)
    ok = True
    # ---- the shards of all ranks tile each matrix exactly once
    for which in (W_QKV, W_O, W_GATE_UP, W_DOWN):
        plan = shard_plan(cfg, which)
        cover = np.zeros((plan["rows"], plan["cols"]), np.int32)
        for r0, rn in plan["row_ranges"]:
            cover[r0:r0 + rn, plan["col_start"]:plan["col_start"] + plan["col_count"]] += 1
        t = torch.from_numpy(cover)
        dist.all_reduce(t)
        if rank == 0 and not bool((t == 1).all()):
            ok = False
    # ---- row-parallel projection: sum over ranks of acc(quant_r(x_r), W_r) * (s_r * s_w)
    rng = np.random.default_rng(0)
    m, k, n = 8, 512, 256
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wq, ws = O.quantize_i8_per_row(w)
    plan = shard_plan(cfg, W_DOWN)                 # [d_model, d_ff] = [256, 512]: columns are split
    c0, cn = plan["col_start"], plan["col_count"]
    xq, sx = O.quantize_i8_per_row(x[:, c0:c0 + cn])
    part = O.epilogue_scaled(O.gemm_i8_s32(xq, np.ascontiguousarray(wq[:, c0:c0 + cn])), sx, True, ws, True)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    if rank == 0:
        want = None
        for r in range(world):
            kk = k // world
            q_r, s_r = O.quantize_i8_per_row(x[:, r * kk:(r + 1) * kk])
            y = O.epilogue_scaled(O.gemm_i8_s32(q_r, np.ascontiguousarray(wq[:, r * kk:(r + 1) * kk])), s_r, True, ws, True)
            want = y if want is None else (want + y).astype(np.float32)
        if O.compare(t.numpy(), want)[0] != 0:
            ok = False
        # and the sharded result stays within quantisation noise of the unsharded linear
        full = O.linear_w8a8(x, wq, ws)
        if float(np.abs(t.numpy() - full).max()) > 0.05 * float(np.abs(full).max()):
            ok = False
    flag = [ok]
    dist.broadcast_object_list(flag, src=0)
    if rank == 0:
        print("TP_GLOO_OK" if ok else "TP_GLOO_FAIL", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if flag[0] else 1)


if __name__ == "__main__":
    main()
