"""Writes tests/golden/oracle_cases.npz: small seeded inputs together with the CPU oracle's outputs for them.

    python tests/golden/make_fixtures.py

The reference (Rust) cannot be built or imported here, so these are outputs of the oracle, whose own pins are the
reference's known-answer vectors (reference_vectors.json).  The fixtures serve two checks: the oracle must keep
reproducing them (tests/test_oracle_golden.py, no GPU) and the CUDA path must match them without the oracle
being called (tests/test_quant_gemm_gpu.py, tests/test_paged_gpu.py)."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import oracle as O  # noqa: E402


def cases() -> dict:
    out = {}
    rng = np.random.default_rng(20240229)
    # ---- quantized linear: the rule of the INT8 linear benchmark on a small shape (M 16, K 256, N 48)
    m, k, n = 16, 256, 48
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, n).astype(np.float32)
    wq, ws = O.quantize_i8_per_row(w)
    xq, xs = O.quantize_i8_per_row(x)
    acc = O.gemm_i8_s32(xq, wq)
    out.update(lin_x=x, lin_w=w, lin_bias=bias, lin_wq=wq, lin_ws=ws, lin_xq=xq, lin_xs=xs, lin_acc=acc,
               lin_y=O.epilogue_scaled(acc, xs, True, ws, True, bias=bias, act=O.ACT_NONE),
               lin_y_silu=O.epilogue_scaled(acc, xs, True, ws, True, bias=bias, act=O.ACT_SILU))
    # ---- FP8 E4M3 per-tensor quantisation
    f = (rng.standard_normal(512) * 3.0).astype(np.float32)
    fq, fs = O.quantize_fp8_per_tensor(f)
    out.update(fp8_x=f, fp8_q=fq, fp8_scale=fs)
    # ---- paged decode attention: GQA 4:2, head_dim 128, bf16 pools, block 16, ragged lengths incl. a block edge
    batch, hq, hkv, dh, bs, nblk, mbps = 3, 4, 2, 128, 16, 8, 4
    lens = np.array([37, 16, 5], np.uint32)
    ekv = hkv * dh
    kp = O.f32_to_bf16(rng.standard_normal((nblk * bs, ekv)).astype(np.float32))
    vp = O.f32_to_bf16(rng.standard_normal((nblk * bs, ekv)).astype(np.float32))
    perm = rng.permutation(nblk).astype(np.uint32)
    tables = np.full((batch, mbps), 0xFFFFFFFF, np.uint32)
    at = 0
    for b in range(batch):
        used = -(-int(lens[b]) // bs)
        tables[b, :used] = perm[at:at + used]
        at += used
    q = rng.standard_normal((batch, 1, hq * dh)).astype(np.float32)
    scale = float(1.0 / np.sqrt(dh))
    att = O.paged_attention(q, kp, vp, tables, lens, batch=batch, l_new=1, num_q_heads=hq, num_kv_heads=hkv, head_dim=dh,
                            block_size=bs, num_blocks=nblk, max_blocks_per_seq=mbps, scale=scale, kv_bf16=True)
    out.update(att_q=q, att_k_pool=kp, att_v_pool=vp, att_tables=tables, att_lens=lens, att_out=att,
               att_shape=np.array([batch, hq, hkv, dh, bs, nblk, mbps], np.int64), att_scale=np.float32(scale))
    return out


if __name__ == "__main__":
    path = Path(__file__).with_name("oracle_cases.npz")
    np.savez_compressed(path, **cases())
    print(path, path.stat().st_size, "bytes")
