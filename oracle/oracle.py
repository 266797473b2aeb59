"""numpy-facing wrapper of the CPU oracle (oracle/oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, `__graft_entry__.smoke()` and the CPU-baseline
legs of bench.py, as the checker and the timed CPU baseline.  The product never imports it.
Parity status is stated piece by piece in the header of oracle.c ("parity unpinned" for the
quantisation rules, GQA/bf16 attention, RoPE and the decoder wiring, which the reference lacks).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = HERE / "oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "-B", "liboracle.so"], check=True, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(str(LIB))
        _lib.orc_f32_to_bf16.restype = C.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [C.c_float]
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_composite_close.restype = C.c_int
        _lib.orc_composite_close.argtypes = [C.c_float, C.c_float]
        _lib.orc_compare.restype = C.c_int64
        _lib.orc_f32_to_e4m3.restype = C.c_uint8
        _lib.orc_f32_to_e4m3.argtypes = [C.c_float]
        _lib.orc_e4m3_to_f32.restype = C.c_float
        _lib.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        _lib.orc_sigmoid_stable.restype = C.c_float
        _lib.orc_sigmoid_stable.argtypes = [C.c_float]
        _lib.orc_silu.restype = C.c_float
        _lib.orc_silu.argtypes = [C.c_float]
        _lib.orc_greedy_argmax.restype = C.c_int64
        _lib.orc_paged_kv_append.restype = C.c_int
        _lib.orc_paged_attention.restype = C.c_int
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---------------------------------------------------------------- scalars / conversions
def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(int(n)))


def f32_to_bf16(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16_array(_p(x), C.c_int64(x.size), _p(out))
    return out


def bf16_to_f32(x) -> np.ndarray:
    x = _c(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32_array(_p(x), C.c_int64(x.size), _p(out))
    return out


def composite_close(actual: float, reference: float) -> bool:
    return bool(lib().orc_composite_close(float(np.float32(actual)), float(np.float32(reference))))


def compare(actual, reference):
    """Returns (fail_count, max_abs, max_rel) under the composite judge."""
    a = _c(actual, np.float32).ravel()
    r = _c(reference, np.float32).ravel()
    assert a.size == r.size
    ma, mr = C.c_double(), C.c_double()
    fails = lib().orc_compare(_p(a), _p(r), C.c_int64(a.size), C.byref(ma), C.byref(mr))
    return int(fails), ma.value, mr.value


def e4m3_to_f32(q) -> np.ndarray:
    q = _c(q, np.uint8)
    out = np.empty(q.shape, np.float32)
    lib().orc_e4m3_to_f32_array(_p(q), C.c_int64(q.size), _p(out))
    return out


def f32_to_e4m3_scalar(x: float) -> int:
    return int(lib().orc_f32_to_e4m3(float(np.float32(x))))


def sigmoid_stable(x: float) -> float:
    return float(lib().orc_sigmoid_stable(float(np.float32(x))))


def silu(x: float) -> float:
    return float(lib().orc_silu(float(np.float32(x))))


# ---------------------------------------------------------------- GEMM contracts
def matmul_reference_fma(a, b) -> np.ndarray:
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.zeros((m, n), np.float32)
    lib().orc_matmul_reference_fma(_p(a), _p(b), _p(c), C.c_int64(m), C.c_int64(n), C.c_int64(k))
    return c


def gemm_i8_s32(a, w) -> np.ndarray:
    a = _c(a, np.int8)
    w = _c(w, np.int8)
    m, k = a.shape
    n, k2 = w.shape
    assert k == k2
    acc = np.empty((m, n), np.int32)
    lib().orc_gemm_i8_s32(_p(a), _p(w), C.c_int64(m), C.c_int64(n), C.c_int64(k), _p(acc))
    return acc


def gemm_fp8_f32(a, b) -> np.ndarray:
    a = _c(a, np.uint8)
    b = _c(b, np.uint8)
    m, k = a.shape
    n, k2 = b.shape
    assert k == k2
    acc = np.empty((m, n), np.float32)
    lib().orc_gemm_fp8_f32(_p(a), _p(b), C.c_int64(m), C.c_int64(n), C.c_int64(k), _p(acc))
    return acc


# ---------------------------------------------------------------- quantisers
def quantize_i8_per_row(x):
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.int8)
    s = np.empty((rows,), np.float32)
    lib().orc_quantize_i8_per_row(_p(x), C.c_int64(rows), C.c_int64(cols), _p(q), _p(s))
    return q, s


def dequantize_i8_per_row(q, s) -> np.ndarray:
    q = _c(q, np.int8)
    s = _c(s, np.float32)
    rows, cols = q.shape
    x = np.empty((rows, cols), np.float32)
    lib().orc_dequantize_i8_per_row(_p(q), _p(s), C.c_int64(rows), C.c_int64(cols), _p(x))
    return x


def quantize_fp8_per_tensor(x):
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    s = np.empty((1,), np.float32)
    lib().orc_quantize_fp8_per_tensor(_p(x), C.c_int64(x.size), _p(q), _p(s))
    return q, s


def quantize_fp8_per_row(x):
    """E4M3 codes [rows, cols] (uint8) and one scale per row (amax / 448): the FP8 decoder's quantiser."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.uint8)
    s = np.empty((rows,), np.float32)
    lib().orc_quantize_fp8_per_row(_p(x), C.c_int64(rows), C.c_int64(cols), _p(q), _p(s))
    return q, s


ACT_NONE, ACT_RELU, ACT_SILU, ACT_SILU_GATE = 0, 1, 2, 3


def epilogue_scaled(acc, a_scale, a_per_row, b_scale, b_per_col, bias=None, act=ACT_NONE, residual=None,
                    out_bf16=False) -> np.ndarray:
    """y = act(fma(acc, sa*sb, bias)) (+ residual) with explicit per-row / per-column scale flags
    (the arguments of b200_gemm_q8_scaled).  acc: int32 or f32 [m, n]."""
    acc = np.ascontiguousarray(acc)
    m, n = acc.shape
    a_scale = _c(a_scale, np.float32).ravel()
    b_scale = _c(b_scale, np.float32).ravel()
    n_out = n // 2 if act == ACT_SILU_GATE else n
    out = np.empty((m, n_out), np.uint16 if out_bf16 else np.float32)
    bias_c = _c(bias, np.float32) if bias is not None else None
    res_c = _c(residual, np.float32) if residual is not None else None
    lib().orc_epilogue(_p(acc), C.c_int(int(acc.dtype == np.int32)), C.c_int64(m), C.c_int64(n), _p(a_scale),
                       C.c_int(int(a_per_row)), _p(b_scale), C.c_int(int(b_per_col)),
                       _p(bias_c) if bias_c is not None else None, C.c_int(act),
                       _p(res_c) if res_c is not None else None, _p(out), C.c_int(int(out_bf16)))
    return out


def linear_w8a8(x, w_q, w_scale, bias=None, act=ACT_NONE, residual=None) -> np.ndarray:
    """f32 activations -> per-token int8 -> exact int32 GEMM -> dequant epilogue (f32)."""
    xq, sx = quantize_i8_per_row(x)
    acc = gemm_i8_s32(xq, w_q)
    return epilogue_scaled(acc, sx, True, w_scale, True, bias, act, residual)


# ---------------------------------------------------------------- decoder glue
def rmsnorm(x, w, eps: float) -> np.ndarray:
    x = _c(x, np.float32)
    rows, hidden = x.shape
    out = np.empty_like(x)
    w_c = _c(w, np.float32) if w is not None else None
    lib().orc_rmsnorm(_p(x), _p(w_c) if w_c is not None else None, C.c_float(eps), C.c_int64(rows), C.c_int64(hidden),
                      _p(out))
    return out


def rope_table(max_pos: int, head_dim: int, theta: float = 10000.0):
    cos_t = np.empty((max_pos, head_dim // 2), np.float32)
    sin_t = np.empty((max_pos, head_dim // 2), np.float32)
    lib().orc_rope_table(C.c_int64(max_pos), C.c_int64(head_dim), C.c_double(theta), _p(cos_t), _p(sin_t))
    return cos_t, sin_t


def rope_apply(x, heads: int, head_dim: int, cos_row, sin_row) -> np.ndarray:
    """x: [heads * head_dim] one token; returns the rotated copy."""
    out = _c(x, np.float32).copy()
    cos_row = _c(cos_row, np.float32)
    sin_row = _c(sin_row, np.float32)
    lib().orc_rope_apply(_p(out), C.c_int64(heads), C.c_int64(head_dim), _p(cos_row), _p(sin_row))
    return out


def greedy_argmax(row) -> int:
    row = _c(row, np.float32).ravel()
    return int(lib().orc_greedy_argmax(_p(row), C.c_int64(row.size)))


# ---------------------------------------------------------------- paged KV
def paged_kv_append(k_new, v_new, k_pool, v_pool, slots, e: int, kv_bf16: bool) -> None:
    """In place on k_pool / v_pool (uint16 when kv_bf16 else float32), shaped [pool_rows * e] or any
    contiguous shape with that many elements."""
    k_new = _c(k_new, np.float32)
    v_new = _c(v_new, np.float32)
    slots = _c(slots, np.uint32)
    assert k_pool.flags.c_contiguous and v_pool.flags.c_contiguous
    assert k_pool.dtype == (np.uint16 if kv_bf16 else np.float32)
    pool_rows = k_pool.size // e
    rc = lib().orc_paged_kv_append(_p(k_new), _p(v_new), _p(k_pool), _p(v_pool), _p(slots), C.c_int64(slots.size),
                                   C.c_int64(e), C.c_int64(pool_rows), C.c_int(int(kv_bf16)))
    if rc != 0:
        raise ValueError("paged_kv_append: slot out of range")


def paged_attention(q, k_pool, v_pool, block_tables, seq_lens, *, batch: int, l_new: int, num_q_heads: int,
                    num_kv_heads: int, head_dim: int, block_size: int, num_blocks: int, max_blocks_per_seq: int,
                    scale: float, kv_bf16: bool) -> np.ndarray:
    q = _c(q, np.float32)
    block_tables = _c(block_tables, np.uint32)
    seq_lens = _c(seq_lens, np.uint32)
    out = np.zeros((batch, l_new, num_q_heads * head_dim), np.float32)
    rc = lib().orc_paged_attention(_p(q), _p(k_pool), _p(v_pool), _p(block_tables), _p(seq_lens), C.c_int64(batch),
                                   C.c_int64(l_new), C.c_int64(num_q_heads), C.c_int64(num_kv_heads),
                                   C.c_int64(head_dim), C.c_int64(block_size), C.c_int64(num_blocks),
                                   C.c_int64(max_blocks_per_seq), C.c_float(scale), C.c_int(int(kv_bf16)), _p(out))
    if rc != 0:
        raise ValueError(f"paged_attention: invalid input ({rc})")
    return out


# ---------------------------------------------------------------- kernel-order restatements
# The CUDA decoder sums in its own fixed order and uses its own exponential; these functions round exactly
# as those kernels do (see the block comment in oracle.c).  Each is checked against its sequential
# counterpart above within the composite tolerance in tests/test_oracle_golden.py.
def exp_det(x) -> np.ndarray:
    x = _c(x, np.float32)
    out = np.empty_like(x)
    lib().orc_exp_det_array(_p(x), C.c_int64(x.size), _p(out))
    return out


def silu_det(x: float) -> float:
    f = lib().orc_silu_det
    f.restype, f.argtypes = C.c_float, [C.c_float]
    return float(f(C.c_float(x)))


def epilogue_det(acc, a_scale, b_scale, act=ACT_NONE) -> np.ndarray:
    """int32 accumulators [m, n] -> f32 with per-row / per-column scales, no bias; SiLU uses exp_det."""
    acc = _c(acc, np.int32)
    m, n = acc.shape
    n_out = n // 2 if act == ACT_SILU_GATE else n
    out = np.empty((m, n_out), np.float32)
    lib().orc_epilogue_det(_p(acc), C.c_int64(m), C.c_int64(n), _p(_c(a_scale, np.float32)), _p(_c(b_scale, np.float32)),
                           C.c_int(act), _p(out))
    return out


def rmsnorm_kernel_order(x, w, eps: float, mode: int, threads: int, vpt_or_cl: int) -> np.ndarray:
    """mode 0: one wide CTA per row (threads, groups of four per thread); mode 1: `vpt_or_cl` chunks of 256 threads."""
    x = _c(x, np.float32)
    rows, hidden = x.shape
    out = np.empty_like(x)
    lib().orc_rmsnorm_kernel_order(_p(x), _p(_c(w, np.float32)), C.c_float(eps), C.c_int64(rows), C.c_int64(hidden),
                                   C.c_int(mode), C.c_int(threads), C.c_int(vpt_or_cl), _p(out))
    return out


def paged_attention_kernel_order(q, k_pool, v_pool, block_tables, seq_lens, *, batch: int, l_new: int, num_q_heads: int,
                                 num_kv_heads: int, head_dim: int, block_size: int, num_blocks: int,
                                 max_blocks_per_seq: int, scale: float, kv_bf16: bool) -> np.ndarray:
    q = _c(q, np.float32)
    block_tables = _c(block_tables, np.uint32)
    seq_lens = _c(seq_lens, np.uint32)
    out = np.zeros((batch, l_new, num_q_heads * head_dim), np.float32)
    f = lib().orc_paged_attention_kernel_order
    f.restype = C.c_int
    rc = f(_p(q), _p(k_pool), _p(v_pool), _p(block_tables), _p(seq_lens), C.c_int64(batch), C.c_int64(l_new),
           C.c_int64(num_q_heads), C.c_int64(num_kv_heads), C.c_int64(head_dim), C.c_int64(block_size),
           C.c_int64(num_blocks), C.c_int64(max_blocks_per_seq), C.c_float(scale), C.c_int(int(kv_bf16)), _p(out))
    if rc != 0:
        raise ValueError(f"paged_attention_kernel_order: invalid input ({rc})")
    return out


def gemm_i8_s32_blas(a, w_float) -> np.ndarray:
    """The int32 accumulators of gemm_i8_s32 through a floating-point BLAS product, for the long decoder runs.
    `w_float` is the weight [n, k] converted once with int8_weight_for_blas().  Every product is an integer of
    at most 127 * 128 and every partial sum an integer below k * 2^14, so the f32 product is exact for
    k <= 1024 (sums < 2^24) and the f64 product for any k here (sums < 2^53), whatever order BLAS adds in."""
    a = np.asarray(a)
    acc = a.astype(w_float.dtype) @ w_float.T
    return acc.astype(np.int64).astype(np.int32)


def int8_weight_for_blas(w_q) -> np.ndarray:
    w_q = np.asarray(w_q)
    return np.ascontiguousarray(w_q.astype(np.float32 if w_q.shape[1] <= 1024 else np.float64))


# ---------------------------------------------------------------- block-scale INT8 contract
def pow2ceil(x: float) -> float:
    f = lib().orc_pow2ceil
    f.restype, f.argtypes = C.c_float, [C.c_float]
    return float(f(C.c_float(x)))


def quantize_i8_block(x, transposed: bool = False):
    """(q int8 [rows, cols], delta f32 [rows, nb] or [nb, rows], saw_non_finite)."""
    x = _c(x, np.float32)
    rows, cols = x.shape
    nb = -(-cols // 128)
    q = np.empty((rows, cols), np.int8)
    d = np.empty((nb, rows) if transposed else (rows, nb), np.float32)
    f = lib().orc_quantize_i8_block
    f.restype = C.c_int
    bad = f(_p(x), C.c_int64(rows), C.c_int64(cols), C.c_int(int(transposed)), _p(q), _p(d))
    return q, d, bool(bad)


def dequantize_i8_block(q, delta, transposed: bool = False) -> np.ndarray:
    q = _c(q, np.int8)
    rows, cols = q.shape
    out = np.empty((rows, cols), np.float32)
    lib().orc_dequantize_i8_block(_p(q), _p(_c(delta, np.float32)), C.c_int64(rows), C.c_int64(cols), C.c_int(int(transposed)),
                                  _p(out))
    return out


def gemm_i8_block_scaled(a, da, w, dw):
    """a [m, k] int8, da [m, nb]; w [n, k] int8, dw [nb, n] -> (out f32 [m, n], overflowed_at_narrowing)."""
    a, w = _c(a, np.int8), _c(w, np.int8)
    m, k = a.shape
    n = w.shape[0]
    out = np.empty((m, n), np.float32)
    f = lib().orc_gemm_i8_block_scaled
    f.restype = C.c_int
    bad = f(_p(a), _p(_c(da, np.float32)), _p(w), _p(_c(dw, np.float32)), C.c_int64(m), C.c_int64(n), C.c_int64(k), _p(out))
    return out, bool(bad)


# ---- sampling weights of generate() (crates/autodiff/src/generate/mod.rs:331-369, 433-455) ----------------------
SAMPLE_GREEDY, SAMPLE_TEMPERATURE, SAMPLE_TOP_K = 0, 1, 2


def top_k_indices(row, k: int):
    """The k largest values by value descending, index ascending (mod.rs:359-369)."""
    row = np.asarray(row, np.float32)
    return sorted(range(len(row)), key=lambda i: (-float(row[i]), i))[:k]


def softmax_weights_f64(row, temperature: float) -> np.ndarray:
    """exp((x - max) / t) in f64, summed in index order, divided, narrowed to f32 (mod.rs:347-355)."""
    import math

    x = np.asarray(row, np.float32).astype(np.float64)
    mx = float(x.max())
    t = float(np.float32(temperature))
    e = [math.exp((float(v) - mx) / t) for v in x]
    total = 0.0
    for v in e:
        total += v
    return np.array([v / total for v in e], np.float64).astype(np.float32)


def sampling_weights(row, strategy: int, k: int = 0, temperature: float = 1.0) -> np.ndarray:
    """sampling_weights_f32 (mod.rs:433-455) for one row of finite logits."""
    row = np.asarray(row, np.float32)
    if strategy == SAMPLE_TEMPERATURE:
        return softmax_weights_f64(row, temperature)
    w = np.zeros(len(row), np.float32)
    if strategy == SAMPLE_GREEDY:
        w[greedy_argmax(row)] = 1.0
        return w
    top = top_k_indices(row, k)
    w[top] = softmax_weights_f64(row[top], temperature)
    return w
