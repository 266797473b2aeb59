"""The oracle of the block-scale INT8 contract (docs/int8-quant-grade-up-verification-plan.md:177-241 of the
reference) against the figures that document states, and against its own deterministic error bound (no GPU)."""
import numpy as np
import pytest

from oracle import oracle as O


def test_pow2ceil_and_the_floor_of_the_scale():
    assert O.pow2ceil(1.0) == 1.0 and O.pow2ceil(1.0000001) == 2.0 and O.pow2ceil(0.75) == 1.0
    assert O.pow2ceil(3.0) == 4.0 and O.pow2ceil(2.0 ** -20) == 2.0 ** -20
    # amax clamp 1e-4: delta never goes below pow2ceil(1e-4 / 127) = 2^-20 (7.87e-7 lies in (2^-21, 2^-20])
    q, d, bad = O.quantize_i8_block(np.zeros((2, 256), np.float32))
    assert not bad and np.all(d == 2.0 ** -20) and not q.any()
    q, d, bad = O.quantize_i8_block(np.full((1, 128), 3e-5, np.float32))
    assert d[0, 0] == 2.0 ** -20 and q[0, 0] == round(3e-5 * 2 ** 20)


def test_codes_never_clamp_and_round_half_even():
    x = np.zeros((1, 128), np.float32)
    x[0, :6] = [127.0, -127.0, 0.5, 1.5, 2.5, -0.5]         # amax 127 -> delta 1
    q, d, _ = O.quantize_i8_block(x)
    assert d[0, 0] == 1.0 and q[0, :6].tolist() == [127, -127, 0, 2, 2, 0]
    x[0, 0] = 127.5                                          # delta = pow2ceil(127.5 / 127) = 2
    q, d, _ = O.quantize_i8_block(x)
    assert d[0, 0] == 2.0 and q[0, 0] == 64 and q[0, 1] == -64          # 63.75 -> 64, -63.5 -> -64 (ties to even)
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((16, 1000)) * rng.uniform(1e-6, 1e6, (16, 1))).astype(np.float32)
    q, d, bad = O.quantize_i8_block(x)
    assert not bad and np.abs(q.astype(np.int32)).max() <= 127
    assert np.all(np.log2(d) == np.round(np.log2(d)))                   # every scale is a power of two
    back = O.dequantize_i8_block(q, d)
    step = np.repeat(d, 128, axis=1)[:, :1000]
    assert np.all(np.abs(back - x) <= step / 2)                         # |e| <= delta / 2
    qt, dt, _ = O.quantize_i8_block(x, transposed=True)
    assert np.array_equal(qt, q) and np.array_equal(dt, d.T)


def test_known_accumulator_values_of_the_contract():
    # K = 128 block of same-sign worst values: 128 * 127^2 = 2 064 512, exact in f32 (< 2^24)
    a = np.full((1, 128), 127, np.int8)
    one = np.ones((1, 1), np.float32)
    out, bad = O.gemm_i8_block_scaled(a, one, a, one)
    assert not bad and out[0, 0] == 2_064_512.0
    out, _ = O.gemm_i8_block_scaled(a, one, -a, one)
    assert out[0, 0] == -2_064_512.0
    assert (2 ** 31 - 1) // (127 * 127) == 133_144                      # K_safe


def test_final_narrowing_overflow_is_reported():
    # the document's example: K = 512, every element 2^60: each block gives 2^127 (finite), four blocks 2^129
    x = np.full((1, 512), 2.0 ** 60, np.float32)
    q, d, bad = O.quantize_i8_block(x)
    assert not bad and d[0, 0] == 2.0 ** 54 and q[0, 0] == 64
    out, overflow = O.gemm_i8_block_scaled(q, d, q, d.T.copy())
    assert overflow and np.isinf(out[0, 0])
    out, overflow = O.gemm_i8_block_scaled(q[:, :128], d[:, :1], q[:, :128], d[:, :1].T.copy())
    assert not overflow and out[0, 0] == 2.0 ** 127
    _, _, bad = O.quantize_i8_block(np.array([[1.0, np.inf] + [0.0] * 126], np.float32))
    assert bad


def error_bound(a, w, da, dw):
    """E(m, n) = sum_k (|a| dw / 2 + |w| da / 2 + da dw / 4), the deterministic bound of the document."""
    k = a.shape[1]
    da_k = np.repeat(da.astype(np.float64), 128, axis=1)[:, :k]          # [m, k]
    dw_k = np.repeat(dw.astype(np.float64), 128, axis=0)[:k, :]          # [k, n]
    aa, ww = np.abs(a.astype(np.float64)), np.abs(w.astype(np.float64))
    return aa @ dw_k / 2 + da_k @ ww.T / 2 + da_k @ dw_k / 4


@pytest.mark.parametrize("dist", ["uniform", "normal", "heavy", "same_sign", "tiny"])
@pytest.mark.parametrize("k", [128, 512, 4096])
def test_result_stays_inside_the_deterministic_bound(dist, k):
    rng = np.random.default_rng(k)
    m, n = 8, 24
    if dist == "uniform":
        a, w = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (n, k))
    elif dist == "normal":
        a, w = rng.standard_normal((m, k)), rng.standard_normal((n, k)) * 0.02
    elif dist == "heavy":
        a, w = rng.standard_t(2, (m, k)), rng.standard_t(2, (n, k))
    elif dist == "same_sign":
        a, w = np.full((m, k), 0.9), np.full((n, k), 1.7)
    else:
        a, w = rng.uniform(-3e-5, 3e-5, (m, k)), rng.uniform(-8e-5, 8e-5, (n, k))      # the clamp path
    a, w = a.astype(np.float32), w.astype(np.float32)
    aq, da, _ = O.quantize_i8_block(a)
    wq, dw, _ = O.quantize_i8_block(w, transposed=True)
    got, overflow = O.gemm_i8_block_scaled(aq, da, wq, dw)
    assert not overflow
    truth = a.astype(np.float64) @ w.astype(np.float64).T
    bound = error_bound(a, w, da, dw) + 2.0 ** -24 * np.abs(truth) + 1e-300
    assert np.all(np.abs(got.astype(np.float64) - truth) <= bound)
    # and equals the exact rational value it stands for, narrowed once: (sum_b part_b * dout_b) in f64
    nb = da.shape[1]
    acc = np.zeros((m, n), np.float64)
    for b in range(nb):
        part = aq[:, b * 128:(b + 1) * 128].astype(np.int64) @ wq[:, b * 128:(b + 1) * 128].astype(np.int64).T
        acc += (part.astype(np.float32) * (da[:, b:b + 1] * dw[b:b + 1, :])).astype(np.float64)
    assert np.array_equal(got, acc.astype(np.float32))
