"""GPU parity of the block-scale INT8 contract (the variant the reference proposes for its QuantOps backend,
docs/int8-quant-grade-up-verification-plan.md:177-241): quantised codes, scales and GEMM results are pure functions
of the inputs, so the acceptance rule is bit-exact (fail_count == 0), through the C ABI."""
import numpy as np
import pytest

from fandhe_ai_b200 import BackendError
from fandhe_ai_b200._lib import check, lib
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def inputs(dist, m, n, k, seed):
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        a, w = rng.uniform(-1, 1, (m, k)), rng.uniform(-1, 1, (n, k))
    elif dist == "normal":
        a, w = rng.standard_normal((m, k)), rng.standard_normal((n, k)) * 0.02
    elif dist == "heavy":
        a, w = rng.standard_t(2, (m, k)), rng.standard_t(2, (n, k))
    elif dist == "same_sign":
        a, w = np.full((m, k), 0.9), np.full((n, k), 1.7)
    else:
        a, w = rng.uniform(-3e-5, 3e-5, (m, k)), rng.uniform(-8e-5, 8e-5, (n, k))      # amax below the 1e-4 clamp
    return a.astype(np.float32), w.astype(np.float32)


@pytest.mark.parametrize("rows,cols", [(128, 4096), (3, 128), (5, 144), (33, 1000), (1, 16)])
def test_block_quantiser_is_byte_identical(be, rows, cols):
    x, _ = inputs("heavy", rows, 1, cols, rows + cols)
    x[0, 0] = 0.0
    for transposed in (False, True):
        q, d = be.quantize_i8_block(be.upload(x), rows, cols, scales_block_major=transposed)
        q_ref, d_ref, bad = O.quantize_i8_block(x, transposed)
        assert not bad
        assert np.array_equal(d.numpy(), d_ref) and np.array_equal(q.numpy(), q_ref)
        back = be.dequantize_i8_block(q, d, rows, cols, scales_block_major=transposed).numpy()
        assert np.array_equal(back, O.dequantize_i8_block(q_ref, d_ref, transposed))
    be.quant_check()


@pytest.mark.parametrize("dist", ["uniform", "normal", "heavy", "same_sign", "tiny"])
@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (128, 256, 512), (300, 208, 4096), (64, 64, 16384), (1, 16, 144)])
def test_block_scaled_gemm_is_bit_exact(be, dist, m, n, k):
    a, w = inputs(dist, m, n, k, m + n + k)
    aq_d, da_d = be.quantize_i8_block(be.upload(a), m, k)
    wq_d, dw_d = be.quantize_i8_block(be.upload(w), n, k, scales_block_major=True)
    aq, da, _ = O.quantize_i8_block(a)
    wq, dw, _ = O.quantize_i8_block(w, transposed=True)
    assert np.array_equal(aq_d.numpy(), aq) and np.array_equal(da_d.numpy(), da)
    assert np.array_equal(wq_d.numpy(), wq) and np.array_equal(dw_d.numpy(), dw)
    got = be.gemm_i8_block_scaled(aq_d, da_d, wq_d, dw_d, m, n, k).numpy()
    want, overflow = O.gemm_i8_block_scaled(aq, da, wq, dw)
    assert not overflow
    fail_count = int((got.view(np.uint32) != want.view(np.uint32)).sum())
    assert fail_count == 0, (fail_count, float(np.abs(got - want).max()))
    be.quant_check()


def test_k128_worst_case_and_the_k_safe_guard(be):
    a = np.full((128, 128), 127, np.int8)
    one_a, one_w = np.ones((128, 1), np.float32), np.ones((1, 128), np.float32)
    out = be.gemm_i8_block_scaled(be.upload(a), be.upload(one_a), be.upload(a), be.upload(one_w), 128, 128, 128).numpy()
    assert np.all(out == 2_064_512.0)                       # 128 * 127^2, exact in f32
    x = be.upload(np.zeros((2, 256), np.float32))
    with pytest.raises(BackendError) as e:                  # a block longer than K_safe could wrap the s32 accumulator
        be.quantize_i8_block(x, 2, 256, block_len=133_145)
    assert e.value.kind == "InvalidArgument" and "K_safe" in e.value.message
    with pytest.raises(BackendError) as e:
        be.gemm_i8_block_scaled(be.upload(a), be.upload(one_a), be.upload(a), be.upload(one_w), 128, 128, 128, block_len=133_145)
    assert e.value.kind == "InvalidArgument" and "K_safe" in e.value.message
    with pytest.raises(BackendError) as e:                  # K_safe itself is inside the contract but not implemented
        be.quantize_i8_block(x, 2, 256, block_len=133_144)
    assert e.value.kind == "Unsupported"
    assert not be.poisoned


def test_non_finite_inputs_and_narrowing_overflow_are_typed_errors(be):
    be.quant_check()
    x = np.ones((2, 256), np.float32)
    x[1, 130] = np.nan
    q, d = be.quantize_i8_block(be.upload(x), 2, 256)
    with pytest.raises(BackendError) as e:
        be.quant_check()
    assert e.value.kind == "InvalidArgument" and "not finite" in e.value.message and not be.poisoned
    assert not q.numpy()[1, 128:].any() and q.numpy()[0].all()           # only the affected block is zeroed
    be.quant_check()                                                      # reported once, then clear
    # the document's example: K = 512, every element 2^60 -> blocks of 2^127 (finite), their f64 sum 2^129 -> inf
    big = np.full((16, 512), 2.0 ** 60, np.float32)
    bq, bd = be.quantize_i8_block(be.upload(big), 16, 512)
    wq, wd = be.quantize_i8_block(be.upload(big), 16, 512, scales_block_major=True)
    out = be.gemm_i8_block_scaled(bq, bd, wq, wd, 16, 16, 512).numpy()
    with pytest.raises(BackendError) as e:
        be.quant_check()
    assert e.value.kind == "InvalidArgument" and "overflowed" in e.value.message and not be.poisoned
    assert np.all(np.isinf(out))
    be.quant_check()
