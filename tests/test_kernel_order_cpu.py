"""The kernel-order restatements of the oracle against their sequential counterparts (no GPU).

The CUDA decoder sums in a fixed order of its own and uses its own exponential; oracle.c restates that order
so that greedy token ids can be compared bit for bit with the device.  A restatement is only acceptable as a
checker if it stays within the composite tolerance (rel < 1e-3 or abs < 1e-5,
crates/tensor-core/src/tolerance.rs:15-37) of the sequential definition on the same inputs: that is what
this file shows, piece by piece and for a whole decoder."""
import numpy as np
import pytest

from oracle import oracle as O
from oracle.decoder_ref import DecoderRef, make_weights, pick_cluster, wide_shape


def test_exp_det_is_within_two_ulp_of_the_exact_exponential_and_handles_the_ends():
    x = np.concatenate([np.linspace(-103.9, 88.7, 400001), [0.0, -0.0, 1e-30, -1e-30]]).astype(np.float32)
    y = O.exp_det(x).astype(np.float64)
    ref = np.exp(x.astype(np.float64))
    normal = ref > 1.2e-38
    assert np.max(np.abs(y[normal] - ref[normal]) / ref[normal]) < 2 * 2.0 ** -23
    assert np.max(np.abs(y[~normal] - ref[~normal])) < 2 * 1.5e-45         # denormal results: one denormal step
    assert O.exp_det(np.array([0.0], np.float32))[0] == 1.0
    ends = O.exp_det(np.array([-np.inf, -200.0, 89.0, np.inf], np.float32))
    assert ends[0] == 0.0 and ends[1] == 0.0 and np.isinf(ends[2]) and np.isinf(ends[3])
    assert np.isnan(O.exp_det(np.array([np.nan], np.float32))[0])
    # against libm's expf, the exponential of the sequential oracle
    lib = O.lib()
    got = O.exp_det(x[::97])
    want = np.array([np.exp(np.float32(v)) for v in x[::97]], np.float32)
    assert O.compare(got, want)[0] == 0


def test_silu_det_against_the_two_branch_silu():
    xs = np.linspace(-30, 30, 6001).astype(np.float32)
    got = np.array([O.silu_det(float(v)) for v in xs], np.float32)
    want = np.array([O.silu(float(v)) for v in xs], np.float32)
    assert O.compare(got, want)[0] == 0
    acc = np.random.default_rng(0).integers(-2_000_000, 2_000_000, (9, 64), dtype=np.int32)
    sa = np.random.default_rng(1).uniform(1e-3, 2e-3, 9).astype(np.float32)
    sb = np.random.default_rng(2).uniform(1e-3, 2e-3, 64).astype(np.float32)
    for act in (O.ACT_NONE, O.ACT_RELU, O.ACT_SILU, O.ACT_SILU_GATE):
        assert O.compare(O.epilogue_det(acc, sa, sb, act), O.epilogue_scaled(acc, sa, True, sb, True, act=act))[0] == 0
    assert np.array_equal(O.epilogue_det(acc, sa, sb, O.ACT_NONE), O.epilogue_scaled(acc, sa, True, sb, True))


@pytest.mark.parametrize("hidden,rows", [(768, 32), (512, 4), (4096, 128), (4096, 300), (14336, 3), (256, 1)])
def test_rmsnorm_in_kernel_order_against_the_sequential_sum(hidden, rows):
    rng = np.random.default_rng(hidden + rows)
    x = (rng.standard_normal((rows, hidden)) * rng.uniform(0.01, 30.0, (rows, 1))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    want = O.rmsnorm(x, w, 1e-5)
    vpt, threads = wide_shape(hidden, rows)
    assert threads % 32 == 0 and vpt * threads * 4 >= hidden
    assert O.compare(O.rmsnorm_kernel_order(x, w, 1e-5, 0, threads, vpt), want)[0] == 0
    cl = pick_cluster(hidden)
    if cl:
        assert O.compare(O.rmsnorm_kernel_order(x, w, 1e-5, 1, 256, cl), want)[0] == 0


def test_launch_shapes_restate_the_driver():
    assert wide_shape(768, 32) == (1, 192) and wide_shape(4096, 128) == (1, 1024) and wide_shape(14336, 128) == (4, 896)
    assert wide_shape(4096, 1024) == (4, 256) and wide_shape(16388) is None and wide_shape(770) is None
    assert pick_cluster(768) == 1 and pick_cluster(4096) == 8 and pick_cluster(16448) is None


@pytest.mark.parametrize("hq,hkv,dh,bs,kv_bf16", [(12, 12, 64, 16, True), (4, 2, 128, 8, True), (3, 3, 40, 4, False),
                                                 (8, 2, 256, 32, True)])
def test_attention_in_kernel_order_against_the_sequential_loop(hq, hkv, dh, bs, kv_bf16):
    rng = np.random.default_rng(hq * dh)
    batch, nblk, mbps = 5, 64, 12
    lens = np.array([1, 2, 5, bs * 3 + 1, bs * mbps], np.uint32)
    tables = np.full((batch, mbps), 0xFFFFFFFF, np.uint32)
    perm = rng.permutation(nblk).astype(np.uint32)
    at = 0
    for b in range(batch):
        need = -(-int(lens[b]) // bs)
        tables[b, :need] = perm[at:at + need]
        at += need
    kp = rng.standard_normal((nblk * bs, hkv * dh)).astype(np.float32)
    vp = rng.standard_normal((nblk * bs, hkv * dh)).astype(np.float32)
    if kv_bf16:
        kp, vp = O.f32_to_bf16(kp), O.f32_to_bf16(vp)
    q = rng.standard_normal((batch, 1, hq * dh)).astype(np.float32)
    kw = dict(batch=batch, l_new=1, num_q_heads=hq, num_kv_heads=hkv, head_dim=dh, block_size=bs, num_blocks=nblk,
              max_blocks_per_seq=mbps, scale=float(1 / np.sqrt(dh)), kv_bf16=kv_bf16)
    want = O.paged_attention(q, kp, vp, tables, lens, **kw)
    got = O.paged_attention_kernel_order(q, kp, vp, tables, lens, **kw)
    fails, max_abs, max_rel = O.compare(got, want)
    assert fails == 0, (max_abs, max_rel)
    # one cached token: the softmax weight is exactly 1 in both orders
    assert np.array_equal(got[0], want[0])


def test_blas_product_of_int8_operands_is_the_exact_accumulator():
    rng = np.random.default_rng(3)
    for m, n, k in [(32, 130, 768), (5, 64, 1024), (7, 33, 3072), (2, 16, 14336)]:
        a = rng.integers(-128, 128, (m, k), dtype=np.int8)
        w = rng.integers(-128, 128, (n, k), dtype=np.int8)
        wf = O.int8_weight_for_blas(w)
        assert wf.dtype == (np.float32 if k <= 1024 else np.float64)
        assert np.array_equal(O.gemm_i8_s32_blas(a, wf), O.gemm_i8_s32(a, w))
    a = np.full((2, 1024), -128, np.int8)                    # the largest sums the f32 product has to hold
    assert np.array_equal(O.gemm_i8_s32_blas(a, O.int8_weight_for_blas(a)), O.gemm_i8_s32(a, a))


def test_decoder_in_kernel_order_stays_within_tolerance_of_the_sequential_decoder():
    """First step: identical inputs reach every operation, so the logits must meet the composite tolerance.
    Later steps run teacher-forced; after a per-token quantiser an int8 code may differ between the two orders,
    so the bound there is relative to the logit range."""
    cfg = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab=1024, max_seq_len=32)
    weights = make_weights(cfg, seed=21)
    seq, exact = DecoderRef(cfg, weights), DecoderRef(cfg, weights, exact=True)
    seq.begin(3)
    exact.begin(3)
    ids = np.random.default_rng(22).integers(0, 1024, (3, 12)).astype(np.int32)
    for t in range(12):
        ls, ns = seq.step(ids[:, t])
        le, ne = exact.step(ids[:, t])
        if t == 0:
            fails, max_abs, max_rel = O.compare(le, ls)
            assert fails == 0, (max_abs, max_rel)
        assert float(np.abs(le - ls).max()) < 0.03 * float(np.abs(ls).max()), t
    with pytest.raises(ValueError):
        DecoderRef(dict(cfg, head_dim=128, n_heads=2, n_kv_heads=1), make_weights(dict(cfg, head_dim=128, n_heads=2, n_kv_heads=1)),
                   exact=True)
