"""CPU side of the FP8 x FP8 form of the decoder: the per-row E4M3 quantiser of the oracle and the CPU decoder that uses
it (the reference has no FP8 decoder: parity unpinned; the E4M3 codec itself is checked against torch's cast in
tests/test_oracle_golden.py)."""
import numpy as np

from oracle import oracle as O
from oracle.decoder_ref import DecoderRef, make_weights


def test_per_row_e4m3_quantiser():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((7, 96)) * rng.uniform(0.01, 30.0, (7, 1))).astype(np.float32)
    x[3] = 0.0                                   # an all-zero row: scale 0, codes 0
    q, s = O.quantize_fp8_per_row(x)
    assert q.dtype == np.uint8 and q.shape == x.shape and s.shape == (7,)
    amax = np.abs(x).max(axis=1)
    assert np.array_equal(s, (amax / np.float32(448.0)).astype(np.float32))
    assert s[3] == 0.0 and not q[3].any()
    back = O.e4m3_to_f32(q) * s[:, None]
    # the row maximum maps to +-448 exactly; every other value lands within half an E4M3 step (2^-4 relative for normals)
    for r in (0, 1, 2, 4, 5, 6):
        j = int(np.argmax(np.abs(x[r])))
        assert abs(O.e4m3_to_f32(q[r:r + 1, j:j + 1])[0, 0]) == 448.0
        big = np.abs(x[r]) > amax[r] / 16
        assert np.all(np.abs(back[r][big] - x[r][big]) <= np.abs(x[r][big]) * 2.0 ** -4 + 1e-12)
    # same codes as the scalar codec applied to x / scale
    for r, c in ((0, 0), (2, 17), (6, 95)):
        assert int(q[r, c]) == O.f32_to_e4m3_scalar(float(np.float32(x[r, c]) / s[r]))


def test_fp8_cpu_decoder_tracks_the_int8_one():
    cfg = dict(n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, d_ff=256, vocab=256, max_seq_len=16)
    w = make_weights(cfg, seed=3)
    a, b = DecoderRef(cfg, w), DecoderRef(cfg, w, fp8=True)
    a.begin(2)
    b.begin(2)
    ids = np.array([5, 77])
    for _ in range(3):
        la, na = a.step(ids)
        lb, _ = b.step(ids)
        assert np.all(np.isfinite(lb))
        dev = float(np.abs(la - lb).max() / np.abs(la).max())
        assert 1e-4 < dev < 0.3, dev              # different arithmetic, same model
        ids = na
