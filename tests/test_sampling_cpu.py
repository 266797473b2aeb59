"""Sampling weights of generate(): the library's host code against the oracle restatement and the reference's own
unit-test vectors (crates/autodiff/src/generate/mod.rs, tests at :760-824).  The functions run on the host in the
reference too (f64 softmax, independent of the backend), so no GPU is needed."""
import numpy as np
import pytest

from fandhe_ai_b200._lib import BackendError
from fandhe_ai_b200.decoder import SAMPLE_GREEDY, SAMPLE_TEMPERATURE, SAMPLE_TOP_K, sampling_weights
from oracle import oracle as O


def test_reference_known_answers_of_top_k_and_softmax():
    # top_k_indices_orders_by_value_desc_then_index_asc / top_k_indices_truncates_to_k
    assert O.top_k_indices([1.0, 5.0, 5.0, 3.0, 0.0], 3) == [1, 2, 3]
    assert O.top_k_indices([4.0, 1.0, 3.0, 2.0], 1) == [0]
    assert O.top_k_indices([4.0, 1.0, 3.0, 2.0], 4) == [0, 2, 3, 1]
    # the same through the library: the support of the top-k weights is the reference's index set
    w = sampling_weights(np.array([[1.0, 5.0, 5.0, 3.0, 0.0]], np.float32), SAMPLE_TOP_K, k=3)[0]
    assert sorted(np.nonzero(w)[0].tolist()) == [1, 2, 3]
    assert w[1] == w[2] > w[3] > 0 and w[0] == 0 and w[4] == 0
    # ties broken by the smaller index: k = 1 over two equal maxima keeps index 1
    w = sampling_weights(np.array([[1.0, 5.0, 5.0, 3.0, 0.0]], np.float32), SAMPLE_TOP_K, k=1)[0]
    assert w.tolist() == [0.0, 1.0, 0.0, 0.0, 0.0]
    # softmax_weights_sum_to_one_and_are_non_negative
    w = sampling_weights(np.array([[1.0, 2.0, 3.0]], np.float32), SAMPLE_TEMPERATURE)[0]
    assert abs(float(w.sum()) - 1.0) < 1e-5 and np.all(w >= 0)
    # softmax_weights_are_numerically_stable_for_large_logits
    w = sampling_weights(np.array([[1e30, 1e30, -1e30]], np.float32), SAMPLE_TEMPERATURE)[0]
    assert np.all(np.isfinite(w)) and abs(float(w.sum()) - 1.0) < 1e-4 and w.tolist() == [0.5, 0.5, 0.0]
    # softmax_weights_lower_temperature_sharpens_distribution
    sharp = sampling_weights(np.array([[1.0, 2.0]], np.float32), SAMPLE_TEMPERATURE, temperature=0.1)[0]
    flat = sampling_weights(np.array([[1.0, 2.0]], np.float32), SAMPLE_TEMPERATURE, temperature=10.0)[0]
    assert sharp[1] > flat[1]
    # greedy: one-hot at the first maximum
    w = sampling_weights(np.array([[0.5, 2.0, 2.0, -1.0]], np.float32), SAMPLE_GREEDY)[0]
    assert w.tolist() == [0.0, 1.0, 0.0, 0.0]


@pytest.mark.parametrize("strategy,k,t", [(SAMPLE_TEMPERATURE, 0, 1.0), (SAMPLE_TEMPERATURE, 0, 0.7), (SAMPLE_TOP_K, 1, 1.0),
                                          (SAMPLE_TOP_K, 40, 0.8), (SAMPLE_TOP_K, 997, 1.3), (SAMPLE_GREEDY, 0, 1.0)])
def test_library_weights_equal_the_oracle(strategy, k, t):
    rng = np.random.default_rng(k + int(t * 10))
    logits = (rng.standard_normal((5, 997)) * 4).astype(np.float32)
    logits[1, 100:110] = logits[1, 5]            # ties inside and across the top-k boundary
    logits[2] = np.round(logits[2])              # many equal values
    got = sampling_weights(logits, strategy, k, t)
    for r in range(logits.shape[0]):
        want = O.sampling_weights(logits[r], strategy, k, t)
        assert np.array_equal(got[r] != 0, want != 0), r            # same support
        # exp() of the C library on both sides; allow the last f32 bit for a differently rounded f64 exp
        assert np.allclose(got[r], want, rtol=2e-7, atol=0), r
        assert abs(float(got[r].astype(np.float64).sum()) - 1.0) < 1e-5


def test_argument_rules_of_generate_config():
    x = np.zeros((1, 8), np.float32)
    for args in [(SAMPLE_TEMPERATURE, 0, 0.0), (SAMPLE_TEMPERATURE, 0, float("nan")), (SAMPLE_TEMPERATURE, 0, -1.0),
                 (SAMPLE_TEMPERATURE, 3, 1.0), (SAMPLE_GREEDY, 0, 0.5), (SAMPLE_GREEDY, 2, 1.0), (SAMPLE_TOP_K, 0, 1.0),
                 (SAMPLE_TOP_K, 9, 1.0), (7, 0, 1.0)]:
        with pytest.raises(BackendError) as e:
            sampling_weights(x, *args)
        assert e.value.kind == "InvalidArgument", args
    bad = x.copy()
    bad[0, 3] = np.inf
    with pytest.raises(BackendError) as e:
        sampling_weights(bad, SAMPLE_TEMPERATURE)
    assert e.value.kind == "InvalidArgument" and "non-finite" in str(e.value)
