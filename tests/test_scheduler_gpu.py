"""Continuous batching on the GPU: every request's tokens equal those of the CPU decoder run on that request alone,
whatever the other rows are doing; requests that cannot be served are set apart."""
import numpy as np
import pytest

from fandhe_ai_b200 import Backend
from fandhe_ai_b200.decoder import Decoder, DecoderConfig
from fandhe_ai_b200.scheduler import BatchScheduler

pytestmark = pytest.mark.gpu

CFG = dict(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, d_ff=512, vocab=512)


def make_decoder(be, slots, max_len):
    blocks_per_seq = -(-max_len // 16)
    dc = DecoderConfig(CFG["n_layers"], CFG["d_model"], CFG["n_heads"], CFG["n_kv_heads"], CFG["head_dim"], CFG["d_ff"],
                       CFG["vocab"], max_batch=slots, max_seq_len=max_len, block_size=16,
                       num_blocks=slots * blocks_per_seq, use_graph=1)
    dec = Decoder(be, dc)
    dec.init_random(seed=3, std=0.05)
    return dec


def test_requests_through_shared_rows_match_requests_run_alone(be):
    slots, max_len = 3, 40
    rng = np.random.default_rng(5)
    reqs = [(rng.integers(0, CFG["vocab"], int(rng.integers(1, 12))).astype(np.int32), int(rng.integers(14, max_len + 1)))
            for _ in range(8)]
    dec = make_decoder(be, slots, max_len)
    try:
        # every request alone (the other rows sit out), in the same decoder and plans
        alone = []
        for prompt, length in reqs:
            s = BatchScheduler(dec, slots, 4, max_len)
            s.submit(prompt, length)
            (tokens,) = s.run_until_idle().values()
            s.close()
            alone.append(tokens)
            assert tokens.size == length and np.array_equal(tokens[: prompt.size], prompt)
        # all of them through three rows, admitted as rows free up
        s = BatchScheduler(dec, slots, len(reqs), max_len)
        ids = [s.submit(p, n) for p, n in reqs]
        assert s.queued_len == len(reqs)
        steps = 0
        while s.queued_len or s.active_len:
            s.step()
            steps += 1
            assert s.active_len <= slots
        got = {}
        while (item := s.take_finished()) is not None:
            got[item[0]] = item[1]
        s.close()
        assert sorted(got) == ids
        for rid, want in zip(ids, alone):
            assert np.array_equal(got[rid], want), rid
        # rows were shared: fewer steps than running the requests one after the other
        assert steps < sum(n - 1 for _, n in reqs)
    finally:
        dec.close()


def test_full_rows_match_generate(be):
    # equal prompts lengths, all rows busy from the first step: the same token sequence as generate()
    slots, plen, total = 4, 5, 20
    rng = np.random.default_rng(11)
    prompts = rng.integers(0, CFG["vocab"], (slots, plen)).astype(np.int32)
    dec = make_decoder(be, slots, total)
    try:
        want = dec.generate(prompts, total)
        s = BatchScheduler(dec, slots, slots, total)
        ids = [s.submit(prompts[i], total) for i in range(slots)]
        got = s.run_until_idle()
        s.close()
        for i, rid in enumerate(ids):
            assert np.array_equal(got[rid], want[i]), i
    finally:
        dec.close()


CFG64 = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab=512, max_seq_len=40)


def test_requests_through_shared_rows_match_the_cpu_decoder_request_by_request(be):
    """Each request against the kernel-order CPU decoder (oracle/decoder_ref.py, exact=True) run on that request
    alone with batch 1: identical token ids.  Prompts of different lengths are prefilled on admission while other rows
    are in the middle of their generation; more requests than rows."""
    from oracle.decoder_ref import DecoderRef, make_weights

    slots, max_len = 3, 40
    weights = make_weights(CFG64, seed=61)
    rng = np.random.default_rng(62)
    reqs = [(rng.integers(0, CFG64["vocab"], int(rng.integers(1, 14))).astype(np.int32), int(rng.integers(15, max_len + 1)))
            for _ in range(7)]
    want = []
    for prompt, length in reqs:
        ids, _ = DecoderRef(CFG64, weights, exact=True).generate(prompt[None, :], length)
        want.append(ids[0])
    dc = DecoderConfig(CFG64["n_layers"], CFG64["d_model"], CFG64["n_heads"], CFG64["n_kv_heads"], CFG64["head_dim"],
                       CFG64["d_ff"], CFG64["vocab"], max_batch=slots, max_seq_len=max_len, block_size=16,
                       num_blocks=slots * 3, use_graph=1)
    dec = Decoder(be, dc)
    try:
        dec.load_weights(weights)
        s = BatchScheduler(dec, slots, 16, max_len)
        ids = [s.submit(p, n) for p, n in reqs[:4]]
        bad = s.submit([3, CFG64["vocab"]], 10)                  # a token the model cannot embed
        ids += [s.submit(p, n) for p, n in reqs[4:]]
        got = s.run_until_idle()
        assert sorted(got) == sorted(ids)
        for rid, w in zip(ids, want):
            assert np.array_equal(got[rid], w), (rid, got[rid].tolist(), w.tolist())
        failed = s.take_failed()
        assert failed is not None and failed[0] == bad and failed[1] == "InvalidArgument" and s.take_failed() is None
        s.close()
    finally:
        dec.close()
