"""Host logic of the continuous-batching scheduler (no GPU): admission order, prompt feeding, completion and limits,
after the contract of the reference's BatchScheduler (crates/autodiff/src/generate/scheduler.rs:395-)."""
import numpy as np
import pytest

from fandhe_ai_b200 import BackendError
from fandhe_ai_b200.scheduler import BatchScheduler


def drive(s, sampler, max_steps=200):
    """Runs plan/commit with `sampler(row, fed_token)` standing in for the decoder; returns the trace of plans."""
    trace = []
    for _ in range(max_steps):
        if not (s.queued_len or s.active_len):
            break
        ids, active, restarts, done0 = s.plan_step()
        trace.append((ids.copy(), active.copy(), restarts, done0))
        if not active.any():
            s.commit_step(np.zeros(s.max_active, np.int32))
            continue
        s.commit_step(np.array([sampler(r, int(ids[r])) if active[r] else -1 for r in range(s.max_active)], np.int32))
    out = {}
    while (item := s.take_finished()) is not None:
        out[item[0]] = item[1].tolist()
    return out, trace


def test_single_request_feeds_its_prompt_then_its_samples():
    s = BatchScheduler(None, 2, 4, 16)
    rid = s.submit([7, 8, 9], 6)
    assert rid == 1 and s.queued_len == 1 and s.active_len == 0
    out, trace = drive(s, lambda row, tok: tok + 100)
    # steps feed 7, 8, 9, then the sample of 9, then the sample of that; samples after the last prompt token are kept
    assert [int(t[0][0]) for t in trace] == [7, 8, 9, 109, 209]
    assert trace[0][2] == [(0, 6)] and all(t[2] == [] for t in trace[1:])
    assert out == {1: [7, 8, 9, 109, 209, 309]}
    assert s.queued_len == 0 and s.active_len == 0


def test_admission_is_fifo_into_ascending_free_rows_and_rows_are_reused():
    s = BatchScheduler(None, 2, 8, 8)
    ids = [s.submit([10 * (i + 1)], 2 + i) for i in range(4)]      # lengths 2, 3, 4, 5: 1, 2, 3, 4 steps
    assert ids == [1, 2, 3, 4]
    out, trace = drive(s, lambda row, tok: tok + 1)
    assert trace[0][2] == [(0, 2), (1, 3)]                  # requests 1, 2 take rows 0, 1
    assert trace[1][2] == [(0, 4)]                          # request 1 finished after one step: request 3 takes row 0
    assert trace[2][2] == [(1, 5)]                          # request 2 finished after two steps: request 4 takes row 1
    assert out == {1: [10, 11], 2: [20, 21, 22], 3: [30, 31, 32, 33], 4: [40, 41, 42, 43, 44]}
    # a row that holds no request sits the step out
    assert trace[-1][1].tolist() == [0, 1]                  # at the end only request 4 is left, in row 1


def test_prompt_that_already_has_max_length_finishes_without_a_forward():
    s = BatchScheduler(None, 1, 4, 8)
    s.submit([1, 2, 3], 3)
    s.submit([4], 2)
    ids, active, restarts, done0 = s.plan_step()
    assert done0 == 1 and restarts == [(0, 2)] and int(ids[0]) == 4 and active[0] == 1
    assert s.commit_step([9]) == 1
    assert s.take_finished()[1].tolist() == [1, 2, 3]
    assert s.take_finished()[1].tolist() == [4, 9]
    assert s.take_finished() is None


def test_limits_and_invalid_requests_leave_the_state_unchanged():
    with pytest.raises(BackendError):
        BatchScheduler(None, 0, 1, 1)
    s = BatchScheduler(None, 1, 2, 4)
    for bad in (([], 3), ([1, 2, 3], 2), ([1], 5), ([1], 0)):
        with pytest.raises(BackendError) as e:
            s.submit(*bad)
        assert e.value.kind == "InvalidArgument"
    s.submit([1], 2)
    s.submit([2], 2)
    with pytest.raises(BackendError):        # queue full
        s.submit([3], 2)
    assert s.queued_len == 2 and s.active_len == 0
    with pytest.raises(BackendError):        # commit without a plan
        s.commit_step([0])
    s.plan_step()
    with pytest.raises(BackendError):        # two plans in a row
        s.plan_step()
    with pytest.raises(BackendError):        # the device half needs a decoder
        s.step()


def test_with_prefill_an_admitted_prompt_counts_as_fed_up_to_its_last_token():
    s = BatchScheduler(None, 2, 4, 16)
    s.configure(prefill=True)
    s.submit([7, 8, 9], 6)
    s.submit([5], 3)
    out, trace = drive(s, lambda row, tok: tok + 100)
    # the first batched step already feeds the LAST prompt token of request 1 (7 and 8 go through the prefill pass)
    assert [int(t[0][0]) for t in trace] == [9, 109, 209]
    assert [int(t[0][1]) for t in trace[:2]] == [5, 105]
    assert out == {1: [7, 8, 9, 109, 209, 309], 2: [5, 105, 205]}


def test_a_request_with_a_token_outside_the_vocabulary_is_set_apart_and_the_others_go_on():
    s = BatchScheduler(None, 2, 8, 8)
    s.configure(prefill=False, vocab=50)
    good1 = s.submit([1, 2], 4)
    bad = s.submit([3, 50], 4)              # 50 is outside [0, 50)
    worse = s.submit([-1], 4)
    good2 = s.submit([4], 3)
    out, trace = drive(s, lambda row, tok: (tok + 1) % 50)
    assert sorted(out) == [good1, good2] and s.failed_len == 2
    # the failed requests never took a row: the second row went to the next good request at once
    assert trace[0][2] == [(0, 4), (1, 3)]
    first, second = s.take_failed(), s.take_failed()
    assert first[0] == bad and second[0] == worse and first[1] == "InvalidArgument" and "vocabulary" in first[2]
    assert s.take_failed() is None and s.failed_len == 0
