"""The per-ordinal error state machine of the boundary on a device: poison -> recover in place -> new generation,
the two transient refusals, and the final unrecoverable state (crates/backend-cuda/src/context_cache.rs,
variants crates/tensor-core/src/device.rs:300-371).  Every failure here is injected on the host; no kernel
faults, traps or hangs."""
import threading

import numpy as np
import pytest

from fandhe_ai_b200 import Backend, BackendError
from fandhe_ai_b200._lib import check, lib

pytestmark = pytest.mark.gpu


def test_poisoned_context_recovers_in_place_with_a_new_generation(fresh_be):
    be = fresh_be
    old = be.upload(np.arange(8, dtype=np.float32))
    gen0 = lib().b200_ctx_generation(be._ctx)
    be.recover()                                             # healthy: nothing happens
    assert lib().b200_ctx_generation(be._ctx) == gen0
    check(lib().b200_test_poison(be._ctx))
    with pytest.raises(BackendError) as e:
        be.upload(np.zeros(4, np.float32))
    assert e.value.kind == "DeviceContextPoisoned"
    check(lib().b200_test_inject_probe_failures(be._ctx, 1))
    with pytest.raises(BackendError) as e:                   # a failed probe keeps the context poisoned, retry allowed
        be.recover()
    assert e.value.kind == "DeviceContextPoisoned" and be.poisoned
    be.recover()
    assert not be.poisoned and lib().b200_ctx_generation(be._ctx) > gen0
    with pytest.raises(BackendError) as e:                   # handles of the old generation are refused, not UB
        be.download(old)
    assert e.value.kind == "StaleDeviceGeneration"
    x = np.arange(64, dtype=np.float32).reshape(2, 32)
    q, s = be.quantize_i8_per_row(be.upload(x), 2, 32)
    assert q.numpy()[1, 31] == 127


def test_three_failed_probes_make_the_context_unrecoverable(fresh_be):
    be = fresh_be
    check(lib().b200_test_poison(be._ctx))
    check(lib().b200_test_inject_probe_failures(be._ctx, 3))
    kinds = []
    for _ in range(3):
        with pytest.raises(BackendError) as e:
            be.recover()
        kinds.append(e.value.kind)
    assert kinds == ["DeviceContextPoisoned", "DeviceContextPoisoned", "DeviceContextUnrecoverable"]
    for call in (be.recover, be.synchronize_device, lambda: be.upload(np.zeros(4, np.float32))):
        with pytest.raises(BackendError) as e:
            call()
        assert e.value.kind == "DeviceContextUnrecoverable" and "injected probe mismatch" in e.value.message
    other = Backend(0)                                       # the device itself is fine
    try:
        assert other.upload(np.ones(4, np.float32)).numpy().sum() == 4
    finally:
        other.close()


def test_other_threads_are_refused_while_one_thread_captures(fresh_be):
    be = fresh_be
    check(lib().b200_test_mark_capturing(be._ctx, 1))
    seen = {}

    def other():
        try:
            be.synchronize_device()
            seen["kind"] = "ok"
        except BackendError as e:
            seen["kind"] = e.kind

    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["kind"] == "DeviceContextCaptureInProgress"
    be.synchronize_device()                                  # the capturing thread itself passes
    assert not be.poisoned                                   # transient: nothing was poisoned
    check(lib().b200_test_mark_capturing(be._ctx, 0))
    t = threading.Thread(target=other)
    t.start()
    t.join()
    assert seen["kind"] == "ok"
