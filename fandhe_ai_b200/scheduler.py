"""Continuous batching over the rows of one decoder: the host-side mirror of the reference's BatchScheduler
(crates/autodiff/src/generate/scheduler.rs:395-).  All logic lives in the C++ library (`b200_scheduler_*`)."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from ._lib import check, lib


class BatchScheduler:
    """FIFO queue + at most `max_active` requests in progress, one decoder row each.  `step()` admits queued
    requests into free rows and advances every request in progress by one token; a request is finished when it
    holds `max_length` tokens.  Without a decoder only `plan_step` / `commit_step` (the host logic) work."""

    def __init__(self, decoder, max_active: int, max_queued: int, max_length: int):
        self._dec = decoder          # keeps the decoder alive
        self.max_active = max_active
        h = C.c_void_p()
        check(lib().b200_scheduler_create(decoder._h if decoder is not None else None, max_active, max_queued,
                                          max_length, C.byref(h)))
        self._h = h

    def close(self) -> None:
        if self._h:
            lib().b200_scheduler_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, prompt, max_length: int) -> int:
        p = np.ascontiguousarray(np.asarray(prompt, np.int32).ravel())
        rid = C.c_uint64()
        check(lib().b200_scheduler_submit(self._h, p.ctypes.data_as(C.c_void_p), p.size, max_length, C.byref(rid)))
        return int(rid.value)

    @property
    def queued_len(self) -> int:
        return int(lib().b200_scheduler_queued_len(self._h))

    @property
    def active_len(self) -> int:
        return int(lib().b200_scheduler_active_len(self._h))

    @property
    def finished_len(self) -> int:
        return int(lib().b200_scheduler_finished_len(self._h))

    def step(self) -> int:
        done = C.c_int32()
        check(lib().b200_scheduler_step(self._h, C.byref(done)))
        return int(done.value)

    def plan_step(self):
        """Host half 1: returns (ids[max_active], active[max_active], [(row, max_length) restarted], completed)."""
        n = self.max_active
        ids = np.zeros(n, np.int32)
        active = np.zeros(n, np.uint8)
        rr, rl = np.zeros(n, np.int32), np.zeros(n, np.int32)
        nr, done = C.c_int32(), C.c_int32()
        check(lib().b200_scheduler_plan_step(self._h, ids.ctypes.data_as(C.c_void_p), active.ctypes.data_as(C.c_void_p),
                                             rr.ctypes.data_as(C.c_void_p), rl.ctypes.data_as(C.c_void_p), C.byref(nr),
                                             C.byref(done)))
        return ids, active, [(int(rr[i]), int(rl[i])) for i in range(nr.value)], int(done.value)

    def commit_step(self, sampled) -> int:
        s = np.ascontiguousarray(np.asarray(sampled, np.int32).ravel())
        assert s.size == self.max_active
        done = C.c_int32()
        check(lib().b200_scheduler_commit_step(self._h, s.ctypes.data_as(C.c_void_p), C.byref(done)))
        return int(done.value)

    def take_finished(self, capacity: int = 1 << 16) -> Optional[tuple[int, np.ndarray]]:
        buf = np.zeros(capacity, np.int32)
        rid, n = C.c_uint64(), C.c_int32()
        check(lib().b200_scheduler_take_finished(self._h, C.byref(rid), buf.ctypes.data_as(C.c_void_p), capacity, C.byref(n)))
        if n.value < 0:
            return None
        return int(rid.value), buf[: n.value].copy()

    @property
    def failed_len(self) -> int:
        return int(lib().b200_scheduler_failed_len(self._h))

    def take_failed(self) -> Optional[tuple[int, str, str]]:
        """Pops the oldest request that was set apart: (request id, error kind, message), or None."""
        rid, status, have = C.c_uint64(), C.c_int32(), C.c_int32()
        msg = C.create_string_buffer(512)
        check(lib().b200_scheduler_take_failed(self._h, C.byref(rid), C.byref(status), msg, 512, C.byref(have)))
        if not have.value:
            return None
        return int(rid.value), lib().b200_status_name(status.value).decode(), msg.value.decode()

    def configure(self, prefill: bool, vocab: int = 0) -> None:
        """Host-logic switches of a scheduler without a decoder (see b200_scheduler_configure)."""
        check(lib().b200_scheduler_configure(self._h, int(prefill), vocab))

    def run_until_idle(self, max_steps: int = 1 << 20) -> dict[int, np.ndarray]:
        """Steps until queue and rows are empty; returns {request id: tokens}."""
        out: dict[int, np.ndarray] = {}
        steps = 0
        while (self.queued_len or self.active_len) and steps < max_steps:
            self.step()
            steps += 1
        while True:
            item = self.take_finished()
            if item is None:
                break
            out[item[0]] = item[1]
        return out
