"""Host logic without a GPU: the page table against the reference's exact slot sequences
(crates/autodiff/src/nn/paged_kv_device.rs:618-637, 744-764; crates/autodiff/src/nn/paged_kv.rs:850-871)."""
import numpy as np
import pytest

from fandhe_ai_b200._lib import BackendError
from fandhe_ai_b200.decoder import BlockTable


def test_append_builds_row_major_slot_mapping():
    # append_builds_row_major_slot_mapping_and_commits: 3 blocks of 2 tokens
    t = BlockTable(3, 2)
    with pytest.raises(BackendError):           # B=2, L_new=3 needs 4 blocks, 3 are free
        t.extend_for_append(2, 3)
    assert t.seq_len == 0 and t.batch is None   # state unchanged by the failure
    assert t.extend_for_append(1, 3) == [0, 1, 2]
    assert t.seq_len == 3 and t.num_used_blocks == 2
    assert t.extend_for_append(1, 2) == [3, 4]  # pos 3 -> block 1 row 1 (slot 3); pos 4 -> new block 2 (slot 4)
    assert t.num_free_blocks == 0


def test_rewind_and_clear_follow_reference_semantics():
    # rewind_and_clear_follow_reference_semantics
    t = BlockTable(3, 2)
    t.extend_for_append(1, 5)
    assert t.num_free_blocks == 0
    with pytest.raises(BackendError):
        t.rewind_to(6)
    assert t.seq_len == 5
    t.rewind_to(2)
    assert (t.seq_len, t.num_used_blocks, t.num_free_blocks) == (2, 1, 2)
    # blocks came back in the order 2, 1; the stack hands out 1 first -> slot 2
    assert t.extend_for_append(1, 1) == [2]
    t.rewind_to(0)
    assert t.batch is None
    t.clear()
    assert t.num_free_blocks == 3 and t.seq_len == 0


def test_batch_rows_are_interleaved_row_major_and_flattened_with_sentinel():
    t = BlockTable(8, 4)
    slots = t.extend_for_append(2, 5)            # row 0 takes blocks 0, 1; row 1 takes 2, 3
    assert slots == [0, 1, 2, 3, 4, 8, 9, 10, 11, 12]
    flat = t.flatten_tables(3)
    assert flat.tolist() == [[0, 1, 0xFFFFFFFF], [2, 3, 0xFFFFFFFF]]
    with pytest.raises(BackendError):            # the batch is fixed once set
        t.extend_for_append(3, 1)
    with pytest.raises(BackendError):            # a row already holds more blocks than the width asked for
        t.flatten_tables(1)
    assert t.extend_for_append(2, 0) == []       # l_new == 0 does nothing
    with pytest.raises(BackendError):
        BlockTable(4, 3)                         # block size must be a power of two
    with pytest.raises(BackendError):
        t.extend_for_append(0, 1)
