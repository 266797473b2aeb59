"""Paged KV cache: argument types, validators and the two device entry points.

Host mirror of crates/tensor-core/src/paged_kv.rs (PagedKvLayout, PagedAttentionArgs,
PagedAttentionPlan, validate_paged_kv_append, validate_paged_attention) and of
BackendOps::paged_kv_append / paged_attention_forward
(crates/tensor-core/src/backend_ops.rs:4709-4786).  The checks themselves run in the shared
library (they are pure host code there and need no GPU); this module only shapes arguments.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import PagedAttentionArgsC, PagedAttentionPlanC, PagedKvLayoutC, check, lib
from .backend import BF16, F32, Backend, DeviceBuffer

SENTINEL = 0xFFFFFFFF  # unused block-table slot


@dataclass(frozen=True)
class PagedKvLayout:
    """K/V pool layout `[num_blocks, block_size, embed_dim]`; `dtype` is BF16 or F32."""
    num_blocks: int
    block_size: int
    embed_dim: int
    dtype: int = BF16

    def to_c(self) -> PagedKvLayoutC:
        return PagedKvLayoutC(self.num_blocks, self.block_size, self.embed_dim, self.dtype)

    @property
    def elem_size(self) -> int:
        return 2 if self.dtype == BF16 else 4

    @property
    def np_dtype(self):
        return np.uint16 if self.dtype == BF16 else np.float32

    def pool_elems(self) -> int:
        return self.num_blocks * self.block_size * self.embed_dim

    def pool_rows(self) -> int:
        return self.num_blocks * self.block_size


@dataclass(frozen=True)
class PagedAttentionArgs:
    layout: PagedKvLayout
    batch: int
    l_new: int
    num_heads: int
    max_blocks_per_seq: int
    scale: float
    num_kv_heads: int = 0  # 0: same as num_heads (the reference's multi-head attention)

    def to_c(self) -> PagedAttentionArgsC:
        kvh = self.num_kv_heads if self.num_kv_heads else self.num_heads
        return PagedAttentionArgsC(self.layout.to_c(), self.batch, self.l_new, self.num_heads, kvh,
                                   self.max_blocks_per_seq, self.scale)

    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads if self.num_kv_heads else self.num_heads

    def head_dim(self) -> int:
        return self.layout.embed_dim // self.kv_heads if self.kv_heads else 0


@dataclass(frozen=True)
class PagedAttentionPlan:
    out_numel: int
    s_max: int
    query_rows: int
    workspace_elems: int


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def validate_paged_kv_append(k_new_numel: int, v_new_numel: int, k_pool_numel: int, v_pool_numel: int, slot_mapping,
                             layout: PagedKvLayout) -> int:
    """Returns the number of rows to append, or raises BackendError(InvalidArgument)."""
    slots = _u32(slot_mapping)
    rows = C.c_uint64()
    lc = layout.to_c()
    check(lib().b200_validate_paged_kv_append(k_new_numel, v_new_numel, k_pool_numel, v_pool_numel,
                                              slots.ctypes.data_as(C.c_void_p), slots.size, C.byref(lc), C.byref(rows)))
    return int(rows.value)


def validate_paged_attention(q_numel: int, k_pool_numel: int, v_pool_numel: int, block_tables, seq_lens,
                             args: PagedAttentionArgs) -> PagedAttentionPlan:
    t = _u32(block_tables).ravel()
    s = _u32(seq_lens).ravel()
    plan = PagedAttentionPlanC()
    ac = args.to_c()
    check(lib().b200_validate_paged_attention(q_numel, k_pool_numel, v_pool_numel, t.ctypes.data_as(C.c_void_p), t.size,
                                              s.ctypes.data_as(C.c_void_p), s.size, C.byref(ac), C.byref(plan)))
    return PagedAttentionPlan(int(plan.out_numel), int(plan.s_max), int(plan.query_rows), int(plan.workspace_elems))


def paged_kv_append(be: Backend, k_new: DeviceBuffer, v_new: DeviceBuffer, k_pool: DeviceBuffer, v_pool: DeviceBuffer,
                    slot_mapping, layout: PagedKvLayout) -> None:
    slots = _u32(slot_mapping)
    lc = layout.to_c()
    check(lib().b200_paged_kv_append(be._ctx, k_new.handle, 0, v_new.handle, 0, k_pool.handle, v_pool.handle,
                                     slots.ctypes.data_as(C.c_void_p), slots.size, C.byref(lc)))


def paged_attention_forward(be: Backend, q: DeviceBuffer, k_pool: DeviceBuffer, v_pool: DeviceBuffer, block_tables,
                            seq_lens, args: PagedAttentionArgs, out: DeviceBuffer | None = None) -> DeviceBuffer:
    t = _u32(block_tables).ravel()
    s = _u32(seq_lens).ravel()
    ac = args.to_c()
    if out is None:
        out = be.alloc_zeroed((args.batch, args.l_new, args.num_heads * args.head_dim()), np.float32)
    check(lib().b200_paged_attention_forward(be._ctx, q.handle, 0, k_pool.handle, v_pool.handle,
                                             t.ctypes.data_as(C.c_void_p), t.size, s.ctypes.data_as(C.c_void_p), s.size,
                                             C.byref(ac), out.handle, 0))
    return out


def paged_attention_forward_resident(be: Backend, q: DeviceBuffer, k_pool: DeviceBuffer, v_pool: DeviceBuffer,
                                     block_tables: DeviceBuffer, seq_lens: DeviceBuffer, max_seq_len: int,
                                     args: PagedAttentionArgs, out: DeviceBuffer) -> DeviceBuffer:
    ac = args.to_c()
    check(lib().b200_paged_attention_forward_resident(be._ctx, q.handle, 0, k_pool.handle, v_pool.handle,
                                                      block_tables.handle, seq_lens.handle, max_seq_len, C.byref(ac),
                                                      out.handle, 0))
    return out


def paged_attention_forward_noalloc(be: Backend, q: DeviceBuffer, k_pool: DeviceBuffer, v_pool: DeviceBuffer,
                                    block_tables: DeviceBuffer, seq_lens: DeviceBuffer, max_seq_len: int,
                                    args: PagedAttentionArgs, out: DeviceBuffer) -> DeviceBuffer:
    """`paged_attention_forward_resident` for callers that must not allocate device memory during the
    call (a serving loop where cudaMalloc is forbidden, a process with a fixed memory budget): the split
    partials use a fixed 32 MiB array inside the library.  Larger requests raise Unsupported.  The first
    call per device resolves the array's address and should precede any stream capture; overlapping calls
    on one GPU race on the array."""
    ac = args.to_c()
    check(lib().b200_paged_attention_forward_noalloc(be._ctx, q.handle, 0, k_pool.handle, v_pool.handle,
                                                     block_tables.handle, seq_lens.handle, max_seq_len, C.byref(ac),
                                                     out.handle, 0))
    return out


def paged_attention_tuning(be: Backend, chunk_blocks: int = 0) -> None:
    check(lib().b200_paged_attention_tuning(be._ctx, chunk_blocks))
