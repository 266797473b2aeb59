"""The C-ABI boundary without a GPU: the library loads, exports every symbol that
include/b200_backend.h declares, and its pure-host validators reproduce the reference's own
validator vectors (crates/tensor-core/src/paged_kv.rs:387-521)."""
import ctypes as C
import re
from pathlib import Path

import pytest

from fandhe_ai_b200 import paged_kv as P
from fandhe_ai_b200._lib import SIGNATURES, BackendError, lib
from fandhe_ai_b200.backend import BF16, F32

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "b200_backend.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    l = lib()
    names = declared_symbols()
    assert len(names) >= 25
    for name in names:
        assert hasattr(l, name), f"{name} is declared in the header but not exported"
        assert name in SIGNATURES, f"{name} has no ctypes signature"
    for name in SIGNATURES:
        assert name in names, f"{name} is bound but not declared in the header"


def test_status_names_follow_backend_error_variants():
    l = lib()
    want = {0: "Ok", 1: "ShapeMismatch", 2: "DeviceMismatch", 3: "DeviceAllocationFailed", 4: "KernelLaunchFailed",
            5: "DeviceUnavailable", 6: "TransferFailed", 7: "Unsupported", 8: "StorePoisoned", 9: "InvalidArgument",
            10: "DeviceContextPoisoned", 11: "StaleDeviceGeneration", 12: "DeviceContextRetiring",
            13: "DeviceContextUnrecoverable", 14: "DeviceContextCaptureInProgress"}
    for code, name in want.items():
        assert l.b200_status_name(code).decode() == name


def test_no_device_means_device_unavailable_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    ctx = C.c_void_p()
    st = lib().b200_ctx_create(0, C.byref(ctx))
    assert lib().b200_status_name(st).decode() == "DeviceUnavailable"
    assert not ctx.value


def L(nb, bs, e, dtype=F32):
    return P.PagedKvLayout(nb, bs, e, dtype)


def ok_layout(*a, **k):
    # a layout is checked by every validator; use the append validator with no rows
    l = L(*a, **k)
    pool = l.pool_elems() if l.num_blocks < 2**40 and l.embed_dim < 2**40 else 0
    return P.validate_paged_kv_append(0, 0, pool, pool, [], l)


def bad(fn, *a, **k):
    with pytest.raises(BackendError) as e:
        fn(*a, **k)
    assert e.value.kind == "InvalidArgument"


def test_layout_rejects_invalid_values():
    # layout_rejects_invalid_values (paged_kv.rs:395-405)
    bad(ok_layout, 0, 2, 4)
    bad(ok_layout, 4, 3, 4)
    bad(ok_layout, 4, 512, 4)
    bad(ok_layout, 4, 2, 0)
    bad(ok_layout, 2**32 - 1, 2, 4)
    bad(ok_layout, 4, 2, 2**64 - 1)
    bad(ok_layout, 1 << 20, 256, (2**63 - 1) // (8 * 256) + 1)
    assert ok_layout(4, 256, 4) == 0
    assert ok_layout(4, 256, 4, BF16) == 0


def args(batch, l_new, max_blocks, heads=2, scale=0.5, layout=None, kv=0):
    return P.PagedAttentionArgs(layout or L(4, 2, 4), batch, l_new, heads, max_blocks, scale, kv)


def test_args_reject_bad_heads_scale_and_sizes():
    # args_reject_bad_heads_scale_and_sizes (paged_kv.rs:408-417)
    v = lambda a: P.validate_paged_attention(a.batch * a.l_new * 4, 32, 32, [0] * (a.batch * a.max_blocks_per_seq)
                                             if a.batch < 100 else [], [2] * a.batch if a.batch < 100 else [], a)
    bad(v, args(1, 1, 2, heads=0, scale=1.0, kv=0))
    bad(v, args(1, 1, 2, heads=3, scale=1.0))
    bad(v, args(1, 1, 2, scale=float("nan")))
    bad(v, args(1, 1, 2, scale=float("inf")))
    bad(v, args(2**63, 1, 2, scale=1.0))
    assert args(1, 1, 2).head_dim() == 2


def test_append_accepts_valid_and_rejects_violations():
    # append_accepts_valid_and_rejects_violations (paged_kv.rs:420-444)
    l = L(4, 2, 4)
    pool = 32
    va = P.validate_paged_kv_append
    assert va(8, 8, pool, pool, [0, 7], l) == 2
    bad(va, 7, 8, pool, pool, [0, 7], l)
    bad(va, 8, 4, pool, pool, [0, 7], l)
    bad(va, 8, 8, pool - 1, pool, [0, 7], l)
    bad(va, 8, 8, pool, pool, [0, 8], l)
    bad(va, 4, 4, pool, pool, [0xFFFFFFFF], l)
    bad(va, 8, 8, pool, pool, [3, 3], l)
    assert va(0, 0, pool, pool, [], l) == 0


def test_attention_accepts_valid_and_reports_plan():
    # attention_accepts_valid_and_reports_plan (paged_kv.rs:447-457)
    plan = P.validate_paged_attention(8, 32, 32, [0, 1, 2, 3], [3, 3], args(2, 1, 2))
    assert (plan.out_numel, plan.s_max, plan.query_rows, plan.workspace_elems) == (8, 3, 4, 12)


def test_attention_rejects_violations():
    # attention_rejects_violations (paged_kv.rs:460-481)
    a = args(1, 2, 2)
    pool = 32
    v = P.validate_paged_attention
    assert v(8, pool, pool, [0, 1], [3], a)
    bad(v, 7, pool, pool, [0, 1], [3], a)
    bad(v, 8, pool - 1, pool, [0, 1], [3], a)
    bad(v, 8, pool, pool, [0], [3], a)
    bad(v, 8, pool, pool, [0, 1], [3, 3], a)
    bad(v, 8, pool, pool, [0, 1], [1], a)
    bad(v, 8, pool, pool, [0, 1], [5], a)
    bad(v, 8, pool, pool, [0, 4], [3], a)
    bad(v, 8, pool, pool, [0, 0xFFFFFFFF], [3], a)
    assert v(8, pool, pool, [0, 0xFFFFFFFF], [2], a)   # the sentinel is fine in an unused slot


def test_attention_rejects_workspace_overflow():
    # attention_rejects_workspace_overflow (paged_kv.rs:484-503): query_rows * s_max above 2^30
    a = P.PagedAttentionArgs(L(4, 2, 4), 1 << 12, 1 << 10, 1, 2, 1.0)
    bad(P.validate_paged_attention, (1 << 12) * (1 << 10) * 4, 32, 32, [0] * ((1 << 12) * 2), [1024] * (1 << 12), a)
    big = P.PagedAttentionArgs(L(4096, 256, 4), 1 << 11, 1, 1, 4096, 1.0)
    n = (1 << 11)
    bad(P.validate_paged_attention, n * 4, big.layout.pool_elems(), big.layout.pool_elems(), [0] * (n * 4096),
        [1 << 20] * n, big)


def test_validators_recheck_every_call():
    # validators_recheck_mutated_public_fields (paged_kv.rs:506-520): the C structs are plain data, so every
    # call re-validates them
    pool = 32
    bad(P.validate_paged_attention, 4, pool, pool, [0, 1], [2], args(1, 1, 2, heads=0))
    bad(P.validate_paged_attention, 4, pool, pool, [0, 1], [2], args(1, 1, 2, layout=L(4, 0, 4)))
    bad(P.validate_paged_kv_append, 0, 0, pool, pool, [], L(4, 0, 4))
    bad(P.validate_paged_attention, 0, pool, pool, [0, 1], [2], args(1, 0, 2, scale=float("nan")))


def test_empty_batch_and_empty_l_new_are_valid():
    # empty_batch_and_empty_l_new_are_valid (paged_kv.rs:523-533)
    plan = P.validate_paged_attention(0, 32, 32, [], [], args(0, 1, 2))
    assert plan.out_numel == 0 and plan.workspace_elems == 0
    plan = P.validate_paged_attention(0, 32, 32, [0, 1], [3], args(1, 0, 2))
    assert plan.out_numel == 0 and plan.workspace_elems == 0


def test_gqa_extension_of_the_validator():
    # 4 query heads on 2 kv heads: q has 2x the pool's embed_dim
    a = args(1, 1, 2, heads=4, kv=2)
    assert a.head_dim() == 2
    plan = P.validate_paged_attention(8, 32, 32, [0, 1], [3], a)
    assert plan.out_numel == 8 and plan.query_rows == 4
    bad(P.validate_paged_attention, 8, 32, 32, [0, 1], [3], args(1, 1, 2, heads=3, kv=2))
