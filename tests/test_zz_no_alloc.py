"""The allocation-free decode-attention entry point.

Some callers of this library may not allocate device memory while they are serving: cudaMalloc can stall
the whole GPU behind a driver lock, and a process that handed out its memory budget at start-up has none
left to give.  b200_paged_attention_forward_noalloc keeps the split partials in a fixed array inside the
library image instead.  This file is collected last on purpose: it must pass on its own in a fresh
process and after every other test has used the same GPU."""
import numpy as np
import pytest

from fandhe_ai_b200 import BF16, BackendError
from fandhe_ai_b200 import paged_kv as P
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def problem(seed, batch=6, heads=8, kv_heads=2, lo=40, hi=1200, nblk=700):
    rng = np.random.default_rng(seed)
    dh, bs = 128, 16
    ekv = kv_heads * dh
    ctx = rng.integers(lo, hi + 1, batch).astype(np.uint32)
    mbps = -(-hi // bs)
    perm = rng.permutation(nblk).astype(np.uint32)
    tables = np.full((batch, mbps), P.SENTINEL, np.uint32)
    at = 0
    for b in range(batch):
        used = -(-int(ctx[b]) // bs)
        tables[b, :used] = perm[at:at + used]
        at += used
    k = O.f32_to_bf16(rng.standard_normal((nblk * bs, ekv), dtype=np.float32))
    v = O.f32_to_bf16(rng.standard_normal((nblk * bs, ekv), dtype=np.float32))
    q = rng.standard_normal((batch, 1, heads * dh), dtype=np.float32)
    args = P.PagedAttentionArgs(P.PagedKvLayout(nblk, bs, ekv, BF16), batch, 1, heads, mbps, float(1.0 / np.sqrt(dh)),
                                kv_heads)
    return q, k, v, tables, ctx, args


def test_noalloc_entry_matches_the_allocating_entry_on_two_calls_in_a_row(be):
    """Two consecutive calls with different inputs: the second one finds the first one's partials in the
    shared array and must not be disturbed by them.  Same kernels, same split sizes: results are identical
    bit for bit, which is stricter than the composite tolerance the other attention tests use."""
    for seed in (21, 22):
        q, k, v, tables, ctx, args = problem(seed)
        qd, kd, vd = be.upload(q), be.upload(k), be.upload(v)
        td, sd = be.upload(tables), be.upload(ctx)
        want = be.alloc_zeroed(q.shape, np.float32)
        P.paged_attention_forward_resident(be, qd, kd, vd, td, sd, int(ctx.max()), args, want)
        got = be.upload(np.full(q.shape, np.nan, np.float32))
        be.synchronize_device()
        free_before = be.memory_info()[0]
        P.paged_attention_forward_noalloc(be, qd, kd, vd, td, sd, int(ctx.max()), args, got)
        be.synchronize_device()
        if seed == 22:
            # the property the entry exists for: by the second call nothing is left to set up, and the amount of
            # free device memory is the same after the call as before it
            assert be.memory_info()[0] == free_before
        a, b = got.numpy(), want.numpy()
        assert np.all(np.isfinite(a))
        assert O.compare(a, b)[0] == 0
        assert np.array_equal(a, b)
        # and both agree with the CPU oracle
        ref = O.paged_attention(q, k, v, tables, ctx, batch=args.batch, l_new=1, num_q_heads=args.num_heads,
                                num_kv_heads=args.kv_heads, head_dim=128, block_size=16,
                                num_blocks=args.layout.num_blocks, max_blocks_per_seq=args.max_blocks_per_seq,
                                scale=args.scale, kv_bf16=True)
        assert O.compare(a, ref)[0] == 0
        for buf in (qd, kd, vd, td, sd, want, got):
            buf.release()


def test_noalloc_entry_refuses_sizes_beyond_its_static_scratch(be):
    # 64 rows x 32 heads x 32 splits x 520 bytes = 34 MB > 32 MiB: refused before any launch
    batch, heads, kv_heads, dh, bs = 64, 32, 8, 128, 16
    mbps = 1024
    nblk = 64
    layout = P.PagedKvLayout(nblk, bs, kv_heads * dh, BF16)
    args = P.PagedAttentionArgs(layout, batch, 1, heads, mbps, 0.1, kv_heads)
    q = be.alloc_zeroed((batch, 1, heads * dh), np.float32)
    out = be.alloc_zeroed((batch, 1, heads * dh), np.float32)
    pool = be.alloc_zeroed((nblk * bs, kv_heads * dh), np.uint16)
    tables = be.upload(np.zeros((batch, mbps), np.uint32))
    lens = be.upload(np.full(batch, 16, np.uint32))
    with pytest.raises(BackendError) as e:
        P.paged_attention_forward_noalloc(be, q, pool, pool, tables, lens, 16384, args, out)
    assert e.value.kind == "Unsupported" and "static scratch" in e.value.message
    assert not be.poisoned
    # the same shape with a smaller bound on the sequence length fits (8 splits) and runs
    P.paged_attention_forward_noalloc(be, q, pool, pool, tables, lens, 2048, args, out)
    assert np.all(np.isfinite(out.numpy()))
    for buf in (q, out, pool, tables, lens):
        buf.release()
