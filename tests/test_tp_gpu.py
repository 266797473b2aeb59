"""Tensor-parallel decode on two GPUs of one box (skipped when fewer are visible)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("exchange", ["2", "1", "0"])
def test_two_rank_tensor_parallel_decode_matches_the_cpu_decoder(exchange):
    """exchange 2: the row-parallel GEMMs store their partial rows into the owner's CUDA-IPC mapped block and the finish
    kernel reads local memory; 1: the finish kernel loads the partials from the peers; 0: ncclAllReduce is forced."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TP_EXCHANGE="0" if exchange == "0" else "1",
               B200_TP_PUSH="1" if exchange == "2" else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", str(ROOT / "tests" / "multi" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-8000:]
    # the path that ran is the path that was asked for: a silent fall-back to ncclAllReduce would leave the finish
    # kernel (peer sum, residual, RMSNorm, int8 delivery) unchecked
    assert f"exchange={exchange}" in r.stdout, r.stdout[-3000:]


@pytest.mark.parametrize("exchange", ["2", "0"])
def test_two_rank_fp8_decoder_matches_the_cpu_fp8_decoder(exchange):
    """The FP8 x FP8 form under tensor parallelism (E4M3 rows delivered by the finish kernel, f32 accumulators scattered
    by the row-parallel GEMMs; or ncclAllReduce) against the CPU FP8 decoder with the same rank split."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TP_FP8="1", B200_TP_EXCHANGE="0" if exchange == "0" else "1",
               B200_TP_PUSH="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29735", str(ROOT / "tests" / "multi" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-8000:]
    assert f"exchange={exchange}" in r.stdout, r.stdout[-3000:]


def test_two_rank_exact_int8_gives_the_logits_of_one_gpu():
    """tp_exact_int8 = 1: one per-token scale over the ranks (max all-reduce) and int32 partial sums (sum all-reduce):
    ids and logits equal those of the kernel-order CPU decoder WITHOUT tensor parallelism, bit for bit."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TP_EXACT="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29733", str(ROOT / "tests" / "multi" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-8000:]


def test_peer_wait_runs_out_with_an_error_status_and_the_device_stays_usable(fresh_be):
    """Failure detection without a fault: a finish kernel whose peer never raises its flag gives up after its
    bounded wait, the context reports the device error and is poisoned, and a new context works."""
    import numpy as np

    from fandhe_ai_b200 import Backend, BackendError
    from fandhe_ai_b200._lib import lib

    with pytest.raises(BackendError) as e:
        from fandhe_ai_b200._lib import check

        check(lib().b200_selftest_peer_wait(fresh_be._ctx))
    assert e.value.kind == "KernelLaunchFailed" and "0x301" in str(e.value)
    assert fresh_be.poisoned
    other = Backend(0)
    try:
        x = np.arange(64, dtype=np.float32).reshape(2, 32)
        q, s = other.quantize_i8_per_row(other.upload(x), 2, 32)
        assert q.numpy()[1, 31] == 127 and not other.poisoned
    finally:
        other.close()


@pytest.mark.parametrize("tp,d", [(2, 512), (4, 4096), (8, 4096), (8, 768)])
def test_finish_kernel_numerics_on_one_gpu(be, tp, d):
    """The cross-GPU finish kernel with nothing to wait for: `tp` exchange blocks on one device, every ready flag
    raised beforehand.  Run as each rank in turn, its rows must equal the CPU restatement bit for bit (partials
    added in rank order, residual, RMSNorm in kernel order, per-token int8) in EVERY rank's block, and its
    delivered flag must carry the epoch everywhere."""
    import ctypes as C

    from fandhe_ai_b200._lib import check, lib
    from oracle import oracle as O
    from oracle.decoder_ref import wide_shape

    rows = 3
    m = tp * rows
    rng = np.random.default_rng(tp * 1000 + d)
    partials = (rng.standard_normal((tp, m, d)) * 0.3).astype(np.float32)
    residual = rng.standard_normal((m, d)).astype(np.float32)
    norm_w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    total = np.zeros((m, d), np.float32)
    for p in range(tp):
        total = (total + partials[p]).astype(np.float32)           # rank order
    h_want = (total + residual).astype(np.float32)
    vpt, threads = wide_shape(d)
    xn = O.rmsnorm_kernel_order(h_want, norm_w, 1e-5, 0, threads, vpt)
    q_want, s_want = O.quantize_i8_per_row(xn)
    for rank in range(tp):
        h_out = np.empty((rows, d), np.float32)
        xq_out = np.empty((tp, rows, d), np.int8)
        sx_out = np.empty((tp, rows), np.float32)
        flags = np.empty((tp, 128), np.uint32)
        check(lib().b200_selftest_tp_finish(be._ctx, tp, rank, rows, d, partials.ctypes.data_as(C.c_void_p),
                                            residual.ctypes.data_as(C.c_void_p), norm_w.ctypes.data_as(C.c_void_p),
                                            C.c_float(1e-5), h_out.ctypes.data_as(C.c_void_p),
                                            xq_out.ctypes.data_as(C.c_void_p), sx_out.ctypes.data_as(C.c_void_p),
                                            flags.ctypes.data_as(C.c_void_p)))
        own = slice(rank * rows, (rank + 1) * rows)
        assert np.array_equal(h_out, h_want[own]), rank
        for p in range(tp):
            assert np.array_equal(xq_out[p], q_want[own]), (rank, p)
            assert np.array_equal(sx_out[p], s_want[own]), (rank, p)
            assert flags[p, 64 + rank] == 1, (rank, p, flags[p, 64:64 + tp])     # delivered, epoch 1
            assert flags[p, rank] == 1                                           # ready, raised again by the kernel
    assert not be.poisoned


@pytest.mark.parametrize("tp,rows,d,k,splits,tile", [
    (2, 64, 512, 256, 0, 0),
    (8, 16, 4096, 512, 0, 0),        # the O projection of one rank of eight (8B shapes)
    (8, 16, 4096, 1792, 0, 0),       # the down projection
    (8, 16, 4096, 512, 4, 64),
    (4, 3, 768, 128, 1, 128),        # one K slice (no cluster), fewer rows than a tile
    (3, 50, 1024, 384, 0, 0),        # owners' row ranges cross the 32-row quarters of a tile, two row tiles
])
def test_scattered_row_parallel_output_on_one_gpu(be, tp, rows, d, k, splits, tile):
    """A row-parallel GEMM that stores every row into the exchange block of the rank that owns it, then the finish
    kernel in its scattered form (local loads only), with `tp` blocks on one device and every GEMM complete before
    the first finish.  Residual rows, int8 rows and scales must equal the CPU restatement bit for bit (exact int32
    GEMM, one rounding of acc * (sa * sb), partials added in rank order, RMSNorm in kernel order), in the first
    and in the last block, and every block must have counted every rank's launch once."""
    import ctypes as C

    from fandhe_ai_b200._lib import check, lib
    from oracle import oracle as O
    from oracle.decoder_ref import wide_shape

    m = tp * rows
    rng = np.random.default_rng(tp * 7919 + d + k)
    a_q = rng.integers(-127, 128, (tp, m, k), dtype=np.int8)
    w_q = rng.integers(-127, 128, (tp, d, k), dtype=np.int8)
    a_s = rng.uniform(0.5e-2, 2e-2, (tp, m)).astype(np.float32)
    w_s = rng.uniform(0.5e-3, 2e-3, (tp, d)).astype(np.float32)
    residual = rng.standard_normal((m, d)).astype(np.float32)
    norm_w = rng.uniform(0.5, 1.5, d).astype(np.float32)
    total = np.zeros((m, d), np.float32)
    for p in range(tp):
        acc = O.gemm_i8_s32(a_q[p], w_q[p]).astype(np.float32)
        scale = (a_s[p][:, None] * w_s[p][None, :]).astype(np.float32)
        total = (total + (acc * scale).astype(np.float32)).astype(np.float32)
    h_want = (total + residual).astype(np.float32)
    vpt, threads = wide_shape(d)
    xn = O.rmsnorm_kernel_order(h_want, norm_w, 1e-5, 0, threads, vpt)
    q_want, s_want = O.quantize_i8_per_row(xn)
    h_out = np.empty((m, d), np.float32)
    xq_out = np.empty((2, m, d), np.int8)
    sx_out = np.empty((2, m), np.float32)
    counts = np.empty((tp, tp), np.uint32)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    check(lib().b200_selftest_tp_scatter(be._ctx, tp, rows, d, k, splits, tile, ptr(a_q), ptr(a_s), ptr(w_q), ptr(w_s),
                                         ptr(residual), ptr(norm_w), C.c_float(1e-5), ptr(h_out), ptr(xq_out), ptr(sx_out),
                                         ptr(counts)))
    assert np.array_equal(h_out, h_want)
    for i in range(2):
        assert np.array_equal(xq_out[i], q_want), i
        assert np.array_equal(sx_out[i], s_want), i
    assert np.all(counts == 1), counts
    assert not be.poisoned
