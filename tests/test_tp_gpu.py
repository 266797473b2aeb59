"""Tensor-parallel decode on two GPUs of one box (skipped when fewer are visible)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("exchange", ["1", "0"])
def test_two_rank_tensor_parallel_decode_matches_the_cpu_decoder(exchange):
    """exchange 1: the row-parallel outputs are finished over the CUDA-IPC mapped peer blocks (falls back to
    ncclAllReduce by itself where IPC is not available); exchange 0: ncclAllReduce is forced."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", B200_TP_EXCHANGE=exchange)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29731", str(ROOT / "tests" / "multi" / "tp_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-3000:]
    # the path that ran is the path that was asked for: a silent fall-back to ncclAllReduce would leave the finish
    # kernel (peer sum, residual, RMSNorm, int8 delivery) unchecked
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
    assert r.returncode == 0 and "TP_OK" in r.stdout, r.stdout[-3000:]


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
