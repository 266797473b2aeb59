"""Tensor-parallel decode on two GPUs of one box (skipped when fewer are visible)."""
import os
import subprocess
import sys
from pathlib import Path

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
