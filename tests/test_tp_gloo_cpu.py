"""Tensor-parallel host logic with two gloo ranks on the CPU (no GPU): shard plan and the cross-rank sum."""
import subprocess
import sys
from pathlib import Path

import pytest

from fandhe_ai_b200._lib import BackendError
from fandhe_ai_b200.decoder import W_DOWN, W_EMBED, W_QKV, DecoderConfig, shard_plan

ROOT = Path(__file__).resolve().parents[1]


def test_two_gloo_ranks_shard_and_sum():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29733", str(ROOT / "tests" / "multi" / "tp_gloo_worker.py")]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0 and "TP_GLOO_OK" in r.stdout, r.stdout[-3000:]


def test_shard_plan_of_the_8b_shape_at_eight_ranks():
    cfg = DecoderConfig(32, 4096, 32, 8, 128, 14336, 128256, tp_rank=3, tp_size=8)
    qkv = shard_plan(cfg, W_QKV)
    assert (qkv["rows"], qkv["cols"]) == (6144, 4096)
    assert qkv["row_ranges"] == [(3 * 512, 512), (4096 + 3 * 128, 128), (5120 + 3 * 128, 128)]   # 4 q heads, 1 k, 1 v
    down = shard_plan(cfg, W_DOWN)
    assert down["row_ranges"] == [(0, 4096)] and (down["col_start"], down["col_count"]) == (3 * 1792, 1792)
    with pytest.raises(BackendError):
        shard_plan(DecoderConfig(32, 4096, 32, 8, 128, 14336, 128256, tp_rank=0, tp_size=3), W_QKV)   # 8 kv heads / 3
    with pytest.raises(BackendError):
        shard_plan(cfg, W_EMBED)
