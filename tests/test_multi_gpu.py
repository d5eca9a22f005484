"""The multi-GPU paths on real GPUs: column-sharded GEMM, the column all-gather (serial and by row blocks), the
sharded host-memory entry and the FLOP-balanced grouped split, one process per GPU over NCCL.  Skipped on a machine
with fewer than two GPUs (the host logic is covered on CPU by tests/test_dist_gloo.py)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_paths_agree_with_one_gpu():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "multi_gpu_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    for r in range(world):
        assert "rank %d ok" % r in res.stdout
