"""Multi-GPU paths that need more than one device on the node (skipped otherwise).  Each test runs its ranks as child
processes, one per GPU, NVLS off; nothing here provokes a fault."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_shot_allreduce_equals_nccl():
    """exb_allreduce_oneshot over peer-mapped memory gives the NCCL sum on every rank, call after call, with identical
    bits on all ranks."""
    n = min(4, torch.cuda.device_count())
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29531", os.path.join(ROOT, "tests", "_oneshot_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0 and "ONESHOT_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
