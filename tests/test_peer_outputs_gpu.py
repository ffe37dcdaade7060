"""KV-head-sharded decode with peer stores (infiniopPagedAttentionMultiOut + symmetric memory) on two
GPUs of one node: each rank stores its head slice into every rank's full output from inside the
attention kernels; a barrier replaces the all-gather.  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_two_ranks_fill_each_others_full_output():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                          "--master-port", "29533", str(ROOT / "tests" / "peer_runner.py")],
                         env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, (res.stdout + res.stderr)[-2000:]
    assert "ok=1" in res.stdout
