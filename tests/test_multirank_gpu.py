"""Two-GPU check of DOSyncBatchNorm2d against nn.SyncBatchNorm (skipped with fewer than two
GPUs).  The ranks are child processes started through torch.distributed.run; they leave between
steps with nothing in flight, and NCCL's in-switch reduction is off for them."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sync_batch_norm_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29541", os.path.join(here, "sync_bn_worker.py")],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "SYNCBN_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
