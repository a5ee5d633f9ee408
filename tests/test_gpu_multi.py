"""Fused compute+communication kernels over peer memory, on 2 GPUs of one box (child processes)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_comm_paths_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "workers", "fused_comm_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert "WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
