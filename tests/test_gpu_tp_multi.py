"""Fused row-parallel exchange across real GPUs (skipped on a single-GPU box): one process per GPU,
NVLS off, every device-side wait bounded."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_row_parallel_matches_nccl_and_single_gpu():
    world = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "TP_WORKER_OK" in r.stdout, r.stdout[-2000:]
