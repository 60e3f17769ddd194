"""Fused peer-memory paths against their NCCL twins on 2+ GPUs (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_paths_match_nccl_on_two_gpus():
    n = 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29631", os.path.join(here, "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_parallel_strategies_match_one_gpu_under_nccl():
    """Tensor / sequence / pipeline / interleaved-pipeline parallelism selected through ``Config``: 2 ranks against 1."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(here, "strategy_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "STRATEGIES_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
