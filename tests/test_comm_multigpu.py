"""Symmetric-memory kernels on 2+ GPUs (all-reduce variants, reduce-scatter + optimizer, sparse rows, bounded wait)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("nvls", ["1", "0"])
def test_comm_kernels(nvls):
    import torch
    n = min(torch.cuda.device_count(), int(os.environ.get("AUTODIST_TEST_RANKS", "2")))
    env = dict(os.environ, AUTODIST_NVLS=nvls, NCCL_NVLS_ENABLE=nvls)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "integration", "run_comm_gpu.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ALL COMM CHECKS PASSED" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.gpu
@pytest.mark.multigpu
def test_fused_engine_matches_nccl_engine():
    import torch
    n = min(torch.cuda.device_count(), int(os.environ.get("AUTODIST_TEST_RANKS", "2")))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29612", os.path.join(HERE, "integration", "run_fused_gpu.py")]
    r = subprocess.run(cmd, env=dict(os.environ), capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "FUSED ENGINE CHECKS PASSED" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
