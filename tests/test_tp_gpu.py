"""Fused tensor-parallel GEMM kernels: world 1 on one GPU, world 2+ on several."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    if nproc == 1:
        cmd = [sys.executable, os.path.join(HERE, "tp_worker.py")]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout


@pytest.mark.gpu
def test_tp_kernels_world1():
    _run(1, 0)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp_kernels_world2():
    _run(2, 29541)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp_kernels_all_gpus():
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    if n == 2:
        pytest.skip("covered by the two-GPU test")
    _run(n, 29542)
