"""Tensor-parallel training (sequence parallel, fused collectives in forward and backward):
world 1 on one GPU, world 2+ on several."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", FT_COMM_TIMEOUT_MS="10000")
    if nproc == 1:
        cmd = [sys.executable, os.path.join(HERE, "tp_train_worker.py")]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "tp_train_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout


@pytest.mark.gpu
def test_tp_training_world1():
    _run(1, 0)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_tp_training_world2():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2, 29551)
