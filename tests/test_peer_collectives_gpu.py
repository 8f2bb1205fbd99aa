"""Stand-alone NVLink peer-memory collectives against torch.distributed (2+ GPUs)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu
def test_peer_collectives_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", FT_COMM_TIMEOUT_MS="8000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29557", os.path.join(HERE, "peer_coll_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout


@pytest.mark.gpu
@pytest.mark.multigpu
def test_peer_collectives_all_gpus():
    import torch

    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    if n == 2:
        pytest.skip("covered by the two-GPU test")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", FT_COMM_TIMEOUT_MS="8000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
           "--master-addr", "127.0.0.1", "--master-port", "29558", os.path.join(HERE, "peer_coll_worker.py")]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout
