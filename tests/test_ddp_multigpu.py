"""Multi-GPU data parallelism: fused all-reduce + AdamW kernel vs NCCL baseline vs single process."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode: str, nproc: int):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "ddp_worker.py"), mode]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "ok" in proc.stdout


@pytest.mark.parametrize("mode", ["fused", "nccl", "fused_clip"])
def test_ddp_two_gpus(mode):
    _run(mode, 2)


@pytest.mark.parametrize("mode", ["fused", "fused_clip"])
def test_ddp_all_gpus(mode):
    n = torch.cuda.device_count()
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    if n == 2:
        pytest.skip("covered by the two-GPU test")
    _run(mode, n)
