"""Failure detection on the device without faulting it: a wait on a flag that nothing raises runs
into its (short) limit, the kernel returns by itself, the host reads the error code from the
device status word and the CUDA context stays usable."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

FT_ERR_TIMEOUT_PEER = 4


def _wait(lib, flags, epoch, timeout_ms, world=2):
    from ferrotorch_b200 import _native

    rc = lib.ft_comm_wait(flags.data_ptr(), 0, 0, 1, 2, world, epoch, timeout_ms, 0,
                          torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "ft_comm_wait")


def test_wait_on_a_flag_nobody_raises_times_out_cleanly():
    from ferrotorch_b200 import _native
    from ferrotorch_b200.ops import functional as F
    from ferrotorch_b200.parallel import ddp  # noqa: F401  (declares the entry points)

    lib = _native.kernels()
    _native.device_status(0)                                   # clear anything left by earlier tests
    flags = torch.zeros(int(lib.ft_comm_flag_count(2)), device="cuda", dtype=torch.int32)
    torch.cuda.synchronize()
    t0 = time.time()
    _wait(lib, flags, epoch=1, timeout_ms=200)                 # peers 0 and 1 never signal epoch 1
    _wait(lib, flags, epoch=1, timeout_ms=200)                 # fails fast: the status word is already set
    torch.cuda.synchronize()
    dt = time.time() - t0
    assert 0.15 < dt < 0.39, "two waits took %.3f s (limit 0.2 s, second must not wait again)" % dt
    assert _native.device_status(0) == FT_ERR_TIMEOUT_PEER
    assert _native.device_status(0) == 0                       # read-and-clear

    # the context is alive: a kernel launched afterwards computes the right thing
    a = torch.randn(256, 128, device="cuda").to(torch.bfloat16)
    b = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    got = F.gemm_nt(a, b).float()
    assert (got - a.float() @ b.float().t()).abs().max().item() < 0.5

    # raised flags let the same wait through at once
    flags[:2] = 1
    t0 = time.time()
    _wait(lib, flags, epoch=1, timeout_ms=5000)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0 and _native.device_status(0) == 0


def test_comm_timeout_exception_from_status_word():
    from ferrotorch_b200 import _native
    from ferrotorch_b200.parallel.ddp import CommTimeout
    from ferrotorch_b200.parallel.tensor_parallel import TPContext

    tp = TPContext(None, torch.device("cuda", 0))
    lib = _native.kernels()
    flags = torch.zeros(int(lib.ft_comm_flag_count(2)), device="cuda", dtype=torch.int32)
    _wait(lib, flags, epoch=3, timeout_ms=100)
    torch.cuda.synchronize()
    with pytest.raises(CommTimeout):
        tp.check_status()
    tp.check_status()                                          # cleared by the read
