"""The allocation-free RMSNorm backward (``ft_rmsnorm_bwd_noalloc``, csrc/ft_noalloc.h).

Embedders that cannot allocate device memory at call time (memory-pool callbacks,
out-of-memory handlers, hosts with a memory budget fixed at start-up) get this entry point; its
scratch is a fixed array inside the library.  The test calls it through its exported C symbol,
twice in a row with different inputs (the array is shared between calls, so a stale-scratch bug
would show on the second call), and compares with the regular entry point that takes
caller-provided scratch.  Collected last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import ctypes

import pytest
import torch

from ferrotorch_b200 import _native

pytestmark = pytest.mark.gpu

vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


def _symbol():
    lib = ctypes.CDLL(str(_native.KERNELS_SO))
    fn = lib.ft_rmsnorm_bwd_noalloc
    fn.restype = ci
    fn.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
    return lib, fn


def _case(rows, H, seed, with_res):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g).to(torch.bfloat16)  # noqa: E731
    x, dy, w = r(rows, H), r(rows, H), r(H)
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, dy, w, rstd, (r(rows, H) if with_res else None)


def _regular(x, dy, w, rstd, dres):
    lib = _native.kernels()
    rows, H = x.shape
    dx, dw = torch.empty_like(x), torch.empty(H, device="cuda", dtype=torch.float32)
    scratch = torch.empty(lib.ft_rmsnorm_bwd_scratch_rows(rows, 0) * H, device="cuda", dtype=torch.float32)
    rc = lib.ft_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                            dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(),
                            scratch.data_ptr(), rows, H, 1, 0, torch.cuda.current_stream().cuda_stream)
    _native.check(rc, "ft_rmsnorm_bwd")
    return dx, dw


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    _, fn = _symbol()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, H, with_res) in enumerate([(1000, 4096, True), (77, 1024, False)]):
        x, dy, w, rstd, dres = _case(rows, H, seed=100 + call, with_res=with_res)
        want_dx, want_dw = _regular(x, dy, w, rstd, dres)
        dx, dw = torch.empty_like(x), torch.empty(H, device="cuda", dtype=torch.float32)
        allocated = torch.cuda.memory_allocated()
        if call == 1:
            # the first call did the once-per-device set-up; from here on the driver's own view of
            # free memory must not move either (it also sees a cudaMalloc made outside PyTorch)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(), rows, H, 1, 0, stream)
        assert rc == 0, _native.kernels().ft_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        # same kernel and the same per-row math; only the number of partial-sum rows differs
        assert torch.equal(dx, want_dx), "call %d: dx differs" % call
        err = (dw - want_dw).abs()
        tol = 2e-2 + 2e-2 * want_dw.abs()
        assert not (err > tol).any(), "call %d: dw max err %g" % (call, float(err.max()))


def test_noalloc_requires_its_device_to_be_current():
    # the entry point never switches devices: naming a device that is not current is an error
    lib, fn = _symbol()
    x = torch.zeros(2, 64, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    w = torch.ones(64, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(64, device="cuda")
    other = torch.cuda.current_device() + 1  # need not exist: the check comes before any launch
    rc = fn(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 2, 64,
            1, other, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    lib.ft_last_error.restype = ctypes.c_char_p
    assert b"must be the current device" in lib.ft_last_error()


def test_noalloc_rejects_sizes_beyond_the_fixed_scratch():
    lib, fn = _symbol()
    x = torch.zeros(2, 16384, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    w = torch.ones(16384, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(16384, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), dw.data_ptr(), 2,
            16384, 1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    lib.ft_last_error.restype = ctypes.c_char_p
    assert b"exceeds the fixed scratch" in lib.ft_last_error()
