"""NHWC max pooling: the kernels' window functions, run on the CPU through the library's host
entry point, against torch's max_pool2d and its gradient; fallbacks."""
import pytest
import torch
import torch.nn.functional as tF

from ferrotorch_b200 import _native
from ferrotorch_b200.ops import pool as P

needs_lib = pytest.mark.skipif(_native.kernels(required=False) is None, reason="kernel library not built")


@needs_lib
@pytest.mark.parametrize("k,s,p,hw", [(3, 2, 1, (9, 10)), (2, 2, 0, (8, 6)), (3, 1, 1, (5, 7)), (3, 3, 0, (10, 9)), ((3, 2), 2, (1, 0), (7, 8)),
                                      (5, 2, 2, (11, 12)), (2, 1, 1, (4, 4))])
def test_forward_and_backward_match_torch(k, s, p, hw):
    torch.manual_seed(0)
    x = torch.randn(2, 8, *hw, requires_grad=True)
    ref = tF.max_pool2d(x, k, s, p)
    gy = torch.randn_like(ref)
    ref.backward(gy)
    y, arg, gx = P.max_pool2d_host(x, k, s, p, gy)
    assert torch.equal(y, ref.detach()) and torch.equal(gx, x.grad)
    kk = (k, k) if isinstance(k, int) else k
    assert int(arg.max()) < kk[0] * kk[1]


@needs_lib
def test_ties_nan_and_bad_geometry():
    x = torch.zeros(1, 8, 4, 4, requires_grad=True)                 # all ties: the first tap of every window wins, as in torch
    ref = tF.max_pool2d(x, 2, 2)
    ref.backward(torch.ones_like(ref))
    y, arg, gx = P.max_pool2d_host(x, 2, 2, 0, torch.ones_like(ref))
    assert torch.equal(gx, x.grad) and int(arg.max()) == 0
    z = torch.randn(1, 8, 4, 4)
    z[0, 3, 1, 1] = float("nan")
    y, _ = P.max_pool2d_host(z, 2, 2)
    assert torch.isnan(y[0, 3, 0, 0]) and torch.equal(torch.isnan(y), torch.isnan(tF.max_pool2d(z, 2, 2)))
    with pytest.raises(_native.NativeError):
        P.max_pool2d_host(z, 2, 2, 2)                               # padding larger than half the window


def test_fallback_and_module():
    x = torch.randn(2, 8, 9, 9, requires_grad=True)
    prev = P.use_native_pool(True)
    try:
        assert not P.supported(x, 3, 2, 1)                          # CPU tensor: torch serves it
        y = P.MaxPool2d(3, 2, 1)(x)
    finally:
        P.use_native_pool(prev)
    torch.testing.assert_close(y, tF.max_pool2d(x, 3, 2, 1))
    y.sum().backward()
    assert x.grad is not None and torch.equal(P.max_pool2d(x, 2), tF.max_pool2d(x, 2))
