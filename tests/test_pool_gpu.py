"""NHWC max-pool kernels against torch on the device (first GPU run is opt-in)."""
import os

import pytest
import torch
import torch.nn.functional as tF

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c,k,s,p,hw", [(64, 3, 2, 1, (112, 112)), (8, 2, 2, 0, (9, 7)), (72, 3, 1, 1, (13, 11)), (16, 5, 2, 2, (31, 33))])
def test_forward_backward_match_torch(c, k, s, p, hw):
    from ferrotorch_b200.ops import pool as P

    torch.manual_seed(0)
    x = torch.randn(3, c, *hw, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_()
    ref = tF.max_pool2d(x, k, s, p)
    gy = torch.randn_like(ref)
    ref.backward(gy)
    gref, x.grad = x.grad, None
    prev = P.use_native_pool(True)
    try:
        assert P.supported(x, k, s, p)
        y = P.max_pool2d(x, k, s, p)
        y.backward(gy)
    finally:
        P.use_native_pool(prev)
    assert torch.equal(y, ref)
    torch.testing.assert_close(x.grad.float(), gref.float(), rtol=2e-2, atol=2e-2)      # sums of up to 4 bf16 terms: order may differ
