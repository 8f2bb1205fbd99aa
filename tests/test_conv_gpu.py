"""Implicit-GEMM convolution kernel against torch's conv2d in fp32 (forward, fused epilogue, input
gradient on the same kernel).  First GPU run of this kernel is opt-in."""
import os

import pytest
import torch
import torch.nn.functional as tF

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,n,hw", [
    (64, 64, 1, 1, 0, 1, 4, (56, 56)), (64, 64, 3, 1, 1, 1, 4, (56, 56)), (128, 128, 3, 2, 1, 1, 2, (28, 28)),
    (256, 72, 3, 1, 2, 2, 1, (15, 17)), (512, 2048, 1, 1, 0, 1, 2, (7, 7)), (64, 136, 3, 1, 1, 1, 3, (9, 5)),
])
def test_forward_matches_torch(cin, cout, k, stride, pad, dil, n, hw):
    from ferrotorch_b200.ops import conv as C

    torch.manual_seed(0)
    x = torch.randn(n, cin, *hw, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(cout, cin, k, k, device="cuda") / (cin * k * k) ** 0.5).to(torch.bfloat16)
    b = torch.randn(cout, device="cuda", dtype=torch.bfloat16)
    ref = tF.conv2d(x.float(), w.float(), b.float(), stride, pad, dil)
    prev = C.use_native_conv(True)
    try:
        assert C.supported(x, w, stride, pad, dil)
        y = C.conv2d(x, w, b, stride, pad, dil)
        res = torch.randn_like(y)
        z = C.conv2d(x, w, b, stride, pad, dil, residual=res, relu=True)
    finally:
        C.use_native_conv(prev)
    torch.testing.assert_close(y.float(), ref, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(z.float(), torch.relu(ref + res.float()), rtol=2e-2, atol=3e-2)


def test_backward_matches_torch():
    from ferrotorch_b200.ops import conv as C

    torch.manual_seed(1)
    x = torch.randn(2, 64, 14, 14, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(128, 64, 3, 3, device="cuda") / 24).to(torch.bfloat16)
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    torch.relu(tF.conv2d(xr, wr, None, 1, 1)).square().sum().backward()
    xn, wn = x.clone().requires_grad_(), w.clone().requires_grad_()
    prev = C.use_native_conv(True)
    try:
        C.conv2d(xn, wn, None, 1, 1, relu=True).float().square().sum().backward()
    finally:
        C.use_native_conv(prev)
    torch.testing.assert_close(xn.grad.float(), xr.grad, rtol=5e-2, atol=5e-2 * float(xr.grad.abs().max()))
    torch.testing.assert_close(wn.grad.float(), wr.grad, rtol=5e-2, atol=5e-2 * float(wr.grad.abs().max()))


def test_folded_resnet_on_the_kernel_matches_eval_model():
    from ferrotorch_b200.models import resnet as R
    from ferrotorch_b200.ops import conv as C

    torch.manual_seed(2)
    m = R.resnet50(num_classes=10).cuda().bfloat16().to(memory_format=torch.channels_last).eval()
    x = torch.randn(4, 3, 64, 64, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    fused = R.fuse_for_inference(m).cuda()
    with torch.no_grad():
        ref = m(x).float()
        prev = C.use_native_conv(True)
        try:
            out = fused(x).float()
        finally:
            C.use_native_conv(prev)
    assert torch.isfinite(out).all()
    torch.testing.assert_close(out, ref, rtol=0.1, atol=0.1 * float(ref.abs().max()))
