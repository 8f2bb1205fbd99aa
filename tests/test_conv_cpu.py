"""Convolution binding: the kernel's tile arithmetic restated on the CPU against torch's conv2d,
the flipped-filter identity the input gradient relies on, fallbacks and the module rewrite."""
import pytest
import torch
import torch.nn.functional as tF

from ferrotorch_b200.ops import conv as C


@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,hw", [
    (64, 16, 3, 1, 1, 1, (9, 7)), (128, 8, 3, 2, 1, 1, (10, 11)), (64, 24, 1, 1, 0, 1, (5, 6)),
    (64, 8, 1, 2, 0, 1, (8, 8)), (64, 8, 3, 1, 2, 2, (9, 9)), (64, 8, 7, 2, 3, 1, (15, 13)), (4, 8, 3, 1, (1, 0), 1, (6, 6)),
])
def test_tile_arithmetic_equals_conv2d(cin, cout, k, stride, pad, dil, hw):
    torch.manual_seed(0)
    x, w = torch.randn(3, cin, *hw), torch.randn(cout, cin, k, k) * 0.1
    ref = tF.conv2d(x, w, None, stride, pad, dil)
    got = C.implicit_gemm_reference(x, w, stride, pad, dil)
    assert got.shape == ref.shape
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("k,pad,dil", [(3, 1, 1), (3, 0, 1), (1, 0, 1), (3, 2, 2), (5, 2, 1)])
def test_input_gradient_is_a_convolution_with_the_flipped_filter(k, pad, dil):
    torch.manual_seed(1)
    x, w = torch.randn(2, 6, 9, 8), torch.randn(5, 6, k, k)
    gy = torch.randn_like(tF.conv2d(x, w, None, 1, pad, dil))
    ref = torch.nn.grad.conv2d_input(x.shape, w, gy, 1, pad, dil)
    bp = dil * (k - 1) - pad
    wt = w.flip(2, 3).transpose(0, 1)
    torch.testing.assert_close(tF.conv2d(gy, wt, None, 1, bp, dil), ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(C.implicit_gemm_reference(gy, wt, 1, bp, dil), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("stride,pad,dil", [(1, 1, 1), (2, 1, 1), (1, 2, 2), (2, 0, 1), (1, (1, 2), 1)])
def test_shifted_row_arithmetic_equals_conv2d(stride, pad, dil):
    torch.manual_seed(3)
    x, w = torch.randn(2, 8, 9, 10), torch.randn(4, 8, 3, 3)
    torch.testing.assert_close(C.shift_conv_reference(x, w, stride, pad, dil), tF.conv2d(x, w, None, stride, pad, dil),
                               rtol=1e-4, atol=1e-4)


def _grads_against_torch(fn, cin, cout, k, stride, pad, dil, hw):
    torch.manual_seed(cin + cout + k + stride)
    x = torch.randn(2, cin, *hw).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(cout, cin, k, k) / (cin * k * k) ** 0.5).to(torch.bfloat16)
    b = torch.randn(cout).to(torch.bfloat16)
    xr, wr, br = x.float().requires_grad_(), w.float().requires_grad_(), b.float().requires_grad_()
    ref = tF.conv2d(xr, wr, br, stride, pad, dil)
    gy = torch.randn_like(ref)
    ref.backward(gy)
    xn, wn, bn = x.clone().requires_grad_(), w.clone().requires_grad_(), b.clone().requires_grad_()
    y = fn(xn, wn, bn)
    y.backward(gy.to(y.dtype))
    for got, want, what in ((y, ref, "y"), (xn.grad, xr.grad, "dx"), (wn.grad, wr.grad, "dw"), (bn.grad, br.grad, "db")):
        err = float((got.float() - want.detach()).abs().max() / (want.detach().abs().max() + 1e-6))
        assert err < 1e-2, "%s: relative error %.3g" % (what, err)


# The autograd functions run on CPU tensors through torch restatements of the layout kernels and
# of the shifted-row GEMMs, so the grid / parity-plane / tap-shift arithmetic of all three
# gradients is checked here against torch's convolution.
@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,hw", [
    (64, 64, 3, 1, 1, 1, (9, 7)), (64, 128, 3, 2, 1, 1, (10, 11)), (64, 64, 3, 2, 1, 1, (8, 8)),
    (64, 64, 3, 1, 2, 2, (9, 9)), (64, 64, 7, 2, 3, 1, (15, 13)), (64, 64, 5, 2, 2, 1, (11, 12)),
    (64, 64, 3, 1, 0, 1, (7, 7)), (64, 64, 3, 2, 0, 1, (9, 10)), (64, 64, 2, 2, 0, 1, (8, 8)), (64, 64, 3, 1, (1, 2), 1, (6, 9)),
])
def test_shift_conv_function_gradients(cin, cout, k, stride, pad, dil, hw):
    _grads_against_torch(lambda x, w, b: C._ShiftConv.apply(x, w, b, stride, C._pair(pad), dil, False),
                         cin, cout, k, stride, pad, dil, hw)


@pytest.mark.parametrize("stride", [1, 2])
def test_pointwise_conv_function_gradients(stride):
    _grads_against_torch(lambda x, w, b: C._PointwiseConv.apply(x, w, b, stride, False), 64, 72, 1, stride, 0, 1, (8, 7))


def test_im2col_conv_function_gradients():
    _grads_against_torch(lambda x, w, b: C._Im2colConv.apply(x, w, b, 2, (3, 3), 1, False), 3, 16, 7, 2, 3, 1, (15, 13))


def test_native_path_selection():
    x = torch.empty(1, 64, 8, 8, dtype=torch.bfloat16)
    assert C.native_path(x, torch.empty(64, 64, 3, 3), 1, 1, 1) is None            # CPU tensors: library
    g = C.ShiftGeometry(2, 56, 56, 3, 3, 2, 1, 1, 1)
    assert (g.Hp, g.Wp, g.planes, g.Ho, g.Wo) == (29, 29, 4, 28, 28) and g.x_rows == 4 * g.P
    assert g.shifts()[4] == 3 * g.P and g.shifts()[8] == 29 + 1                     # tap (1,1): plane 3; tap (2,2): plane 0
    g1 = C.ShiftGeometry(1, 7, 7, 3, 3, 1, 1, 1, 1)
    assert g1.shifts() == [0, 1, 2, 9, 10, 11, 18, 19, 20]


def test_fallback_module_and_rewrite():
    torch.manual_seed(2)
    net = torch.nn.Sequential(torch.nn.Conv2d(8, 16, 3, 1, 1), torch.nn.ReLU(), torch.nn.Conv2d(16, 4, 1, bias=False))
    x = torch.randn(2, 8, 6, 6, requires_grad=True)
    ref = net(x)
    keys = list(net.state_dict())
    assert C.convert_convs(net) == 2 and isinstance(net[0], C.IgemmConv2d) and list(net.state_dict()) == keys
    prev = C.use_native_conv(True)                              # CPU tensors: not supported, so torch runs
    try:
        out = net(x)
        assert not C.supported(x, net[0].weight, 1, 1, 1)
    finally:
        C.use_native_conv(prev)
    torch.testing.assert_close(out, ref)
    out.sum().backward()
    assert x.grad is not None
    res = torch.randn(2, 16, 6, 6)
    fused = net[0](x, residual=res, relu=True)
    torch.testing.assert_close(fused, torch.relu(tF.conv2d(x, net[0].weight, net[0].bias, 1, 1) + res))
    assert C.out_size(224, 7, 2, 3, 1) == 112 and C.out_size(56, 3, 1, 1, 1) == 56


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the failure mode of a box without a GPU")
def test_binding_marshals_arguments_and_fails_with_the_library_error(monkeypatch):
    from ferrotorch_b200 import _native
    from ferrotorch_b200.ops import functional as F

    if _native.kernels(required=False) is None:
        pytest.skip("kernel library not built")
    monkeypatch.setattr(F, "_dev", lambda t: 0)
    monkeypatch.setattr(F, "_stream", lambda: None)
    x = torch.randn(1, 64, 8, 8).bfloat16().contiguous(memory_format=torch.channels_last)
    w = torch.randn(8, 64, 3, 3).bfloat16()
    with pytest.raises(_native.NativeError, match="ft_conv2d_fprop_nhwc"):    # reached the C entry point: no ctypes TypeError
        C._fprop(x, w, None, None, 1, (1, 1), 1, False)


@pytest.mark.parametrize("cin,cout,k,stride,pad,dil,hw", [
    (64, 8, 3, 1, 1, 1, (7, 6)), (128, 16, 3, 2, 1, 1, (9, 10)), (64, 8, 1, 2, 0, 1, (8, 8)), (64, 8, 3, 1, 2, 2, (9, 9)),
    (64, 8, 7, 2, 3, 1, (13, 15)), (192, 8, 3, 1, (1, 0), 1, (5, 6)),
])
def test_the_kernels_own_index_functions_reproduce_conv2d(cin, cout, k, stride, pad, dil, hw):
    """The gather offsets come from the functions the CUDA kernel itself calls (compiled for host
    too): assembling the implicit matrix from them and multiplying by the OHWI filter must give
    ``conv2d``."""
    from ferrotorch_b200 import _native

    if _native.kernels(required=False) is None:
        pytest.skip("kernel library not built")
    torch.manual_seed(0)
    n = 2
    x, w = torch.randn(n, cin, *hw), torch.randn(cout, cin, k, k) * 0.1
    off = C.kernel_gather_offsets(n, hw[0], hw[1], cin, k, k, stride, pad, dil)
    flat = torch.cat([x.permute(0, 2, 3, 1).reshape(-1), torch.zeros(64)])          # NHWC, plus a zero run for padding taps
    idx = torch.where(off >= 0, off, torch.full_like(off, flat.numel() - 64))
    A = flat[(idx[..., None] + torch.arange(64)).reshape(off.shape[0], -1)]           # [M, K]
    ref = torch.nn.functional.conv2d(x, w, None, stride, pad, dil)
    got = (A @ w.permute(0, 2, 3, 1).reshape(cout, -1).t()).reshape(n, ref.shape[2], ref.shape[3], cout).permute(0, 3, 1, 2)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-4)
    assert (off % 64 == 0)[off >= 0].all()                                           # every run starts on a 128-byte boundary
