"""Fused batch norm (+ residual, + ReLU) kernels against the fp32 torch composition."""
import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


def _case(N, C, H, W, residual, relu, seed=0):
    from ferrotorch_b200.ops.batchnorm import batch_norm_act

    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    x = (torch.randn(N, C, H, W, generator=g) * 1.5 + 0.3).to(torch.bfloat16).to(dev).contiguous(memory_format=torch.channels_last)
    res = torch.randn(N, C, H, W, generator=g).to(torch.bfloat16).to(dev).contiguous(memory_format=torch.channels_last) if residual else None
    dy = torch.randn(N, C, H, W, generator=g).to(torch.bfloat16).to(dev).contiguous(memory_format=torch.channels_last)
    bn = nn.BatchNorm2d(C).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        bn.weight.copy_(torch.rand(C, generator=g) + 0.5)
        bn.bias.copy_(torch.randn(C, generator=g) * 0.2)
    ref_bn = nn.BatchNorm2d(C).to(dev).float()
    with torch.no_grad():
        ref_bn.weight.copy_(bn.weight.float())
        ref_bn.bias.copy_(bn.bias.float())

    xs = x.clone().requires_grad_()
    rs = res.clone().requires_grad_() if residual else None
    y = batch_norm_act(xs, bn, rs, relu)
    assert y.is_contiguous(memory_format=torch.channels_last) and y.dtype == torch.bfloat16
    y.backward(dy)

    xr = x.float().requires_grad_()
    rr = res.float().requires_grad_() if residual else None
    o = ref_bn(xr)
    if residual:
        o = o + rr
    if relu:
        o = torch.relu(o)
    o.backward(dy.float())

    def close(a, b, tol, what):
        err = (a.float() - b.float()).abs().max().item()
        scale = max(1.0, b.float().abs().max().item())
        assert err <= tol * scale, "%s: err %g (scale %g) C=%d res=%s relu=%s" % (what, err, scale, C, residual, relu)

    close(y, o, 1.2e-2, "y")
    close(bn.running_mean, ref_bn.running_mean, 1e-2, "running_mean")
    close(bn.running_var, ref_bn.running_var, 1e-2, "running_var")
    # elements whose pre-activation is within bf16 rounding of zero may flip the mask: compare in aggregate
    d = (xs.grad.float() - xr.grad).abs()
    assert d.mean().item() < 2e-3 * max(1.0, xr.grad.abs().mean().item()) + 1e-3, "dx mean err %g" % d.mean().item()
    assert (d > 0.1 * max(1.0, xr.grad.abs().max().item())).float().mean().item() < 1e-3, "dx outliers"
    if residual:
        dr = (rs.grad.float() - rr.grad).abs()
        assert (dr > 1e-2).float().mean().item() < 1e-3, "dres"
    R = N * H * W
    close(bn.weight.grad, ref_bn.weight.grad, 2e-2 + 2e-3 * R ** 0.5 / max(1.0, ref_bn.weight.grad.abs().max().item()), "dgamma")
    close(bn.bias.grad, ref_bn.bias.grad, 2e-2 + 2e-3 * R ** 0.5 / max(1.0, ref_bn.bias.grad.abs().max().item()), "dbeta")


@pytest.mark.parametrize("C", [64, 256, 2048, 24])
@pytest.mark.parametrize("residual,relu", [(False, True), (True, True), (False, False), (True, False)])
def test_bn_act_matches_torch(C, residual, relu):
    _case(3, C, 13, 11, residual, relu)


def test_bn_act_large_rows():
    _case(16, 64, 56, 56, True, True, seed=1)


def test_bn_eval_mode_and_launch_count():
    from ferrotorch_b200 import _native
    from ferrotorch_b200.ops.batchnorm import batch_norm_act

    bn = nn.BatchNorm2d(32).cuda().to(torch.bfloat16).eval()
    with torch.no_grad():
        bn.running_mean.normal_()
        bn.running_var.uniform_(0.5, 2.0)
    x = torch.randn(4, 32, 7, 7, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    n0 = _native.launch_count()
    with torch.no_grad():
        y = batch_norm_act(x, bn, None, True)
        ref = torch.relu(nn.functional.batch_norm(x.float(), bn.running_mean.float(), bn.running_var.float(),
                                                  bn.weight.float(), bn.bias.float(), False, 0.0, bn.eps))
    assert _native.launch_count() == n0 + 1
    assert (y.float() - ref).abs().max().item() < 3e-2


def test_resnet_uses_fused_bn_and_matches_fp32_as_well_as_torch_bf16():
    import copy

    from ferrotorch_b200 import _native
    from ferrotorch_b200.models.resnet import resnet18
    from ferrotorch_b200.ops import functional as F

    torch.manual_seed(0)
    ref = resnet18(num_classes=10).cuda().to(memory_format=torch.channels_last)          # fp32 oracle
    m = copy.deepcopy(ref).to(torch.bfloat16)
    x = torch.randn(16, 3, 96, 96, device="cuda").contiguous(memory_format=torch.channels_last)
    wsum = torch.randn(16, 10, device="cuda")

    def run(model, inp, native):
        model.zero_grad()
        old = F.set_native(native)
        try:
            out = model(inp)
            (out.float() * wsum).sum().backward()
        finally:
            F.set_native(old)
        return out.float().detach(), [p.grad.float().clone() for p in model.parameters()]

    o_ref, g_ref = run(ref, x, False)
    n0 = _native.launch_count()
    o_nat, g_nat = run(m, x.to(torch.bfloat16), True)
    assert _native.launch_count() - n0 >= 6 * 20           # 20 batch norms, 3 launches each way
    o_tor, g_tor = run(m, x.to(torch.bfloat16), False)

    def rel(gs):
        num = sum(((a - b) ** 2).sum() for a, b in zip(gs, g_ref))
        den = sum((b ** 2).sum() for b in g_ref)
        return float(num / den) ** 0.5

    e_nat, e_tor = rel(g_nat), rel(g_tor)
    assert e_nat < 1.5 * e_tor + 0.02, "gradient error vs fp32: native %g, torch bf16 %g" % (e_nat, e_tor)
    eo_nat = float((o_nat - o_ref).norm() / o_ref.norm())
    eo_tor = float((o_tor - o_ref).norm() / o_ref.norm())
    assert eo_nat < 1.5 * eo_tor + 0.02, "output error vs fp32: native %g, torch bf16 %g" % (eo_nat, eo_tor)


def test_bn_grads_accumulate_into_arena():
    from ferrotorch_b200.ops.batchnorm import batch_norm_act

    bn = nn.BatchNorm2d(64).cuda().to(torch.bfloat16)
    x = torch.randn(8, 64, 9, 9, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    dy = torch.randn_like(x)
    xs = x.clone().requires_grad_()
    batch_norm_act(xs, bn, None, True).backward(dy)
    gw, gb = bn.weight.grad.float().clone(), bn.bias.grad.float().clone()
    bn.weight.grad = bn.bias.grad = None
    for dt in (torch.float32, torch.bfloat16):
        bn.weight.main_grad = torch.ones(64, device="cuda", dtype=dt)
        bn.bias.main_grad = torch.ones(64, device="cuda", dtype=dt)
        seen = []
        bn.weight.grad_ready_hook = bn.bias.grad_ready_hook = lambda p: seen.append(p)
        xs = x.clone().requires_grad_()
        batch_norm_act(xs, bn, None, True).backward(dy)
        assert bn.weight.grad is None and bn.bias.grad is None and len(seen) == 2
        tol = 0.01 if dt == torch.float32 else 0.05     # the reference gradients were rounded to bf16
        assert (bn.weight.main_grad.float() - 1 - gw).abs().max().item() <= tol * max(1.0, gw.abs().max().item()) + 0.02
        assert (bn.bias.main_grad.float() - 1 - gb).abs().max().item() <= tol * max(1.0, gb.abs().max().item()) + 0.02
