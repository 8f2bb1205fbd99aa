"""Batch normalisation fused with the residual add and ReLU that follow it (channels-last bf16).

``batch_norm_act(x, bn, residual=None, relu=True)`` computes ``relu(bn(x) + residual)`` for an
``nn.BatchNorm2d`` ``bn`` (its weight / bias / running statistics / momentum / eps are used and
updated as ``bn(x)`` would).  On CUDA with bf16 channels-last activations the native kernels of
``csrc/bn_act.cu`` run: the activation tensor is read twice and written once in the forward, and
the backward recomputes the ReLU mask instead of storing it.  Anything else goes through the
plain torch composition, which is also the oracle for the tests.

The reference's BatchNorm2d is ferrotorch-nn/src/norm.rs:1389 (module) on the kernels of
ferrotorch-gpu/src/group_norm.rs:697-1095; it has no fused activation.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _native
from . import functional as F

_i, _ll, _f, _vp = _native._i, _native._ll, _native._f, _native._vp
_native.register_protos({
    "ft_bn_scratch_floats": (_ll, [_i]),
    "ft_bn_act_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _f, _f, _i, _ll, _i, _vp, _vp, _i, _vp]),
    "ft_bn_act_apply": (_i, [_vp, _vp, _vp, _vp, _i, _ll, _i, _i, _vp]),
    "ft_bn_act_bwd": (_i, [_vp, _vp, _vp, _vp, _i, _ll, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp]),
})

MAX_C = 2048


def _is_nhwc(t: torch.Tensor) -> bool:
    return t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last)


def _native_ok(x: torch.Tensor, residual) -> bool:
    if not (F.native_enabled() and x.is_cuda and x.dtype == torch.bfloat16):
        return False
    C = x.shape[1]
    if C % 8 or C > MAX_C or not (_is_nhwc(x) or x.dim() == 2 and x.is_contiguous()):
        return False
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or
                                 residual.stride() != x.stride()):
        return False
    return True


def _scratch(x: torch.Tensor) -> torch.Tensor:
    n = int(_native.kernels().ft_bn_scratch_floats(MAX_C))
    return F._get_scratch("bn_partial", n, x.device)


def _ptr(t):
    return t.data_ptr() if t is not None else None


class _BatchNormActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, running_mean, running_var, momentum, eps, relu):
        C = x.shape[1]
        R = x.numel() // C
        y = torch.empty_like(x)
        stats = torch.empty(4 * C, device=x.device, dtype=torch.float32)
        affine_f32 = int(weight is not None and weight.dtype == torch.float32)
        running_f32 = int(running_mean is not None and running_mean.dtype == torch.float32)
        rc = _native.kernels().ft_bn_act_fwd(
            x.data_ptr(), _ptr(residual), y.data_ptr(), _ptr(weight), _ptr(bias), affine_f32, _ptr(running_mean),
            _ptr(running_var), running_f32, float(momentum), float(eps), int(relu), R, C, stats.data_ptr(),
            _scratch(x).data_ptr(), F._dev(x), F._stream())
        _native.check(rc, "ft_bn_act_fwd")
        keep_y = relu and residual is not None
        ctx.save_for_backward(x, y if keep_y else x.new_empty(0), stats)
        ctx.cfg = (bool(relu), residual is not None, keep_y)
        ctx.affine = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, stats = ctx.saved_tensors
        relu, has_res, keep_y = ctx.cfg
        weight, bias = ctx.affine
        C = x.shape[1]
        R = x.numel() // C
        if dy.stride() != x.stride():
            dy = dy.contiguous(memory_format=torch.channels_last) if x.dim() == 4 else dy.contiguous()
        dx = torch.empty_like(x)
        # without a ReLU the residual branch's gradient is dy itself
        dres = torch.empty_like(x) if (has_res and relu) else None
        coef = torch.empty(3 * C, device=x.device, dtype=torch.float32)
        need_w = weight is not None and ctx.needs_input_grad[1]
        need_b = bias is not None and ctx.needs_input_grad[2]
        # the flat-arena trainer owns the gradients: the finalize kernel adds into its arena
        wg = getattr(weight, "main_grad", None) if need_w else None
        bg = getattr(bias, "main_grad", None) if need_b else None
        arena = (wg is not None or not need_w) and (bg is not None or not need_b) and (need_w or need_b) and \
            all(g is None or g.dtype in (torch.bfloat16, torch.float32) for g in (wg, bg)) and \
            (wg is None or bg is None or wg.dtype == bg.dtype)
        dgdb = None
        if arena:
            gp, bp = _ptr(wg), _ptr(bg)
            kind = 1 if (wg if wg is not None else bg).dtype == torch.bfloat16 else 2
        else:
            dgdb = torch.empty(2 * C, device=x.device, dtype=torch.float32)
            gp, bp, kind = dgdb.data_ptr(), dgdb.data_ptr() + 4 * C, 0
        rc = _native.kernels().ft_bn_act_bwd(
            x.data_ptr(), dy.data_ptr(), y.data_ptr() if keep_y else None, stats.data_ptr(), int(relu), R, C,
            dx.data_ptr(), _ptr(dres), gp, bp, kind, coef.data_ptr(), _scratch(x).data_ptr(), F._dev(x), F._stream())
        _native.check(rc, "ft_bn_act_bwd")
        dw = db = None
        if arena:
            for p in (weight if need_w else None, bias if need_b else None):
                hook = getattr(p, "grad_ready_hook", None) if p is not None else None
                if hook is not None:
                    hook(p)
        else:
            dw = dgdb[:C].to(weight.dtype) if need_w else None
            db = dgdb[C:].to(bias.dtype) if need_b else None
        if has_res:
            dres = dres if relu else dy
        return dx, dw, db, (dres if has_res else None), None, None, None, None, None


def batch_norm_act(x: torch.Tensor, bn: nn.modules.batchnorm._BatchNorm, residual: torch.Tensor | None = None,
                   relu: bool = True) -> torch.Tensor:
    """``relu(bn(x) + residual)`` (``residual`` and ``relu`` optional) with ``bn``'s parameters."""
    use_batch_stats = bn.training or not bn.track_running_stats
    if _native_ok(x, residual):
        if use_batch_stats:
            momentum = bn.momentum
            if bn.track_running_stats and bn.training:
                if bn.num_batches_tracked is not None:
                    bn.num_batches_tracked.add_(1)
                if momentum is None:
                    momentum = 1.0 / float(bn.num_batches_tracked)
            track = bn.track_running_stats and bn.training
            return _BatchNormActFn.apply(x, bn.weight, bn.bias, residual, bn.running_mean if track else None,
                                         bn.running_var if track else None, momentum or 0.0, bn.eps, relu)
        if not torch.is_grad_enabled() or not (x.requires_grad or (bn.weight is not None and bn.weight.requires_grad)):
            C = x.shape[1]
            inv = torch.rsqrt(bn.running_var.float() + bn.eps)
            scale = inv * (bn.weight.float() if bn.weight is not None else 1.0)
            shift = (bn.bias.float() if bn.bias is not None else 0.0) - bn.running_mean.float() * scale
            ss = torch.cat([scale, shift.expand_as(scale)]).contiguous()
            y = torch.empty_like(x)
            rc = _native.kernels().ft_bn_act_apply(x.data_ptr(), _ptr(residual), y.data_ptr(), ss.data_ptr(), int(relu),
                                                   x.numel() // C, C, F._dev(x), F._stream())
            _native.check(rc, "ft_bn_act_apply")
            return y
    out = nn.modules.batchnorm._BatchNorm.forward(bn, x)
    if residual is not None:
        out = out + residual
    return torch.relu(out) if relu else out


class BatchNormAct2d(nn.BatchNorm2d):
    """``nn.BatchNorm2d`` whose forward also applies the ReLU (and an optional residual add)."""

    def __init__(self, num_features: int, relu: bool = True, **kw):
        super().__init__(num_features, **kw)
        self.relu = relu

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:  # noqa: D102
        return batch_norm_act(x, self, residual, self.relu)
