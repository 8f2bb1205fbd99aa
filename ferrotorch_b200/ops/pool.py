"""Max pooling on NHWC bf16 activations (``csrc/pool_nhwc.cu``): forward writes the winning tap of
every window beside the output, backward gathers from the windows that cover each input pixel --
deterministic, no atomics, neither the input nor a comparison needed.  The reference pools forward
on the GPU in NCHW f32 and backward on the host (ferrotorch-gpu/src/kernels.rs:11265, 11410).

Tensors keep torch's logical NCHW shape in ``channels_last`` memory format.  The native path needs
CUDA, bf16 and ``C % 8 == 0``; it is on by default (:func:`use_native_pool` or ``FT_POOL_NHWC=0`` switch it off) and
``torch.nn.functional.max_pool2d`` serves everything else.  :func:`max_pool2d_host` runs the
kernels' window functions on the CPU (the library's host entry point) for the tests.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as tF

from .. import _native
from . import functional as F
from .conv import _pair

_i, _vp = _native._i, _native._vp
_native.register_protos({
    "ft_maxpool2d_fwd_nhwc": (_i, [_vp] * 3 + [_i] * 10 + [_vp]),
    "ft_maxpool2d_bwd_nhwc": (_i, [_vp] * 3 + [_i] * 10 + [_vp]),
    "ft_maxpool2d_host": (_i, [_vp] * 5 + [_i] * 9),
})

_enabled = os.environ.get("FT_POOL_NHWC", "1") != "0"
CL = torch.channels_last


def use_native_pool(on: bool = True) -> bool:
    global _enabled
    prev, _enabled = _enabled, bool(on)
    return prev


def supported(x: torch.Tensor, kernel_size, stride, padding) -> bool:
    k, s, p = _pair(kernel_size), _pair(stride), _pair(padding)
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 4 and x.shape[1] % 8 == 0 and s[0] == s[1]
            and 2 * p[0] <= k[0] and 2 * p[1] <= k[1] and k[0] * k[1] < 255
            and x.shape[2] + 2 * p[0] >= k[0] and x.shape[3] + 2 * p[1] >= k[1])


def _out(size, k, s, p):
    return (size + 2 * p - k) // s + 1


class _MaxPoolNhwc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p):
        N, C, H, W = x.shape
        x = x.contiguous(memory_format=CL)
        Ho, Wo = _out(H, k[0], s, p[0]), _out(W, k[1], s, p[1])
        y = torch.empty((N, C, Ho, Wo), device=x.device, dtype=x.dtype, memory_format=CL)
        arg = torch.empty((N, Ho, Wo, C), device=x.device, dtype=torch.uint8)
        rc = _native.kernels().ft_maxpool2d_fwd_nhwc(x.data_ptr(), y.data_ptr(), arg.data_ptr(), N, H, W, C, k[0], k[1], s,
                                                     p[0], p[1], F._dev(x), F._stream())
        _native.check(rc, "ft_maxpool2d_fwd_nhwc")
        ctx.save_for_backward(arg)
        ctx.geom = (N, C, H, W, k, s, p)
        return y

    @staticmethod
    def backward(ctx, gy):
        (arg,) = ctx.saved_tensors
        N, C, H, W, k, s, p = ctx.geom
        gy = gy.contiguous(memory_format=CL)
        gx = torch.empty((N, C, H, W), device=gy.device, dtype=gy.dtype, memory_format=CL)
        rc = _native.kernels().ft_maxpool2d_bwd_nhwc(gy.data_ptr(), arg.data_ptr(), gx.data_ptr(), N, H, W, C, k[0], k[1], s,
                                                     p[0], p[1], F._dev(gy), F._stream())
        _native.check(rc, "ft_maxpool2d_bwd_nhwc")
        return gx, None, None, None


def max_pool2d(x: torch.Tensor, kernel_size, stride=None, padding=0) -> torch.Tensor:
    stride = kernel_size if stride is None else stride
    if _enabled and supported(x, kernel_size, stride, padding):
        return _MaxPoolNhwc.apply(x, _pair(kernel_size), _pair(stride)[0], _pair(padding))
    return tF.max_pool2d(x, kernel_size, stride, padding)


class MaxPool2d(torch.nn.MaxPool2d):
    """``nn.MaxPool2d`` that takes the NHWC kernel when it is switched on and the options allow it
    (no dilation, no ceil mode, no returned indices)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.dilation in (1, (1, 1)) and not self.ceil_mode and not self.return_indices:
            return max_pool2d(x, self.kernel_size, self.stride, self.padding)
        return super().forward(x)


def max_pool2d_host(x: torch.Tensor, kernel_size, stride=None, padding=0, grad_output: torch.Tensor | None = None):
    """Forward (and, with ``grad_output``, backward) through the kernels' window functions on the
    CPU in fp32: returns ``(y, winning taps)`` or ``(y, winning taps, grad_input)``; logical NCHW in and out."""
    k, s, p = _pair(kernel_size), _pair(kernel_size if stride is None else stride)[0], _pair(padding)
    N, C, H, W = x.shape
    Ho, Wo = _out(H, k[0], s, p[0]), _out(W, k[1], s, p[1])
    xn = x.detach().float().permute(0, 2, 3, 1).contiguous()
    y, arg = torch.empty(N, Ho, Wo, C), torch.empty(N, Ho, Wo, C, dtype=torch.uint8)
    gy = grad_output.detach().float().permute(0, 2, 3, 1).contiguous() if grad_output is not None else None
    gx = torch.empty(N, H, W, C) if gy is not None else None
    rc = _native.kernels().ft_maxpool2d_host(xn.data_ptr(), y.data_ptr(), arg.data_ptr(), gy.data_ptr() if gy is not None else None,
                                             gx.data_ptr() if gx is not None else None, N, H, W, C, k[0], k[1], s, p[0], p[1])
    _native.check(rc, "ft_maxpool2d_host")
    out = (y.permute(0, 3, 1, 2), arg.permute(0, 3, 1, 2))
    return out if gx is None else out + (gx.permute(0, 3, 1, 2),)
