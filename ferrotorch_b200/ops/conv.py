"""2-D convolution on the implicit-GEMM tcgen05 kernel (``csrc/conv_igemm.cu``).

The reference writes an im2col buffer and calls SGEMM for the forward pass and computes the
backward pass on the host (ferrotorch-gpu/src/conv.rs:520, ferrotorch-nn/src/conv.rs:1173).  Here
tensors keep torch's logical NCHW shape in ``channels_last`` memory format -- which *is* NHWC for
activations and OHWI for filters, the two layouts the kernel reads -- so nothing is permuted or
copied on the way in or out.

* :func:`conv2d` -- forward (+ bias, + residual, ReLU in the epilogue) with autograd: the input
  gradient of a stride-1 convolution runs on the same kernel (dy against the flipped filter with
  its channel axes swapped); strided input gradients and the filter gradient go through torch.
* :class:`IgemmConv2d`, :func:`convert_convs` -- drop-in module / model rewrite.
* :func:`implicit_gemm_reference` -- the kernel's tile arithmetic (row = output pixel, k-block =
  one filter tap x 64 channels) restated with torch ops; the CPU tests check it against
  ``torch.nn.functional.conv2d``.

The native path needs CUDA, bf16, ``Cin % 64 == 0``, ``Cout % 8 == 0`` and groups == 1; anything
else falls back to ``torch.nn.functional.conv2d``.  It is opt-in (:func:`use_native_conv` or
``FT_CONV_IGEMM=1``).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as tF
from torch import nn

from .. import _native
from . import functional as F

_i, _vp = _native._i, _native._vp
_native.register_protos({
    "ft_conv2d_fprop_nhwc": (_i, [_vp] * 5 + [_i] * 13 + [_vp]),
    "ft_conv2d_gather_offsets_host": (_i, [_vp] + [_i] * 10),
})

_enabled = os.environ.get("FT_CONV_IGEMM") == "1"
CL = torch.channels_last


def use_native_conv(on: bool = True) -> bool:
    """Switch the implicit-GEMM kernel on or off for :func:`conv2d`; returns the previous setting."""
    global _enabled
    prev, _enabled = _enabled, bool(on)
    return prev


def native_conv_enabled() -> bool:
    return _enabled


def _pair(v) -> tuple:
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def out_size(size: int, k: int, stride: int, pad: int, dil: int) -> int:
    return (size + 2 * pad - dil * (k - 1) - 1) // stride + 1


def supported(x: torch.Tensor, w: torch.Tensor, stride, padding, dilation, groups: int = 1) -> bool:
    """Whether the kernel takes this problem (square stride / dilation; any padding >= 0)."""
    s, d, p = _pair(stride), _pair(dilation), _pair(padding)
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 4 and groups == 1
            and s[0] == s[1] and d[0] == d[1] and min(p) >= 0 and w.shape[1] == x.shape[1]
            and x.shape[1] % 64 == 0 and w.shape[0] % 8 == 0
            and x.shape[2] + 2 * p[0] >= d[0] * (w.shape[2] - 1) + 1 and x.shape[3] + 2 * p[1] >= d[0] * (w.shape[3] - 1) + 1)


def _fprop(x, w, bias, residual, stride, pad, dil, relu):
    """Launch the kernel: ``x`` / ``w`` / ``residual`` channels-last bf16, returns channels-last bf16."""
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = w.shape
    Ho, Wo = out_size(H, KH, stride, pad[0], dil), out_size(W, KW, stride, pad[1], dil)
    x, w = x.contiguous(memory_format=CL), w.contiguous(memory_format=CL)
    y = torch.empty((N, Cout, Ho, Wo), device=x.device, dtype=torch.bfloat16, memory_format=CL)
    if residual is not None:
        residual = residual.contiguous(memory_format=CL)
        assert residual.shape == y.shape and residual.dtype == torch.bfloat16
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
    rc = _native.kernels().ft_conv2d_fprop_nhwc(
        x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
        residual.data_ptr() if residual is not None else None, y.data_ptr(), N, H, W, Cin, Cout, KH, KW, stride,
        pad[0], pad[1], dil, int(relu), F._dev(x), F._stream())
    _native.check(rc, "ft_conv2d_fprop_nhwc")
    return y


class _Conv2dIgemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual, stride, pad, dil, relu):
        y = _fprop(x, w, bias, residual, stride, pad, dil, relu)
        ctx.save_for_backward(x, w, y if relu else None)
        ctx.cfg = (stride, pad, dil, relu, bias is not None, residual is not None)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, w, y = ctx.saved_tensors
        stride, pad, dil, relu, has_bias, has_res = ctx.cfg
        if relu:
            gy = gy * (y > 0)
        gy = gy.contiguous(memory_format=CL)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            KH, KW = w.shape[2], w.shape[3]
            bp = (dil * (KH - 1) - pad[0], dil * (KW - 1) - pad[1])
            wt = w.flip(2, 3).transpose(0, 1)                       # [Cin, Cout, KH, KW]: dx = conv(dy, wt)
            if stride == 1 and min(bp) >= 0 and supported(gy, wt, 1, bp, dil):
                gx = _fprop(gy, wt, None, None, 1, bp, dil, False)
            else:
                gx = torch.nn.grad.conv2d_input(x.shape, w, gy, stride, pad, dil)
        if ctx.needs_input_grad[1]:
            gw = torch.nn.grad.conv2d_weight(x, w.shape, gy, stride, pad, dil)
        if has_bias and ctx.needs_input_grad[2]:
            gb = gy.float().sum(dim=(0, 2, 3)).to(gy.dtype)
        gr = gy if has_res and ctx.needs_input_grad[3] else None
        return gx, gw, gb, gr, None, None, None, None


def conv2d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride=1, padding=0, dilation=1,
           groups: int = 1, residual: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """``relu(conv2d(x, weight) + bias + residual)`` (the last three optional).  Logical NCHW
    tensors; on the native path the result is bf16 in channels-last memory format."""
    if _enabled and supported(x, weight, stride, padding, dilation, groups):
        return _Conv2dIgemm.apply(x, weight, bias, residual, _pair(stride)[0], _pair(padding), _pair(dilation)[0], relu)
    if x.is_cuda and _enabled and os.environ.get("FT_CONV_IGEMM_STRICT") == "1":
        raise RuntimeError("conv2d: the implicit-GEMM kernel does not take this problem (needs bf16, Cin % 64 == 0, "
                           "Cout % 8 == 0, groups == 1): x %s w %s" % (tuple(x.shape), tuple(weight.shape)))
    y = tF.conv2d(x, weight, bias, stride, padding, dilation, groups)
    if residual is not None:
        y = y + residual
    return torch.relu(y) if relu else y


def implicit_gemm_reference(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, padding=0, dilation: int = 1) -> torch.Tensor:
    """The kernel's arithmetic with torch ops in fp32: build the A matrix row by row the way the
    gather warps do (row m -> (n, ho, wo); k-block kb -> tap (kh, kw), channels c0..c0+63; a tap
    outside the image contributes zeros), multiply by the OHWI filter viewed as ``[Cout, K]``."""
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = weight.shape
    ph, pw = _pair(padding)
    Ho, Wo = out_size(H, KH, stride, ph, dilation), out_size(W, KW, stride, pw, dilation)
    xn = x.permute(0, 2, 3, 1).contiguous().float()                 # NHWC
    wk = weight.permute(0, 2, 3, 1).contiguous().float().reshape(Cout, KH * KW * Cin)
    M = N * Ho * Wo
    m = torch.arange(M)
    wo, ho, n = m % Wo, (m // Wo) % Ho, m // (Wo * Ho)
    hi0, wi0 = ho * stride - ph, wo * stride - pw
    A = torch.zeros(M, KH * KW * Cin)
    bk = 64 if Cin % 64 == 0 else Cin                                # the kernel needs 64; the restatement takes any Cin
    c_blocks = Cin // bk
    for kb in range(KH * KW * c_blocks):
        tap, c0 = kb // c_blocks, (kb % c_blocks) * bk
        kh, kw = tap // KW, tap % KW
        hi, wi = hi0 + kh * dilation, wi0 + kw * dilation
        ok = (hi >= 0) & (hi < H) & (wi >= 0) & (wi < W)
        rows = xn[n[ok], hi[ok], wi[ok], c0:c0 + bk]
        A[ok, kb * bk:(kb + 1) * bk] = rows
    return (A @ wk.t()).reshape(N, Ho, Wo, Cout).permute(0, 3, 1, 2)


def kernel_gather_offsets(N: int, H: int, W: int, Cin: int, KH: int, KW: int, stride: int = 1, padding=0,
                          dilation: int = 1) -> torch.Tensor:
    """The gather indices as the kernel's own index functions compute them (they are compiled for
    host and device; this calls the host side, no GPU needed): int64 ``[M, K / 64]``, the element
    offset into NHWC ``x`` of the 64 channels each (row, k-block) reads, -1 where the tap is padding."""
    ph, pw = _pair(padding)
    M = N * out_size(H, KH, stride, ph, dilation) * out_size(W, KW, stride, pw, dilation)
    out = torch.empty((M, KH * KW * Cin // 64), dtype=torch.int64)
    rc = _native.kernels().ft_conv2d_gather_offsets_host(out.data_ptr(), N, H, W, Cin, KH, KW, stride, ph, pw, dilation)
    _native.check(rc, "ft_conv2d_gather_offsets_host")
    return out


class IgemmConv2d(nn.Conv2d):
    """``nn.Conv2d`` (same parameters, same state-dict keys) whose forward calls :func:`conv2d`."""

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
        if self.padding_mode != "zeros" or isinstance(self.padding, str):
            y = super().forward(x)
            y = y if residual is None else y + residual
            return torch.relu(y) if relu else y
        return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups, residual, relu)


def convert_convs(model: nn.Module) -> int:
    """Re-class every plain ``nn.Conv2d`` of ``model`` to :class:`IgemmConv2d` in place (parameters
    are shared, not copied); returns how many were converted."""
    n = 0
    for mod in model.modules():
        if type(mod) is nn.Conv2d:
            mod.__class__ = IgemmConv2d
            n += 1
    return n
