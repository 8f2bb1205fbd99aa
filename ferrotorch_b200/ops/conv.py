"""2-D convolution on this library's tcgen05 GEMM kernels (NHWC bf16, fp32 accumulation).

The reference writes an im2col buffer and calls SGEMM for the forward pass and computes the
backward pass on the host (ferrotorch-gpu/src/conv.rs:239-520, ferrotorch-nn/src/conv.rs:1173-1190).
Here tensors keep torch's logical NCHW shape in ``channels_last`` memory format -- which *is*
NHWC for activations and OHWI for filters.  Forward, input gradient and filter gradient all run
on the CTA-pair GEMM kernel (``csrc/gemm_tcgen05.cu``):

* **1 x 1 filters** are plain GEMMs over the ``[pixels, channels]`` view (a stride-2 filter first
  keeps every second pixel).
* **k x k filters, stride 1 or 2** use the *shifted-row* form: the input is copied once into a
  zero-padded grid (``csrc/conv_layout.cu``; for stride 2 split into its four parity planes), in
  which the pixel a filter tap reads is a constant row offset away from the output pixel.  The
  forward and input-gradient GEMMs then load their A tiles with ordinary 2-D TMA boxes at
  ``row + shift[tap]``, and the filter gradient is one GEMM per tap over the pixel dimension,
  split across the GPU and added into an fp32 result by TMA reduce-add.  No im2col matrix exists.
* **channel counts that are not a multiple of 64** (the 3-channel stem) take an explicit im2col
  (own kernel) followed by the same GEMM.

* :func:`conv2d` -- forward (+ bias, + residual, ReLU) with autograd over the three gradients.
* :class:`IgemmConv2d`, :func:`convert_convs` -- drop-in module / model rewrite.
* :func:`implicit_gemm_reference`, :func:`shift_conv_reference` -- the kernels' index arithmetic
  restated with torch ops; the CPU tests check them against ``torch.nn.functional.conv2d``.

The native path needs CUDA, bf16 activations, groups == 1, square stride 1 or 2 and (for
k x k) ``Cin % 64 == 0`` and ``Cout % 64 == 0``; other problems fall back to
``torch.nn.functional.conv2d``.  It is on by default on a GPU (``use_native_conv(False)`` or
``FT_CONV_NATIVE=0`` switches it off); the older gather-based kernel (``csrc/conv_igemm.cu``)
stays available as ``conv2d_gather``.
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as tF
from torch import nn

from .. import _native
from . import functional as F

_i, _vp = _native._i, _native._vp
_ll = _native._ll
_native.register_protos({
    "ft_conv2d_fprop_nhwc": (_i, [_vp] * 5 + [_i] * 13 + [_vp]),
    "ft_conv2d_gather_offsets_host": (_i, [_vp] + [_i] * 10),
    "ft_conv_shift_gemm": (_i, [_vp] * 4 + [_ll, _ll, _i, _i, _i, _vp, _ll, _ll, _i, _vp, _i, _i, _vp]),
    "ft_conv_shift_wgrad": (_i, [_vp] * 3 + [_ll, _ll, _i, _i, _i, _vp, _ll, _ll, _i, _i, _i, _vp]),
    "ft_conv_embed": (_i, [_vp, _vp] + [_i] * 11 + [_vp]),
    "ft_conv_crop": (_i, [_vp, _vp] + [_i] * 10 + [_vp]),
    "ft_im2col_nhwc": (_i, [_vp, _vp] + [_i] * 12 + [_vp]),
})

_enabled = os.environ.get("FT_CONV_NATIVE", "1") != "0"
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
    """Whether the gather-based kernel (:func:`conv2d_gather`) takes this problem (square stride /
    dilation; any padding >= 0)."""
    s, d, p = _pair(stride), _pair(dilation), _pair(padding)
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 4 and groups == 1
            and s[0] == s[1] and d[0] == d[1] and min(p) >= 0 and w.shape[1] == x.shape[1]
            and x.shape[1] % 64 == 0 and w.shape[0] % 8 == 0
            and x.shape[2] + 2 * p[0] >= d[0] * (w.shape[2] - 1) + 1 and x.shape[3] + 2 * p[1] >= d[0] * (w.shape[3] - 1) + 1)


def _fprop(x, w, bias, residual, stride, pad, dil, relu):
    """Launch the gather-based kernel: ``x`` / ``w`` / ``residual`` channels-last bf16, returns
    channels-last bf16."""
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


def conv2d_gather(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride=1, padding=0,
                  dilation=1, residual: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """The gather-based implicit-GEMM kernel (``csrc/conv_igemm.cu``): forward with bias / residual /
    ReLU in its epilogue, stride-1 input gradient on the same kernel, other gradients through torch."""
    if not supported(x, weight, stride, padding, dilation, 1):
        raise RuntimeError("conv2d_gather: needs CUDA bf16, Cin % 64 == 0, Cout % 8 == 0: x %s w %s"
                           % (tuple(x.shape), tuple(weight.shape)))
    return _Conv2dIgemm.apply(x, weight, bias, residual, _pair(stride)[0], _pair(padding), _pair(dilation)[0], relu)


# --------------------------------------------------------------------------- shifted-row convolution
class ShiftGeometry:
    """Index arithmetic of the shifted-row form for one convolution shape.

    stride 1: the input sits at offset ``(ph, pw)`` of a zeroed ``[N, Hp, Wp]`` grid; output pixel
    ``(n, i, j)`` is row ``(n * Hp + i) * Wp + j`` of the GEMM and tap ``(kh, kw)`` reads the row
    ``kh * d * Wp + kw * d`` further on.  stride 2: the padded image (extents rounded up to even)
    is split into its four parity planes of ``[N, Hp, Wp]`` (= half extents) stacked one after the
    other; tap ``(kh, kw)`` reads plane ``(kh & 1, kw & 1)`` at offset ``(kh >> 1, kw >> 1)``."""

    def __init__(self, N, H, W, KH, KW, stride, ph, pw, dil):
        assert stride in (1, 2) and (stride == 1 or dil == 1)
        self.N, self.H, self.W, self.KH, self.KW = N, H, W, KH, KW
        self.stride, self.ph, self.pw, self.dil = stride, ph, pw, dil
        self.Ho, self.Wo = out_size(H, KH, stride, ph, dil), out_size(W, KW, stride, pw, dil)
        if stride == 1:
            self.planes, self.Hp, self.Wp = 1, H + 2 * ph, W + 2 * pw
        else:
            self.planes, self.Hp, self.Wp = 4, (H + 2 * ph + 1) // 2, (W + 2 * pw + 1) // 2
        self.P = N * self.Hp * self.Wp                  # GEMM rows (one plane)
        self.x_rows = self.planes * self.P

    def shifts(self) -> list[int]:
        out = []
        for kh in range(self.KH):
            for kw in range(self.KW):
                if self.stride == 1:
                    out.append(kh * self.dil * self.Wp + kw * self.dil)
                else:
                    out.append(((kh & 1) * 2 + (kw & 1)) * self.P + (kh >> 1) * self.Wp + (kw >> 1))
        return out


def _nhwc(t: torch.Tensor) -> torch.Tensor:
    """NHWC-contiguous storage of a logical NCHW tensor (a no-op for channels-last tensors)."""
    return t.contiguous(memory_format=CL)


def _embed(x: torch.Tensor, Hp: int, Wp: int, oh: int, ow: int, planes: int = 1) -> torch.Tensor:
    """``x`` (logical NCHW, channels-last storage) -> ``[planes * N * Hp * Wp, C]`` padded grid."""
    N, C, H, W = x.shape
    x = _nhwc(x)
    if not x.is_cuda:   # the kernel's arithmetic with torch ops (CPU tests of the index math)
        xn = x.permute(0, 2, 3, 1)
        if planes == 1:
            grid = xn.new_zeros(N, Hp, Wp, C)
            h0, w0 = max(0, -oh), max(0, -ow)
            h1, w1 = min(H, Hp - oh), min(W, Wp - ow)
            if h1 > h0 and w1 > w0:
                grid[:, h0 + oh:h1 + oh, w0 + ow:w1 + ow] = xn[:, h0:h1, w0:w1]
            return grid.reshape(-1, C)
        full = xn.new_zeros(N, 2 * Hp, 2 * Wp, C)
        full[:, oh:oh + H, ow:ow + W] = xn
        return torch.cat([full[:, a::2, b::2].reshape(-1, C) for a in range(2) for b in range(2)], 0)
    out = torch.empty((planes * N * Hp * Wp, C), device=x.device, dtype=x.dtype)
    rc = _native.kernels().ft_conv_embed(x.data_ptr(), out.data_ptr(), N, H, W, C, Hp, Wp, oh, ow, planes,
                                         x.element_size(), F._dev(x), F._stream())
    _native.check(rc, "ft_conv_embed")
    return out


def _crop(src: torch.Tensor, N: int, Hp: int, Wp: int, Ho: int, Wo: int, oh: int = 0, ow: int = 0) -> torch.Tensor:
    """``[N * Hp * Wp, C]`` grid -> logical ``[N, C, Ho, Wo]`` channels-last tensor (window at ``(oh, ow)``)."""
    C = src.shape[1]
    if not src.is_cuda:
        return src.view(N, Hp, Wp, C)[:, oh:oh + Ho, ow:ow + Wo].permute(0, 3, 1, 2).contiguous(memory_format=CL)
    out = torch.empty((N, C, Ho, Wo), device=src.device, dtype=src.dtype, memory_format=CL)
    rc = _native.kernels().ft_conv_crop(src.data_ptr(), out.data_ptr(), N, Ho, Wo, C, Hp, Wp, oh, ow,
                                        src.element_size(), F._dev(src), F._stream())
    _native.check(rc, "ft_conv_crop")
    return out


def _int_array(vals: list[int]):
    import ctypes

    return (ctypes.c_int * len(vals))(*vals)


def _shift_gemm(xp: torch.Tensor, w2d: torch.Tensor, P: int, shifts: list[int], bias=None, relu: bool = False,
                out_dtype=torch.bfloat16, crop: tuple | None = None) -> torch.Tensor:
    """``y[p, co] = sum_t sum_ci xp[p + shifts[t], ci] * w2d[co, t * Cin + ci]`` for ``p < P``.

    ``crop = (Hp, Wp, Ho, Wo, oh, ow)``: the rows form ``[images, Hp, Wp]`` grids and only the
    ``Ho x Wo`` window at ``(oh, ow)`` of each image is kept; the result is then the logical
    ``[images, Cout, Ho, Wo]`` channels-last tensor, written by the GEMM epilogue itself."""
    Cin, Cout = xp.shape[1], w2d.shape[0]
    assert w2d.shape[1] == len(shifts) * Cin and w2d.is_contiguous() and xp.is_contiguous()
    if not xp.is_cuda:
        acc = torch.zeros(P, Cout)
        rows = xp.shape[0]
        wk = w2d.float().view(Cout, len(shifts), Cin)
        for t, sh in enumerate(shifts):
            lo, hi = max(0, -sh), min(P, rows - sh)        # rows outside the array read as zeros
            if hi > lo:
                acc[lo:hi] += xp[lo + sh:hi + sh].float() @ wk[:, t].t()
        if bias is not None:
            acc += bias.float()
        acc = (torch.relu(acc) if relu else acc).to(out_dtype)
        if crop is None:
            return acc
        Hp, Wp, Ho, Wo, oh, ow = crop
        return _crop(acc, P // (Hp * Wp), Hp, Wp, Ho, Wo, oh, ow)
    if crop is None:
        y = torch.empty((P, Cout), device=xp.device, dtype=out_dtype)
        y2, crop_arr = y, None
    else:
        Hp, Wp, Ho, Wo, oh, ow = crop
        y = torch.empty((P // (Hp * Wp), Cout, Ho, Wo), device=xp.device, dtype=out_dtype, memory_format=CL)
        y2, crop_arr = y.permute(0, 2, 3, 1).reshape(-1, Cout), _int_array(list(crop))
    flags = (F.GEMM_OUT_F32 if out_dtype == torch.float32 else 0) | (F.GEMM_RELU if relu else 0)
    bias_ptr = None
    if bias is not None:
        bias = bias.contiguous()
        flags |= F.GEMM_BIAS_F32 if bias.dtype == torch.float32 else F.GEMM_BIAS
        bias_ptr = bias.data_ptr()
    arr = _int_array(shifts)
    rc = _native.kernels().ft_conv_shift_gemm(xp.data_ptr(), w2d.data_ptr(), y2.data_ptr(), bias_ptr, P, xp.shape[0],
                                              Cin, Cout, len(shifts), arr, Cin, Cout, flags, crop_arr, 0, F._dev(xp),
                                              F._stream())
    _native.check(rc, "ft_conv_shift_gemm")
    return y


def _shift_wgrad(dyp: torch.Tensor, xp: torch.Tensor, P: int, shifts: list[int], out: torch.Tensor | None = None):
    """``dw[co, t * Cin + ci] (+)= sum_p dyp[p, co] * xp[p + shifts[t], ci]`` in fp32."""
    Cin, Cout = xp.shape[1], dyp.shape[1]
    if out is None:
        out = torch.zeros((Cout, len(shifts) * Cin), device=xp.device, dtype=torch.float32)
    if not xp.is_cuda:
        rows = xp.shape[0]
        for t, sh in enumerate(shifts):
            lo, hi = max(0, -sh), min(P, rows - sh)
            if hi > lo:
                out[:, t * Cin:(t + 1) * Cin] += dyp[lo:hi].float().t() @ xp[lo + sh:hi + sh].float()
        return out
    arr = _int_array(shifts)
    rc = _native.kernels().ft_conv_shift_wgrad(dyp.data_ptr(), xp.data_ptr(), out.data_ptr(), P, xp.shape[0], Cin, Cout,
                                               len(shifts), arr, Cout, Cin, 0, 0, F._dev(xp), F._stream())
    _native.check(rc, "ft_conv_shift_wgrad")
    return out


def _ohwi(w: torch.Tensor) -> torch.Tensor:
    """Filter ``[Cout, Cin, KH, KW]`` -> contiguous ``[Cout, KH * KW * Cin]`` bf16 (tap-major)."""
    return w.to(torch.bfloat16).permute(0, 2, 3, 1).reshape(w.shape[0], -1).contiguous()


def _deliver_weight_grad(w: torch.Tensor, dw_ohwi: torch.Tensor):
    """``dw_ohwi``: fp32 ``[Cout, KH, KW, Cin]``.  Adds into ``w.main_grad`` when a flat-arena trainer
    owns the gradient (and returns None), else returns the gradient in ``w``'s layout and dtype."""
    g = dw_ohwi.permute(0, 3, 1, 2)
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        mg.add_(g.to(mg.dtype))
        hook = getattr(w, "grad_ready_hook", None)
        if hook is not None:
            hook(w)
        return None
    return g.to(w.dtype)


def _shift_supported(x, w, s, p, d) -> bool:
    Cout, Cin, KH, KW = w.shape
    if not (s[0] == s[1] and d[0] == d[1] and s[0] in (1, 2) and (s[0] == 1 or d[0] == 1)):
        return False
    if Cin % 64 or Cout % 64 or KH * KW > 49 or min(p) < 0:
        return False
    if x.shape[2] + 2 * p[0] < d[0] * (KH - 1) + 1 or x.shape[3] + 2 * p[1] < d[0] * (KW - 1) + 1:
        return False
    # input gradient of a stride-1 filter: dy padded by d (K - 1) - p on each side
    if s[0] == 1 and (d[0] * (KH - 1) - p[0] < 0 or d[0] * (KW - 1) - p[1] < 0):
        return False
    return x.shape[0] * (x.shape[2] + 2 * p[0] + 1) * (x.shape[3] + 2 * p[1] + 1) < 2 ** 31 - 2 ** 17


class _ShiftConv(torch.autograd.Function):
    """k x k convolution, stride 1 or 2, all three GEMMs on the shifted-row kernels."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, pad, dil, relu):
        N, Cin, H, W = x.shape
        Cout, _, KH, KW = w.shape
        g = ShiftGeometry(N, H, W, KH, KW, stride, pad[0], pad[1], dil)
        xp = _embed(x, g.Hp, g.Wp, pad[0], pad[1], g.planes)
        y = _shift_gemm(xp, _ohwi(w), g.P, g.shifts(), bias, relu, crop=(g.Hp, g.Wp, g.Ho, g.Wo, 0, 0))
        ctx.save_for_backward(xp if w.requires_grad else None, w, y if relu else None)
        ctx.g, ctx.relu, ctx.has_bias, ctx.xshape = g, relu, bias is not None, tuple(x.shape)
        return y

    @staticmethod
    def backward(ctx, gy):
        xp, w, y = ctx.saved_tensors
        g: ShiftGeometry = ctx.g
        N, Cin, H, W = ctx.xshape
        Cout, _, KH, KW = w.shape
        if ctx.relu:
            gy = gy * (y > 0)
        gy = _nhwc(gy.to(torch.bfloat16))
        gx = gw = gb = None
        # "same" stride-1 filters (2 p = d (K - 1)): dy padded for the input gradient has the grid of
        # the forward pass, so one padded copy of dy serves both gradients (the filter gradient then
        # reads x at shifts taken relative to dy's offset (p, p) in that grid)
        same = (g.stride == 1 and g.dil * (KH - 1) == 2 * g.ph and g.dil * (KW - 1) == 2 * g.pw
                and ctx.needs_input_grad[0] and ctx.needs_input_grad[1])
        dyp_same = _embed(gy, g.Hp, g.Wp, g.ph, g.pw, 1) if same else None
        if ctx.needs_input_grad[1]:
            if same:
                off = g.ph * g.Wp + g.pw
                dw = _shift_wgrad(dyp_same, xp, g.P, [sh - off for sh in g.shifts()])
            else:
                dyp = _embed(gy, g.Hp, g.Wp, 0, 0, 1)      # dy at the output's own rows of the grid
                dw = _shift_wgrad(dyp, xp, g.P, g.shifts())
            gw = _deliver_weight_grad(w, dw.view(Cout, KH, KW, Cin))
        if ctx.needs_input_grad[0]:
            gx = _shift_dgrad(gy, w, g, H, W, dyp_same)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy.float().sum(dim=(0, 2, 3))
        return gx, gw, gb, None, None, None, None


def _shift_dgrad(gy: torch.Tensor, w: torch.Tensor, g: ShiftGeometry, H: int, W: int,
                 dyp_same: torch.Tensor | None = None) -> torch.Tensor:
    """Input gradient ``[N, Cin, H, W]`` of the convolution described by ``g``.  ``dyp_same``: dy
    already embedded at offset ``(d (KH - 1) - ph, d (KW - 1) - pw)`` of the right grid, if the caller has it."""
    N, Cout = gy.shape[0], gy.shape[1]
    Cin, KH, KW, d = w.shape[1], g.KH, g.KW, g.dil
    wb = w.to(torch.bfloat16)
    if g.stride == 1:
        # dx = conv(dy padded by d (K - 1) - p, filter flipped and its channel axes swapped)
        bh, bw = d * (KH - 1) - g.ph, d * (KW - 1) - g.pw
        gd = ShiftGeometry(N, g.Ho, g.Wo, KH, KW, 1, bh, bw, d)
        dyp = dyp_same if dyp_same is not None else _embed(gy, gd.Hp, gd.Wp, bh, bw, 1)
        wt = wb.flip(2, 3).permute(1, 2, 3, 0).reshape(Cin, KH * KW * Cout).contiguous()
        return _shift_gemm(dyp, wt, gd.P, gd.shifts(), crop=(gd.Hp, gd.Wp, H, W, 0, 0))
    # stride 2: the padded input splits into four parity planes; plane (a, b) is a stride-1
    # correlation of dy with the taps kh = a + 2 r, kw = b + 2 t, read at offsets (-r, -t)
    He, We = 2 * g.Hp, 2 * g.Wp
    dxp = torch.zeros((N, He, We, Cin), device=gy.device, dtype=torch.bfloat16)
    for a in range(2):
        for b in range(2):
            rs, ts = list(range((KH - a + 1) // 2)), list(range((KW - b + 1) // 2))
            if not rs or not ts:
                continue
            R, T = rs[-1], ts[-1]
            Hg, Wg = max(g.Ho, g.Hp) + R, max(g.Wo, g.Wp) + T
            dyp = _embed(gy, Hg, Wg, R, T, 1)
            taps = [(a + 2 * r, b + 2 * t) for r in rs for t in ts]
            shifts = [-(r * Wg + t) for r in rs for t in ts]
            wsub = torch.stack([wb[:, :, kh, kw] for kh, kw in taps], dim=0)      # [taps, Cout, Cin]
            wt = wsub.permute(2, 0, 1).reshape(Cin, len(taps) * Cout).contiguous()
            pl = _shift_gemm(dyp, wt, N * Hg * Wg, shifts, crop=(Hg, Wg, g.Hp, g.Wp, R, T))   # logical [N, Cin, Hp, Wp]
            dxp[:, a::2, b::2, :] = pl.permute(0, 2, 3, 1)
    dx = dxp[:, g.ph:g.ph + H, g.pw:g.pw + W, :].permute(0, 3, 1, 2)
    return dx.contiguous(memory_format=CL)


class _PointwiseConv(torch.autograd.Function):
    """1 x 1 convolution (padding 0): three plain GEMMs over the ``[pixels, channels]`` view."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, relu):
        N, Cin, H, W = x.shape
        Cout = w.shape[0]
        xs = x if stride == 1 else x[:, :, ::stride, ::stride]
        xs = _nhwc(xs)
        Ho, Wo = xs.shape[2], xs.shape[3]
        x2 = xs.permute(0, 2, 3, 1).reshape(-1, Cin)
        w2 = w.to(torch.bfloat16).reshape(Cout, Cin)
        y = torch.empty((N, Cout, Ho, Wo), device=x.device, dtype=torch.bfloat16, memory_format=CL)
        F.gemm_nt(x2, w2, bias=bias, out=y.permute(0, 2, 3, 1).reshape(-1, Cout), activation="relu" if relu else None)
        ctx.save_for_backward(x2 if w.requires_grad else None, w, y if relu else None)
        ctx.cfg = (stride, relu, bias is not None, tuple(x.shape), (Ho, Wo))
        return y

    @staticmethod
    def backward(ctx, gy):
        x2, w, y = ctx.saved_tensors
        stride, relu, has_bias, xshape, (Ho, Wo) = ctx.cfg
        N, Cin, H, W = xshape
        Cout = w.shape[0]
        if relu:
            gy = gy * (y > 0)
        gy = _nhwc(gy.to(torch.bfloat16))
        g2 = gy.permute(0, 2, 3, 1).reshape(-1, Cout)
        gx = gw = gb = None
        if ctx.needs_input_grad[1]:
            if x2.is_cuda and Cin % 64 == 0 and Cout % 64 == 0:
                # pixels are the contraction dimension: split over the GPU, tiles added in fp32
                dw = _shift_wgrad(g2, x2, g2.shape[0], [0])
            else:
                dw = F.gemm_nt(g2.t(), x2.t(), out_dtype=torch.float32)          # [Cout, Cin]
            gw = _deliver_weight_grad(w, dw.view(Cout, 1, 1, Cin))
        if ctx.needs_input_grad[0]:
            w2 = w.to(torch.bfloat16).reshape(Cout, Cin)
            if stride == 1:
                gx = torch.empty((N, Cin, H, W), device=gy.device, dtype=torch.bfloat16, memory_format=CL)
                F.gemm_nt(g2, w2.t(), out=gx.permute(0, 2, 3, 1).reshape(-1, Cin))
            else:
                gs = F.gemm_nt(g2, w2.t()).view(N, Ho, Wo, Cin)
                gx = torch.empty((N, Cin, H, W), device=gy.device, dtype=torch.bfloat16, memory_format=CL).zero_()
                gx[:, :, ::stride, ::stride] = gs.permute(0, 3, 1, 2)
        if has_bias and ctx.needs_input_grad[2]:
            gb = gy.float().sum(dim=(0, 2, 3))
        return gx, gw, gb, None, None


class _Im2colConv(torch.autograd.Function):
    """Convolution through an explicit patch matrix (own im2col kernel) and the GEMM; for channel
    counts the shifted-row form does not take.  Channels are zero-padded to a multiple of 4 (8-byte
    pixels) first.  The input gradient goes through torch."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, pad, dil, relu):
        N, Cin, H, W = x.shape
        Cout, _, KH, KW = w.shape
        Ho, Wo = out_size(H, KH, stride, pad[0], dil), out_size(W, KW, stride, pad[1], dil)
        Cp = (Cin + 3) // 4 * 4
        Kpad = (KH * KW * Cp + 7) // 8 * 8
        xn = _pad_channels(_nhwc(x), Cp)
        patches = _im2col(xn, KH, KW, stride, pad, dil, Ho, Wo, Kpad)
        w2 = torch.zeros((Cout, Kpad), device=x.device, dtype=torch.bfloat16)
        w2[:, :KH * KW * Cp].view(Cout, KH * KW, Cp)[:, :, :Cin] = w.to(torch.bfloat16).permute(0, 2, 3, 1).reshape(Cout, KH * KW, Cin)
        y = torch.empty((N, Cout, Ho, Wo), device=x.device, dtype=torch.bfloat16, memory_format=CL)
        F.gemm_nt(patches, w2, bias=bias, out=y.permute(0, 2, 3, 1).reshape(-1, Cout),
                  activation="relu" if relu else None)
        ctx.save_for_backward(xn, w, y if relu else None)     # the patch matrix is rebuilt in backward
        ctx.cfg = (stride, pad, dil, relu, bias is not None, Ho, Wo, Kpad, Cp)
        return y

    @staticmethod
    def backward(ctx, gy):
        xn, w, y = ctx.saved_tensors
        stride, pad, dil, relu, has_bias, Ho, Wo, Kpad, Cp = ctx.cfg
        Cout, Cin, KH, KW = w.shape
        if relu:
            gy = gy * (y > 0)
        gy = _nhwc(gy.to(torch.bfloat16))
        g2 = gy.permute(0, 2, 3, 1).reshape(-1, Cout)
        gx = gw = gb = None
        if ctx.needs_input_grad[1]:
            patches = _im2col(xn, KH, KW, stride, pad, dil, Ho, Wo, Kpad)
            if g2.is_cuda and Cout % 64 == 0:
                dw = _shift_wgrad(g2, patches, g2.shape[0], [0])                  # pixels split over the GPU
            else:
                dw = F.gemm_nt(g2.t(), patches.t(), out_dtype=torch.float32)      # [Cout, Kpad]
            gw = _deliver_weight_grad(w, dw[:, :KH * KW * Cp].reshape(Cout, KH, KW, Cp)[..., :Cin])
        if ctx.needs_input_grad[0]:
            gx = torch.nn.grad.conv2d_input((xn.shape[0], Cin, xn.shape[2], xn.shape[3]), w.to(torch.bfloat16), gy,
                                            stride, pad, dil)
        if has_bias and ctx.needs_input_grad[2]:
            gb = gy.float().sum(dim=(0, 2, 3))
        return gx, gw, gb, None, None, None, None


def _pad_channels(xn: torch.Tensor, Cp: int) -> torch.Tensor:
    """Zero-pad the channel dimension of a channels-last tensor to ``Cp`` (NHWC-contiguous result)."""
    N, C, H, W = xn.shape
    if C == Cp:
        return xn
    out = torch.zeros((N, Cp, H, W), device=xn.device, dtype=xn.dtype).contiguous(memory_format=CL)
    out[:, :C] = xn
    return out


def _im2col(xn: torch.Tensor, KH, KW, stride, pad, dil, Ho, Wo, Kpad) -> torch.Tensor:
    N, C, H, W = xn.shape
    if not xn.is_cuda:
        cols = tF.unfold(xn.float(), (KH, KW), dil, pad, stride)                  # [N, C * KH * KW, L], channel-major
        cols = cols.view(N, C, KH * KW, Ho * Wo).permute(0, 3, 2, 1).reshape(N * Ho * Wo, KH * KW * C)
        out = torch.zeros((N * Ho * Wo, Kpad), dtype=xn.dtype)
        out[:, :KH * KW * C] = cols.to(xn.dtype)
        return out
    out = torch.empty((N * Ho * Wo, Kpad), device=xn.device, dtype=torch.bfloat16)
    rc = _native.kernels().ft_im2col_nhwc(xn.data_ptr(), out.data_ptr(), N, H, W, C, KH, KW, stride, pad[0], pad[1],
                                          dil, Kpad, F._dev(xn), F._stream())
    _native.check(rc, "ft_im2col_nhwc")
    return out


stats = {"pointwise": 0, "shift": 0, "im2col": 0, "library": 0}


def native_path(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation, groups: int = 1) -> str | None:
    """Which native path takes this problem: "pointwise", "shift", "im2col", or None (library)."""
    if not (x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and groups == 1 and weight.shape[1] == x.shape[1]):
        return None
    if weight.dtype not in (torch.bfloat16, torch.float32) or isinstance(padding, str):
        return None
    s, d, p = _pair(stride), _pair(dilation), _pair(padding)
    Cout, Cin, KH, KW = weight.shape
    if KH == 1 and KW == 1 and p == (0, 0) and s[0] == s[1] and Cin % 8 == 0 and Cout % 8 == 0:
        return "pointwise"
    if _shift_supported(x, weight, s, p, d):
        return "shift"
    if (s[0] == s[1] and d[0] == d[1] and min(p) >= 0 and Cout % 8 == 0 and KH * KW * Cin <= 4096
            and x.shape[2] + 2 * p[0] >= d[0] * (KH - 1) + 1 and x.shape[3] + 2 * p[1] >= d[0] * (KW - 1) + 1):
        return "im2col"
    return None


def conv2d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride=1, padding=0, dilation=1,
           groups: int = 1, residual: torch.Tensor | None = None, relu: bool = False) -> torch.Tensor:
    """``relu(conv2d(x, weight) + bias + residual)`` (the last three optional).  Logical NCHW
    tensors; on the native paths the result is bf16 in channels-last memory format and all three
    gradients come from this library's GEMM kernels."""
    path = native_path(x, weight, stride, padding, dilation, groups) if _enabled else None
    if path is not None:
        s, p, d = _pair(stride)[0], _pair(padding), _pair(dilation)[0]
        fuse_relu = relu and residual is None
        stats[path] += 1
        if path == "pointwise":
            y = _PointwiseConv.apply(x, weight, bias, s, fuse_relu)
        elif path == "shift":
            y = _ShiftConv.apply(x, weight, bias, s, p, d, fuse_relu)
        else:
            y = _Im2colConv.apply(x, weight, bias, s, p, d, fuse_relu)
        if residual is not None:
            y = y + residual
            y = torch.relu(y) if relu else y
        return y
    if x.is_cuda and _enabled and os.environ.get("FT_CONV_STRICT") == "1":
        raise RuntimeError("conv2d: no native path takes this problem (needs bf16 activations, groups == 1): "
                           "x %s w %s" % (tuple(x.shape), tuple(weight.shape)))
    stats["library"] += 1
    y = tF.conv2d(x, weight.to(x.dtype) if weight.dtype != x.dtype else weight,
                  bias.to(x.dtype) if bias is not None and bias.dtype != x.dtype else bias, stride, padding, dilation, groups)
    if residual is not None:
        y = y + residual
    return torch.relu(y) if relu else y


def shift_conv_reference(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, padding=0, dilation: int = 1) -> torch.Tensor:
    """The shifted-row arithmetic with torch ops in fp32, on any device: build the padded grid
    (parity planes for stride 2), add up ``grid[p + shift[tap]] @ W[tap]`` over the taps with plain
    row slices, crop.  The CPU tests compare it with ``torch.nn.functional.conv2d``."""
    N, Cin, H, W = x.shape
    Cout, _, KH, KW = weight.shape
    ph, pw = _pair(padding)
    g = ShiftGeometry(N, H, W, KH, KW, stride, ph, pw, dilation)
    xn = x.permute(0, 2, 3, 1).float()
    if stride == 1:
        grid = torch.zeros(N, g.Hp, g.Wp, Cin)
        grid[:, ph:ph + H, pw:pw + W] = xn
        flat = grid.reshape(-1, Cin)
    else:
        full = torch.zeros(N, 2 * g.Hp, 2 * g.Wp, Cin)
        full[:, ph:ph + H, pw:pw + W] = xn
        flat = torch.cat([full[:, a::2, b::2].reshape(-1, Cin) for a in range(2) for b in range(2)], 0)
    wk = weight.permute(0, 2, 3, 1).float().reshape(Cout, KH * KW, Cin)
    y = torch.zeros(g.P, Cout)
    rows = flat.shape[0]
    for t, sh in enumerate(g.shifts()):
        lo, hi = max(0, -sh), min(g.P, rows - sh)           # rows outside the array read as zeros
        if hi > lo:
            y[lo:hi] += flat[lo + sh:hi + sh] @ wk[:, t].t()
    return y.view(N, g.Hp, g.Wp, Cout)[:, :g.Ho, :g.Wo].permute(0, 3, 1, 2)


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
