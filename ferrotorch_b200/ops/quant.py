"""Quantised and semi-structured-sparse linear algebra on the expand-GEMM kernel
(``csrc/quant_gemm.cu``).

* GGUF Q4_0 weights: :func:`q4_0_planes` splits raw blocks into the nibble / scale planes the
  kernel reads; :func:`q4_0_linear` computes ``x @ dequant(W).T`` without ever materialising the
  bf16 weights (the reference dequantises to f32 and bounces through the host,
  ferrotorch-llama/src/gpu_gguf.rs:14-27).  GPTQ / AWQ / HQQ 4-bit checkpoints
  (ferrotorch-llama/src/quant_loaders.rs:41-670) are converted with :func:`requantize_q4_0`.
* 2:4 sparsity: :func:`apply_2_4_mask` (keep the two largest magnitudes of every 4 consecutive
  weights, ferrotorch-core/src/pruning.rs:243), :func:`pack_2_4` (values + 2-bit positions,
  the role of ferrotorch-gpu/src/semi_structured.rs:79-580) and :func:`sparse24_linear`
  (the reference calls cuSPARSELt, ferrotorch-gpu/src/cusparselt.rs:547-932).
* int8 post-training quantisation helpers (ferrotorch-core/src/quantize.rs:36-627) over torch ops.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import _native
from . import functional as F

_i, _ll, _vp = _native._i, _native._ll, _native._vp
_native.register_protos({
    "ft_q4_0_gemm": (_i, [_vp] * 5 + [_i, _i, _i, _ll, _ll, _i, _i, _vp]),
    "ft_sparse24_gemm": (_i, [_vp] * 5 + [_i, _i, _i, _ll, _ll, _i, _i, _vp]),
})


# --------------------------------------------------------------------------- Q4_0
def q4_0_planes(blocks: torch.Tensor, rows: int, cols: int, nibble_order: str = "ggml"):
    """Raw Q4_0 blocks (uint8 ``[rows*cols/32, 18]``) -> ``(nibbles u8 [rows, cols/2], scales fp16 [rows, cols/32])``.
    The kernel reads the file format's element order (byte j = elements j, j + 16); blocks whose
    bytes mean elements (2j, 2j + 1) -- ``nibble_order="interleaved"``, the order the reference's
    decoder emits -- are re-packed here first."""
    if nibble_order == "interleaved":
        q = blocks.reshape(-1, 18)[:, 2:]
        e = torch.stack([q & 0xF, q >> 4], dim=2).reshape(-1, 32)
        blocks = torch.cat([blocks.reshape(-1, 18)[:, :2], e[:, :16] | (e[:, 16:] << 4)], dim=1)
    elif nibble_order != "ggml":
        raise ValueError("nibble_order must be 'ggml' or 'interleaved'")
    b = blocks.reshape(rows, cols // 32, 18)
    scales = b[:, :, :2].contiguous().view(torch.float16).reshape(rows, cols // 32)
    nibbles = b[:, :, 2:].contiguous().reshape(rows, cols // 2)
    return nibbles, scales


def dequant_q4_0_planes(nibbles: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    rows = nibbles.shape[0]
    nb = nibbles.view(rows, -1, 16)
    lo, hi = (nb & 0xF).float() - 8.0, (nb >> 4).float() - 8.0
    return (torch.cat([lo, hi], dim=-1) * scales.float().unsqueeze(-1)).reshape(rows, -1)


def q4_0_linear(x: torch.Tensor, nibbles: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None,
                out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x [..., K] @ dequant(W)[N, K].T (+ bias)``."""
    N, K = nibbles.shape[0], nibbles.shape[1] * 2
    x2 = x.reshape(-1, K)
    native = x.is_cuda and x.dtype == torch.bfloat16 and K % 64 == 0 and N % 8 == 0
    if not native:
        w = dequant_q4_0_planes(nibbles, scales).to(x.dtype)
        return torch.nn.functional.linear(x, w, bias)
    x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
    out_dtype = out_dtype or x.dtype
    y = torch.empty((x2.shape[0], N), device=x.device, dtype=out_dtype)
    rc = _native.kernels().ft_q4_0_gemm(x2.data_ptr(), nibbles.data_ptr(), scales.data_ptr(), y.data_ptr(),
                                        bias.data_ptr() if bias is not None else None, x2.shape[0], N, K,
                                        x2.stride(0), y.stride(0), int(out_dtype == torch.float32), F._dev(x),
                                        F._stream())
    _native.check(rc, "ft_q4_0_gemm")
    return y.view(*x.shape[:-1], N)


def quantize_q4_0_planes(w: torch.Tensor, chunk_rows: int = 8192):
    """Quantise a float matrix ``[N, K]`` (K % 32 == 0) straight to the kernel's planes
    ``(nibbles u8 [N, K/2], scales fp16 [N, K/32])`` on the tensor's own device, ``chunk_rows``
    rows at a time (ggml rule: ``d = signed value of largest magnitude / -8``,
    ``q = clamp(floor(x / d + 8.5), 0, 15)``; same result as ``serialize.gguf.quantize_q4_0``)."""
    N, K = w.shape
    assert K % 32 == 0
    nib = torch.empty((N, K // 2), device=w.device, dtype=torch.uint8)
    sc = torch.empty((N, K // 32), device=w.device, dtype=torch.float16)
    for r0 in range(0, N, chunk_rows):
        x = w[r0:r0 + chunk_rows].detach().float().reshape(-1, 32)
        mx = x.gather(1, x.abs().argmax(dim=1, keepdim=True))
        d = mx / -8.0
        inv = torch.where(d != 0, 1.0 / d, torch.zeros_like(d))
        q = (x * inv + 8.5).floor_().clamp_(0, 15).to(torch.uint8)
        rows = min(chunk_rows, N - r0)
        nib[r0:r0 + rows] = (q[:, :16] | (q[:, 16:] << 4)).reshape(rows, K // 2)
        sc[r0:r0 + rows] = d.to(torch.float16).reshape(rows, K // 32)
    return nib, sc


def requantize_q4_0(w: torch.Tensor):
    """Any float weight ``[N, K]`` (e.g. a dequantised GPTQ / AWQ / HQQ tensor) -> Q4_0 planes."""
    from ..serialize.gguf import quantize_q4_0

    N, K = w.shape
    return q4_0_planes(quantize_q4_0(w), N, K)


class Q4Linear(nn.Module):
    """Inference-only linear layer holding Q4_0 planes."""

    def __init__(self, nibbles: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None = None):
        super().__init__()
        self.register_buffer("nibbles", nibbles.contiguous())
        self.register_buffer("scales", scales.contiguous())
        self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None
        self.out_features, self.in_features = nibbles.shape[0], nibbles.shape[1] * 2

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "Q4Linear":
        nib, sc = requantize_q4_0(lin.weight.detach())
        return cls(nib.to(lin.weight.device), sc.to(lin.weight.device), lin.bias.detach() if lin.bias is not None else None)

    def forward(self, x):
        return q4_0_linear(x, self.nibbles, self.scales, self.bias)


# --------------------------------------------------------------------------- 2:4 sparsity
def apply_2_4_mask(w: torch.Tensor) -> torch.Tensor:
    """Zero the two smallest magnitudes in every group of 4 along the last dim."""
    g = w.reshape(-1, 4)
    keep = g.abs().topk(2, dim=1).indices
    mask = torch.zeros_like(g, dtype=torch.bool).scatter_(1, keep, True)
    return (g * mask).reshape(w.shape)


def pack_2_4(w: torch.Tensor):
    """2:4-sparse ``[N, K]`` -> ``(values [N, K/2], meta u8 [N, K/8])``; each metadata nibble holds the
    slots of a group's two kept values (bits 0-1 first, bits 2-3 second, first < second)."""
    N, K = w.shape
    g = w.reshape(N, K // 4, 4)
    nz = g != 0
    # choose exactly two slots per group: the non-zeros first, padded with the lowest free slots
    order = torch.argsort((~nz).to(torch.int8) * 4 + torch.arange(4, device=w.device, dtype=torch.int8), dim=-1)
    pos = order[..., :2].sort(dim=-1).values
    if bool((nz.sum(-1) > 2).any()):
        raise ValueError("pack_2_4: a group of 4 has more than 2 non-zeros")
    values = g.gather(-1, pos).reshape(N, K // 2).contiguous()
    nib = (pos[..., 0] | (pos[..., 1] << 2)).to(torch.uint8)             # [N, K/4]
    meta = (nib[:, 0::2] | (nib[:, 1::2] << 4)).contiguous()             # two groups per byte
    return values, meta


def unpack_2_4(values: torch.Tensor, meta: torch.Tensor) -> torch.Tensor:
    N, K2 = values.shape
    nib = torch.stack([meta & 0xF, meta >> 4], dim=-1).reshape(N, -1).long()
    pos = torch.stack([nib & 3, nib >> 2], dim=-1)
    out = torch.zeros(N, K2 // 2, 4, dtype=values.dtype, device=values.device)
    out.scatter_(-1, pos, values.reshape(N, K2 // 2, 2))
    return out.reshape(N, K2 * 2)


def sparse24_linear(x: torch.Tensor, values: torch.Tensor, meta: torch.Tensor, bias: torch.Tensor | None = None):
    """``x [..., K] @ W.T`` for 2:4-compressed ``W`` (``sparse_matmul_24``, ferrotorch-core/src/sparse.rs:2201)."""
    N, K = values.shape[0], values.shape[1] * 2
    native = x.is_cuda and x.dtype == torch.bfloat16 and values.dtype == torch.bfloat16 and K % 64 == 0 and N % 8 == 0
    if not native:
        return torch.nn.functional.linear(x, unpack_2_4(values, meta).to(x.dtype), bias)
    x2 = x.reshape(-1, K)
    x2 = x2 if x2.stride(-1) == 1 else x2.contiguous()
    y = torch.empty((x2.shape[0], N), device=x.device, dtype=x.dtype)
    rc = _native.kernels().ft_sparse24_gemm(x2.data_ptr(), values.data_ptr(), meta.data_ptr(), y.data_ptr(),
                                            bias.data_ptr() if bias is not None else None, x2.shape[0], N, K,
                                            x2.stride(0), y.stride(0), 0, F._dev(x), F._stream())
    _native.check(rc, "ft_sparse24_gemm")
    return y.view(*x.shape[:-1], N)


class SemiStructuredLinear(nn.Module):
    def __init__(self, values, meta, bias=None):
        super().__init__()
        self.register_buffer("values", values.contiguous())
        self.register_buffer("meta", meta.contiguous())
        self.bias = nn.Parameter(bias, requires_grad=False) if bias is not None else None

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "SemiStructuredLinear":
        v, m = pack_2_4(apply_2_4_mask(lin.weight.detach()))
        return cls(v, m, lin.bias.detach() if lin.bias is not None else None)

    def forward(self, x):
        return sparse24_linear(x, self.values, self.meta, self.bias)


# --------------------------------------------------------------------------- int8 PTQ helpers
def quantize_per_channel_int8(w: torch.Tensor, dim: int = 0):
    """Symmetric per-channel int8: returns ``(q int8, scale fp32)`` with ``w ~= q * scale``."""
    red = [d for d in range(w.dim()) if d != dim]
    scale = w.abs().amax(dim=red, keepdim=True).clamp_min(1e-12) / 127.0
    return (w / scale).round().clamp(-127, 127).to(torch.int8), scale.float()


def quantized_matmul_int8(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """``x @ (q * scale).T`` with per-tensor dynamic int8 activations and int32 accumulation."""
    sx = x.abs().amax().clamp_min(1e-12) / 127.0
    qx = (x / sx).round().clamp(-127, 127).to(torch.int8)
    acc = (qx.to(torch.int32) @ q.to(torch.int32).t()) if not x.is_cuda else torch._int_mm(qx, q.t().contiguous()) \
        if qx.shape[0] > 16 and qx.shape[0] % 8 == 0 and q.shape[0] % 8 == 0 and q.shape[1] % 8 == 0 else \
        (qx.float() @ q.float().t()).to(torch.int32)
    return acc.float() * sx * scale.reshape(1, -1)
