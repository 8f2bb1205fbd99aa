"""Int4 checkpoint layouts: GPTQ, AWQ and HQQ -> float weights (and on to this framework's Q4_0
planes for the fused dequant-GEMM).

Layouts follow the public formats the reference also reads (ferrotorch-llama/src/quant_loaders.rs:41-670):

* **GPTQ** (AutoGPTQ v1): ``qweight int32 [K/8, N]`` -- eight 4-bit values per word along K, low
  nibble first; ``qzeros int32 [K/g, N/8]`` packed along N (stored zero is ``zero - 1``);
  ``scales fp16 [K/g, N]``; optional ``g_idx int32 [K]`` (group of every input channel).
* **AWQ** (AutoAWQ GEMM): ``qweight int32 [K, N/8]`` and ``qzeros int32 [K/g, N/8]`` packed along N
  in the interleaved order 0,2,4,6,1,3,5,7; ``scales fp16 [K/g, N]``.
* **HQQ** (4-bit, grouped along the input axis): the weight is viewed as ``[groups, group_size]``
  and transposed; ``W_q uint8`` holds the first half of every group in the high nibbles and the
  second half in the low nibbles of the same bytes; ``scale`` / ``zero`` per group:
  ``W = (W_q - zero) * scale``.

All functions return the weight as ``[N, K]`` (out_features, in_features) float tensors, the
layout ``nn.Linear`` uses.  ``pack_*`` are the inverse transforms (used by the tests and to write
fixtures).
"""
from __future__ import annotations

import torch

_AWQ_ORDER = [0, 2, 4, 6, 1, 3, 5, 7]


def _unpack_int32(words: torch.Tensor, dim: int, order=None) -> torch.Tensor:
    """Expand every int32 into its eight nibbles along ``dim`` (low nibble first, or ``order``)."""
    shifts = torch.arange(0, 32, 4, device=words.device, dtype=torch.int32)
    w = words.to(torch.int32).unsqueeze(dim + 1 if dim >= 0 else dim)
    shape = [1] * w.dim()
    shape[dim + 1 if dim >= 0 else dim] = 8
    nib = (w >> shifts.view(shape)) & 0xF
    if order is not None:
        inv = torch.tensor([order.index(i) for i in range(8)], device=words.device)
        nib = nib.index_select(dim + 1 if dim >= 0 else dim, inv)
    out_shape = list(words.shape)
    out_shape[dim] *= 8
    return nib.reshape(out_shape)


def _pack_int32(nib: torch.Tensor, dim: int, order=None) -> torch.Tensor:
    shape = list(nib.shape)
    shape[dim] //= 8
    shape.insert(dim + 1, 8)
    n = nib.to(torch.int64).reshape(shape)
    if order is not None:
        n = n.index_select(dim + 1, torch.tensor(order, device=nib.device))
    shifts = torch.arange(0, 32, 4, device=nib.device, dtype=torch.int64)
    vshape = [1] * n.dim()
    vshape[dim + 1] = 8
    word = (n << shifts.view(vshape)).sum(dim + 1)
    return torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)


# --------------------------------------------------------------------------- GPTQ
def dequantize_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                    g_idx: torch.Tensor | None = None, group_size: int = 128) -> torch.Tensor:
    K = qweight.shape[0] * 8
    w = _unpack_int32(qweight, 0).float()                       # [K, N]
    z = _unpack_int32(qzeros, 1).float() + 1.0                  # [K/g, N]
    if g_idx is None:
        g_idx = torch.arange(K, device=qweight.device) // group_size
    g = g_idx.long()
    return ((w - z[g]) * scales.float()[g]).t().contiguous()    # [N, K]


def pack_gptq(w: torch.Tensor, group_size: int = 128):
    """Quantise ``w [N, K]`` to the GPTQ layout (asymmetric, per group of input channels)."""
    N, K = w.shape
    wt = w.float().t().reshape(K // group_size, group_size, N)
    lo, hi = wt.amin(1), wt.amax(1)
    scales = ((hi - lo) / 15.0).clamp_min(1e-8)
    zeros = (-lo / scales).round().clamp(1, 16)                 # stored as zero - 1 in 4 bits
    q = (wt / scales[:, None] + zeros[:, None]).round().clamp(0, 15)
    return (_pack_int32(q.reshape(K, N).to(torch.int32), 0), _pack_int32((zeros - 1).to(torch.int32), 1),
            scales.to(torch.float16))


# --------------------------------------------------------------------------- AWQ
def dequantize_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    K = qweight.shape[0]
    w = _unpack_int32(qweight, 1, _AWQ_ORDER).float()           # [K, N]
    z = _unpack_int32(qzeros, 1, _AWQ_ORDER).float()            # [K/g, N]
    g = torch.arange(K, device=qweight.device) // group_size
    return ((w - z[g]) * scales.float()[g]).t().contiguous()


def pack_awq(w: torch.Tensor, group_size: int = 128):
    N, K = w.shape
    wt = w.float().t().reshape(K // group_size, group_size, N)
    lo, hi = wt.amin(1), wt.amax(1)
    scales = ((hi - lo) / 15.0).clamp_min(1e-8)
    zeros = (-lo / scales).round().clamp(0, 15)
    q = (wt / scales[:, None] + zeros[:, None]).round().clamp(0, 15)
    return (_pack_int32(q.reshape(K, N).to(torch.int32), 1, _AWQ_ORDER),
            _pack_int32(zeros.to(torch.int32), 1, _AWQ_ORDER), scales.to(torch.float16))


# --------------------------------------------------------------------------- HQQ
def dequantize_hqq(w_q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, shape: tuple[int, int],
                   group_size: int = 64) -> torch.Tensor:
    N, K = shape
    packed = w_q.reshape(group_size // 2, -1).to(torch.uint8)   # [g/2, groups]
    q = torch.cat([(packed >> 4) & 0xF, packed & 0xF], 0).float()  # [g, groups]
    w = (q - zero.float().reshape(1, -1)) * scale.float().reshape(1, -1)
    return w.t().reshape(N, K).contiguous()


def pack_hqq(w: torch.Tensor, group_size: int = 64):
    N, K = w.shape
    g = w.float().reshape(-1, group_size).t()                   # [g, groups]
    lo, hi = g.amin(0), g.amax(0)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8)
    zero = -lo / scale
    q = (g / scale + zero).round().clamp(0, 15).to(torch.uint8)
    half = group_size // 2
    return ((q[:half] << 4) | q[half:]).reshape(-1), scale, zero


# --------------------------------------------------------------------------- to the fused kernel
def to_q4_linear(weight: torch.Tensor, bias: torch.Tensor | None = None):
    """Re-block a dequantised ``[N, K]`` weight as Q4_0 planes in a :class:`~ferrotorch_b200.ops.quant.Q4Linear`
    (the fused dequant-GEMM's input); a second rounding to symmetric 32-wide blocks."""
    from ..ops.quant import Q4Linear, requantize_q4_0

    nib, sc = requantize_q4_0(weight)
    return Q4Linear(nib, sc, bias)


# names of the reference's loaders (ferrotorch-llama/src/quant_loaders.rs:41-670)
dequantize_gptq_q4, dequantize_awq_q4, dequantize_hqq_q4_axis1 = dequantize_gptq, dequantize_awq, dequantize_hqq
hqq_q4_axis1_to_dense = dequantize_hqq


def hqq_state_dict_to_dense(sd: dict, dtype=torch.float32) -> dict:
    """Replace every HQQ-quantised linear of a state dict (keys ``<name>.W_q``, ``<name>.scale``,
    ``<name>.zero``, ``<name>.shape``) by a dense ``<name>.weight``; other entries pass through."""
    out, done = {}, set()
    for k in sd:
        if k.endswith(".W_q"):
            base = k[:-4]
            shape = tuple(int(v) for v in sd[base + ".shape"].tolist())
            out[base + ".weight"] = dequantize_hqq(sd[k], sd[base + ".scale"], sd[base + ".zero"], shape).to(dtype)
            done.update({k, base + ".scale", base + ".zero", base + ".shape"})
    out.update({k: v for k, v in sd.items() if k not in done})
    return out
