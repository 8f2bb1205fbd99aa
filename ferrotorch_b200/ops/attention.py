"""Differentiable flash attention (GQA, causal/full) on the tcgen05 kernels.

Forward: ``csrc/attn_fwd.cu``.  Backward: ``csrc/attn_bwd.cu`` (dK/dV kernel + dQ kernel that
recompute P from the saved log-sum-exp).  CPU tensors use the PyTorch reference.
"""
from __future__ import annotations

import torch

from .. import _native
from . import functional as F
from . import reference as ref

_i, _ll, _f, _vp = _native._i, _native._ll, _native._f, _native._vp
_native.register_protos({
    "ft_flash_attn_bwd": (_i, [_vp] * 10 + [_i] * 6 + [_ll] * 7 + [_f, _i, _i, _i, _vp]),
})


def native_bwd_available() -> bool:
    lib = _native.kernels(required=False)
    return lib is not None and hasattr(lib, "ft_flash_attn_bwd")


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, causal_offset):
        out, lse = F.flash_attn_fwd(q, k, v, causal, scale, causal_offset)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (causal, scale, causal_offset)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        causal, scale, causal_offset = ctx.cfg
        B, Sq, Hq, D = q.shape
        Sk, Hkv = k.shape[1], k.shape[2]
        dout = dout if dout.is_contiguous() else dout.contiguous()
        # gradients are written as one packed [B, S, Hq + 2 Hkv, D] buffer when q/k/v are
        # slices of a packed projection output (self-attention), so that the backward of the
        # slicing is free
        if Sq == Sk:
            dqkv = torch.empty((B, Sq, Hq + 2 * Hkv, D), device=q.device, dtype=q.dtype)
            dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        else:
            dq = torch.empty((B, Sq, Hq, D), device=q.device, dtype=q.dtype)
            dk = torch.empty((B, Sk, Hkv, D), device=q.device, dtype=q.dtype)
            dv = torch.empty_like(dk)
        sc = scale if scale is not None else D ** -0.5
        off = (Sk - Sq) if causal_offset is None else causal_offset
        lib = _native.kernels()
        rc = lib.ft_flash_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            F._get_scratch("attn_delta", 2 * B * Hq * Sq, q.device).data_ptr(),
            B, Sq, Sk, Hq, Hkv, D, F._tok_stride(q), F._tok_stride(k), F._tok_stride(v), Hq * D,
            F._tok_stride(dq), F._tok_stride(dk), F._tok_stride(dv), float(sc), int(causal), off,
            F._dev(q), F._stream())
        _native.check(rc, "ft_flash_attn_bwd")
        return dq, dk, dv, None, None, None


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
                    scale: float | None = None, causal_offset: int | None = None) -> torch.Tensor:
    """``softmax(q k^T * scale + mask) v`` for ``q [B,Sq,Hq,D]``, ``k/v [B,Sk,Hkv,D]``; returns
    ``[B,Sq,Hq,D]``.  ``Hq`` must be a multiple of ``Hkv`` (query head h uses kv head
    ``h // (Hq/Hkv)``, the ``repeat_kv`` order of ferrotorch-gpu/src/bf16.rs:2405-2410)."""
    native = q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)
    if not native:
        if q.is_cuda:
            # head dims without a native kernel: library attention, explicit and counted
            F.stats["attn_library"] = F.stats.get("attn_library", 0) + 1
            qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))
            o = torch.nn.functional.scaled_dot_product_attention(
                qt, kt, vt, is_causal=causal and q.shape[1] == k.shape[1], scale=scale,
                enable_gqa=q.shape[2] != k.shape[2])
            return o.transpose(1, 2)
        off = causal_offset
        return ref.attention(q, k, v, causal, scale, off)[0]
    return _FlashAttnFn.apply(q, k, v, causal, scale, causal_offset)
