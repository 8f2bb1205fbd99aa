"""Differentiable flash attention (GQA, causal/full) on the tcgen05 kernels.

Forward: ``csrc/attn_fwd.cu``.  Backward: ``csrc/attn_bwd.cu`` -- head_dim 128 runs one fused
kernel that recomputes P from the saved log-sum-exp once and produces dK, dV and (through an
fp32 accumulator) dQ; head_dim 64, or :func:`deterministic`, the dK/dV kernel + dQ kernel pair.
CPU tensors use the PyTorch reference.
"""
from __future__ import annotations

import torch

from .. import _native
from . import functional as F
from . import reference as ref

_i, _ll, _f, _vp = _native._i, _native._ll, _native._f, _native._vp
_native.register_protos({
    "ft_flash_attn_bwd": (_i, [_vp] * 11 + [_i] * 6 + [_ll] * 7 + [_f, _i, _i, _i, _vp]),
})


# The fused single-pass backward (head_dim 128) sums dQ over key tiles with fp32 atomic adds into
# a scratch accumulator; deterministic() switches back to the bit-reproducible two-pass kernels.
_FUSED_BWD = True


def deterministic(on: bool = True) -> bool:
    """Use the two-pass backward kernels (run-to-run identical dQ) instead of the fused one;
    returns the previous setting."""
    global _FUSED_BWD
    old, _FUSED_BWD = not _FUSED_BWD, not on
    return old


def _dq_scratch(B: int, S: int, Hq: int, D: int, device):
    if not _FUSED_BWD or D != 128:
        return None
    return F._get_scratch("attn_dq_acc", B * S * Hq * D, device).data_ptr()


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
            F._get_scratch("attn_delta", 2 * B * Hq * Sq, q.device).data_ptr(), _dq_scratch(B, Sq, Hq, D, q.device),
            B, Sq, Sk, Hq, Hkv, D, F._tok_stride(q), F._tok_stride(k), F._tok_stride(v), Hq * D,
            F._tok_stride(dq), F._tok_stride(dk), F._tok_stride(dv), float(sc), int(causal), off,
            F._dev(q), F._stream())
        _native.check(rc, "ft_flash_attn_bwd")
        return dq, dk, dv, None, None, None


def attention_block_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                             dout: torch.Tensor, causal: bool, scale: float | None = None):
    """Gradients of attention restricted to one key block when the softmax statistics are those
    of the **whole** key sequence: ``out`` and ``lse`` are the final output and log-sum-exp of the
    rows (over every key block), ``k / v`` one block.  ``P = exp(q k^T scale - lse)`` is then that
    block's share of the full probabilities and ``dS = P (dP - rowsum(dout * out))``; returns the
    block's contribution to ``dq`` and its ``dk``, ``dv``.  This is the step a ring (context
    parallel) backward repeats for every block it receives.  On a GPU with bf16 inputs and head
    dim 64 / 128 it is the flash backward kernel (it takes ``out`` and ``lse`` as inputs);
    elsewhere fp32 torch math."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    sc = scale if scale is not None else D ** -0.5
    if F.native_enabled() and q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and native_bwd_available():
        q, k, v, out, dout = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v, out, dout))
        lse = lse.float().contiguous()
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        rc = _native.kernels().ft_flash_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            F._get_scratch("attn_delta", 2 * B * Hq * Sq, q.device).data_ptr(), _dq_scratch(B, Sq, Hq, D, q.device),
            B, Sq, Sk, Hq, Hkv, D, F._tok_stride(q), F._tok_stride(k), F._tok_stride(v), Hq * D,
            F._tok_stride(dq), F._tok_stride(dk), F._tok_stride(dv), float(sc), int(causal), Sk - Sq,
            F._dev(q), F._stream())
        _native.check(rc, "ft_flash_attn_bwd")
        return dq, dk, dv
    g = Hq // Hkv
    qf, dof, of = (t.float().permute(0, 2, 1, 3) for t in (q, dout, out))          # [B, Hq, Sq, D]
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)                  # [B, Hq, Sk, D]
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sc
    if causal:
        i = torch.arange(Sq, device=q.device)[:, None] + (Sk - Sq)
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    p = torch.exp(s - lse.float().unsqueeze(-1))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (torch.matmul(dof, vf.transpose(-1, -2)) - delta)
    dq = torch.matmul(ds, kf) * sc
    dk = (torch.matmul(ds.transpose(-1, -2), qf) * sc).reshape(B, Hkv, g, Sk, D).sum(2)
    dv = torch.matmul(p.transpose(-1, -2), dof).reshape(B, Hkv, g, Sk, D).sum(2)
    return (dq.permute(0, 2, 1, 3).to(q.dtype), dk.permute(0, 2, 1, 3).to(k.dtype), dv.permute(0, 2, 1, 3).to(v.dtype))


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True,
                    scale: float | None = None, causal_offset: int | None = None) -> torch.Tensor:
    """``softmax(q k^T * scale + mask) v`` for ``q [B,Sq,Hq,D]``, ``k/v [B,Sk,Hkv,D]``; returns
    ``[B,Sq,Hq,D]``.  ``Hq`` must be a multiple of ``Hkv`` (query head h uses kv head
    ``h // (Hq/Hkv)``, the ``repeat_kv`` order of ferrotorch-gpu/src/bf16.rs:2405-2410)."""
    native = F.native_enabled() and q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128)
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


class _QKVAttentionFn(torch.autograd.Function):
    """QKV projection + in-place RoPE + flash attention as one autograd node.

    Keeping the packed ``[B, S, Hq + 2 Hkv, D]`` buffer private to the node means RoPE runs in
    place with no autograd bookkeeping and the backward writes one packed gradient buffer that
    feeds the projection's dgrad / wgrad GEMMs directly (no per-slice zero-fill and add)."""

    @staticmethod
    def forward(ctx, x, w, bias, cos, sin, Hq, Hkv, D, causal, interleaved):
        B, S, H = x.shape
        x2 = x.reshape(B * S, H)
        qkv = torch.empty((B, S, Hq + 2 * Hkv, D), device=x.device, dtype=x.dtype)
        F.gemm_nt(x2, w, bias=bias, out=qkv.view(B * S, -1))
        if cos is not None:
            F._rope_launch(qkv, cos, sin, None, Hq + Hkv, S, 0, interleaved, False)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        out, lse = F.flash_attn_fwd(q, k, v, causal)
        ctx.save_for_backward(x2, w, qkv, out, lse, cos if cos is not None else x.new_empty(0),
                              sin if sin is not None else x.new_empty(0))
        ctx.cfg = (Hq, Hkv, D, causal, interleaved, bias is not None, cos is not None, x.shape)
        return out.view(B, S, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        x2, w, qkv, out, lse, cos, sin = ctx.saved_tensors
        Hq, Hkv, D, causal, interleaved, has_bias, has_rope, xshape = ctx.cfg
        B, S = qkv.shape[0], qkv.shape[1]
        dout = dout.reshape(B, S, Hq, D)
        dout = dout if dout.is_contiguous() else dout.contiguous()
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        ld = (Hq + 2 * Hkv) * D
        lib = _native.kernels()
        rc = lib.ft_flash_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            F._get_scratch("attn_delta", 2 * B * Hq * S, q.device).data_ptr(), _dq_scratch(B, S, Hq, D, q.device),
            B, S, S, Hq, Hkv, D, ld, ld, ld, Hq * D, ld, ld, ld, float(D ** -0.5), int(causal), 0,
            F._dev(q), F._stream())
        _native.check(rc, "ft_flash_attn_bwd")
        if has_rope:
            F._rope_launch(dqkv, cos, sin, None, Hq + Hkv, S, 0, interleaved, True)
        d2 = dqkv.view(B * S, -1)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = F.gemm_nt(d2, w.t()).view(xshape)
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                F.gemm_nt(d2.t(), x2.t(), out=mg, accumulate=True)
                hook = getattr(w, "grad_ready_hook", None)
                if hook is not None:
                    hook(w)
            else:
                dw = F.gemm_nt(d2.t(), x2.t())
        if has_bias and ctx.needs_input_grad[2]:
            db = d2.float().sum(0).to(d2.dtype)
        return dx, dw, db, None, None, None, None, None, None, None


def qkv_attention(x: torch.Tensor, w_qkv: torch.Tensor, bias: torch.Tensor | None, cos, sin, *,
                  n_heads: int, n_kv_heads: int, head_dim: int, causal: bool = True,
                  interleaved: bool = False) -> torch.Tensor:
    """Self-attention core from the normed hidden states: ``attn(rope(x W_qkv^T))`` -> ``[B, S, Hq*D]``."""
    if F.native_enabled() and x.is_cuda and x.dtype == torch.bfloat16 and head_dim in (64, 128):
        return _QKVAttentionFn.apply(x, w_qkv, bias, cos, sin, n_heads, n_kv_heads, head_dim, causal,
                                     interleaved)
    B, S, _ = x.shape
    qkv = torch.nn.functional.linear(x, w_qkv, bias).view(B, S, n_heads + 2 * n_kv_heads, head_dim)
    if cos is not None:
        qkv = F.rope_(qkv, cos, sin, n_rot_heads=n_heads + n_kv_heads, seq_len=S, interleaved=interleaved)
    q, k, v = qkv[:, :, :n_heads], qkv[:, :, n_heads:n_heads + n_kv_heads], qkv[:, :, n_heads + n_kv_heads:]
    return flash_attention(q, k, v, causal=causal).reshape(B, S, n_heads * head_dim)


class _PackedAttentionFn(torch.autograd.Function):
    """In-place RoPE + flash attention on an already projected packed ``[B, S, Hq + 2 Hkv, D]``
    buffer (the tensor-parallel block produces it with the fused all-gather GEMM).  The buffer is
    rotated in place and kept for the backward; the gradient comes back packed the same way."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, Hq, Hkv, D, causal, interleaved):
        B, S = qkv.shape[0], qkv.shape[1]
        if cos is not None:
            F._rope_launch(qkv, cos, sin, None, Hq + Hkv, S, 0, interleaved, False)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        out, lse = F.flash_attn_fwd(q, k, v, causal)
        ctx.save_for_backward(qkv, out, lse, cos if cos is not None else qkv.new_empty(0),
                              sin if sin is not None else qkv.new_empty(0))
        ctx.cfg = (Hq, Hkv, D, causal, interleaved, cos is not None)
        return out.view(B, S, Hq * D)

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, cos, sin = ctx.saved_tensors
        Hq, Hkv, D, causal, interleaved, has_rope = ctx.cfg
        B, S = qkv.shape[0], qkv.shape[1]
        dout = dout.reshape(B, S, Hq, D)
        dout = dout if dout.is_contiguous() else dout.contiguous()
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :Hq], dqkv[:, :, Hq:Hq + Hkv], dqkv[:, :, Hq + Hkv:]
        ld = (Hq + 2 * Hkv) * D
        rc = _native.kernels().ft_flash_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
            F._get_scratch("attn_delta", 2 * B * Hq * S, q.device).data_ptr(), _dq_scratch(B, S, Hq, D, q.device),
            B, S, S, Hq, Hkv, D, ld, ld, ld, Hq * D, ld, ld, ld, float(D ** -0.5), int(causal), 0,
            F._dev(q), F._stream())
        _native.check(rc, "ft_flash_attn_bwd")
        if has_rope:
            F._rope_launch(dqkv, cos, sin, None, Hq + Hkv, S, 0, interleaved, True)
        return dqkv, None, None, None, None, None, None, None


def packed_attention(qkv: torch.Tensor, cos, sin, *, n_heads: int, n_kv_heads: int, head_dim: int,
                     causal: bool = True, interleaved: bool = False) -> torch.Tensor:
    """``attn(rope(qkv))`` for a packed projection output ``[B, S, Hq + 2 Hkv, D]`` -> ``[B, S, Hq*D]``.
    On the native path ``qkv`` is rotated in place."""
    B, S = qkv.shape[0], qkv.shape[1]
    if F.native_enabled() and qkv.is_cuda and qkv.dtype == torch.bfloat16 and head_dim in (64, 128) \
            and qkv.is_contiguous():
        return _PackedAttentionFn.apply(qkv, cos, sin, n_heads, n_kv_heads, head_dim, causal, interleaved)
    if cos is not None:
        qkv = F.rope_(qkv, cos, sin, n_rot_heads=n_heads + n_kv_heads, seq_len=S, interleaved=interleaved)
    q, k, v = qkv[:, :, :n_heads], qkv[:, :, n_heads:n_heads + n_kv_heads], qkv[:, :, n_heads + n_kv_heads:]
    return flash_attention(q, k, v, causal=causal).reshape(B, S, n_heads * head_dim)
