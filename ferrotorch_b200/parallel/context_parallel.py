"""Context parallelism for long sequences: ring attention and Ulysses (all-to-all) attention over
any :class:`~.backend.Group`, forward and backward.

The reference has neither (its sequence scaling is single-device: RoPE scaling, tiled attention,
KV caches).  Both schemes are outer loops around an attention function that returns the
log-sum-exp of its rows, which the kernels here do (``ops.functional.flash_attn_fwd`` on a GPU,
``ops.reference.attention`` anywhere): partial results over different key blocks merge exactly.

Sequence layout: rank r holds the contiguous tokens ``[r * S_loc, (r + 1) * S_loc)``.

Backward of the ring: the key / value blocks go round once more, each with an fp32 accumulator for
its ``dk / dv``; for the block it currently holds a rank runs
:func:`~ferrotorch_b200.ops.attention.attention_block_backward` (probabilities rebuilt from the
**global** log-sum-exp, so the pieces add up to the exact gradient), adds to its own ``dq`` and to
the travelling accumulator, and after ``W`` hops every accumulator is back at its owner.  Ulysses
is differentiable through its two all-to-alls (an all-to-all is its own adjoint).
"""
from __future__ import annotations

import torch

from ..ops import reference as ref
from .backend import Group
from .ring import _exchange


def merge_attention(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor):
    """Combine attention over two disjoint key sets: ``o [B, S, H, D]``, ``lse [B, H, S]``.  With
    ``w_i = exp(lse_i - logaddexp(lse_1, lse_2))`` the result is ``w_1 o_1 + w_2 o_2``."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).transpose(1, 2).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).transpose(1, 2).unsqueeze(-1)
    return (o1.float() * w1 + o2.float() * w2).to(o1.dtype), lse


def _default_attn(q, k, v, causal):
    return ref.attention(q, k, v, causal=causal)


def _default_block_bwd(q, k, v, out, lse, dout, causal):
    from ..ops.attention import attention_block_backward

    return attention_block_backward(q, k, v, out, lse, dout, causal)


def _ring_forward(q, k, v, group: Group, causal: bool, attn_fn):
    W, r = group.world_size, group.rank
    out, lse = attn_fn(q, k, v, causal)
    if W == 1:
        return out, lse
    right, left = (r + 1) % W, (r - 1) % W
    kv = torch.stack([k, v]).contiguous()
    for s in range(1, W):
        nxt = torch.empty_like(kv)
        _exchange(group, kv, right, nxt, left)
        kv = nxt
        src = (r - s) % W                       # whose block this is
        if causal and src > r:
            continue                            # entirely in the future of every local query
        o2, l2 = attn_fn(q, kv[0], kv[1], False)
        out, lse = merge_attention(out, lse, o2, l2)
    return out, lse


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, group, causal, attn_fn, bwd_fn):
        with torch.no_grad():
            out, lse = _ring_forward(q, k, v, group, causal, attn_fn)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (group, causal, bwd_fn)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        group, causal, bwd_fn = ctx.cfg
        W, r = group.world_size, group.rank
        right, left = (r + 1) % W, (r - 1) % W
        dout = dout.contiguous()
        dq = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
        kv = torch.stack([k, v]).contiguous()
        dkv = torch.zeros(kv.shape, device=q.device, dtype=torch.float32)   # travels with its block
        for s in range(W):
            src = (r - s) % W
            if not (causal and src > r):
                dq_p, dk_p, dv_p = bwd_fn(q, kv[0], kv[1], out, lse, dout, causal and s == 0)
                dq += dq_p.float()
                dkv[0] += dk_p.float()
                dkv[1] += dv_p.float()
            if W > 1:
                # the block moves on with its accumulator; after the last hop it is home again
                nxt_d = torch.empty_like(dkv)
                _exchange(group, dkv, right, nxt_d, left)
                dkv = nxt_d
                if s + 1 < W:
                    nxt = torch.empty_like(kv)
                    _exchange(group, kv, right, nxt, left)
                    kv = nxt
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Group, causal: bool = True,
                   attn_fn=None, block_bwd_fn=None) -> torch.Tensor:
    """Attention of this rank's queries over the whole sequence.  ``q [B, S_loc, Hq, D]``,
    ``k / v [B, S_loc, Hkv, D]`` are the local shards; the key / value blocks travel round the ring
    (W - 1 exchanges of one block each) while every rank attends to the block it currently holds.
    Under a causal mask a block from a later rank is skipped, the own block is attended causally and
    earlier blocks fully.  ``attn_fn(q, k, v, causal) -> (out, lse)`` defaults to the fp32 reference;
    ``block_bwd_fn(q, k, v, out, lse, dout, causal) -> (dq, dk, dv)`` to
    ``ops.attention.attention_block_backward``.  Differentiable in q, k and v."""
    attn_fn = attn_fn or _default_attn
    if not (q.requires_grad or k.requires_grad or v.requires_grad) or not torch.is_grad_enabled():
        return _ring_forward(q, k, v, group, causal, attn_fn)[0]
    return _RingAttention.apply(q, k, v, group, causal, attn_fn, block_bwd_fn or _default_block_bwd)


class _AllToAll(torch.autograd.Function):
    """``group.all_to_all`` on ``[W, n]`` rows; the gradient is the same exchange of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return group.all_to_all(x.contiguous())

    @staticmethod
    def backward(ctx, g):
        return ctx.group.all_to_all(g.contiguous()), None


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Group, causal: bool = True,
                      attn_fn=None) -> torch.Tensor:
    """DeepSpeed-Ulysses: one all-to-all turns the sequence sharding into a head sharding (every rank
    gets the whole sequence for ``H / W`` heads), attention runs locally, a second all-to-all turns
    it back.  Needs ``Hq % W == 0`` and ``Hkv % W == 0``; moves ``O(S H D / W)`` per rank instead of
    the ring's ``O(S H D)``, but cannot use more ranks than there are KV heads.  Differentiable
    when ``attn_fn`` is (the default reference and ``ops.attention.flash_attention`` both are)."""
    attn_fn = attn_fn or _default_attn
    W = group.world_size
    if W == 1:
        return attn_fn(q, k, v, causal)[0]
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if Hq % W or Hkv % W:
        raise ValueError("ulysses_attention: %d query / %d key-value heads do not divide by %d ranks" % (Hq, Hkv, W))

    def seq_to_heads(x):                        # [B, S_loc, H, D] -> [B, W * S_loc, H / W, D]
        H = x.shape[2]
        parts = x.reshape(B, S, W, H // W, D).permute(2, 0, 1, 3, 4).contiguous()      # destination rank first
        got = _AllToAll.apply(parts.reshape(W, -1), group).reshape(W, B, S, H // W, D)  # source rank = sequence block
        return got.permute(1, 0, 2, 3, 4).reshape(B, W * S, H // W, D)

    def heads_to_seq(x):                        # [B, W * S_loc, H / W, D] -> [B, S_loc, H, D]
        Hl = x.shape[2]
        parts = x.reshape(B, W, S, Hl, D).permute(1, 0, 2, 3, 4).contiguous()          # destination = sequence block
        got = _AllToAll.apply(parts.reshape(W, -1), group).reshape(W, B, S, Hl, D)      # source rank = head group
        return got.permute(1, 2, 0, 3, 4).reshape(B, S, W * Hl, D)

    res = attn_fn(seq_to_heads(q), seq_to_heads(k), seq_to_heads(v), causal)
    o = res[0] if isinstance(res, tuple) else res
    return heads_to_seq(o.contiguous())
