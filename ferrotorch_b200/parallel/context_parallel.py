"""Context parallelism for long sequences: ring attention and Ulysses (all-to-all) attention over
any :class:`~.backend.Group`.  Forward only -- the long-context prefill / evaluation path.

The reference has neither (its sequence scaling is single-device: RoPE scaling, tiled attention,
KV caches).  Both schemes are outer loops around an attention function that returns the
log-sum-exp of its rows, which the kernels here do (``ops.functional.flash_attn_fwd`` on a GPU,
``ops.reference.attention`` anywhere): partial results over different key blocks merge exactly.

Sequence layout: rank r holds the contiguous tokens ``[r * S_loc, (r + 1) * S_loc)``.
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


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Group, causal: bool = True,
                   attn_fn=None) -> torch.Tensor:
    """Attention of this rank's queries over the whole sequence.  ``q [B, S_loc, Hq, D]``,
    ``k / v [B, S_loc, Hkv, D]`` are the local shards; the key / value blocks travel round the ring
    (W - 1 exchanges of one block each) while every rank attends to the block it currently holds.
    Under a causal mask a block from a later rank is skipped, the own block is attended causally and
    earlier blocks fully.  ``attn_fn(q, k, v, causal) -> (out, lse)`` defaults to the fp32 reference."""
    attn_fn = attn_fn or _default_attn
    W, r = group.world_size, group.rank
    out, lse = attn_fn(q, k, v, causal)
    if W == 1:
        return out
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
    return out


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group: Group, causal: bool = True,
                      attn_fn=None) -> torch.Tensor:
    """DeepSpeed-Ulysses: one all-to-all turns the sequence sharding into a head sharding (every rank
    gets the whole sequence for ``H / W`` heads), attention runs locally, a second all-to-all turns
    it back.  Needs ``Hq % W == 0`` and ``Hkv % W == 0``; moves ``O(S H D / W)`` per rank instead of
    the ring's ``O(S H D)``, but cannot use more ranks than there are KV heads."""
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
        got = group.all_to_all(parts.reshape(W, -1)).reshape(W, B, S, H // W, D)       # source rank = sequence block
        return got.permute(1, 0, 2, 3, 4).reshape(B, W * S, H // W, D)

    def heads_to_seq(x):                        # [B, W * S_loc, H / W, D] -> [B, S_loc, H, D]
        Hl = x.shape[2]
        parts = x.reshape(B, W, S, Hl, D).permute(1, 0, 2, 3, 4).contiguous()          # destination = sequence block
        got = group.all_to_all(parts.reshape(W, -1)).reshape(W, B, S, Hl, D)           # source rank = head group
        return got.permute(1, 2, 0, 3, 4).reshape(B, S, W * Hl, D)

    o, _ = attn_fn(seq_to_heads(q), seq_to_heads(k), seq_to_heads(v), causal)
    return heads_to_seq(o.contiguous())
