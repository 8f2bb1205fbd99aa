"""Sampling from logits that are sharded over the vocabulary (the lm_head of a tensor-parallel
model): temperature, top-k and nucleus (top-p) sampling without ever gathering the full
``[B, V]`` logits.

The reference samples on one device from full logits (ferrotorch-llama/src/generation.rs:238-345:
temperature, top-k, top-p, then a multinomial draw).  With the vocabulary split over ``W`` ranks
the same distribution is obtained from three small exchanges:

1. every rank finds its ``k`` best local logits and the ranks all-gather ``(value, global id)``
   pairs: ``W * k`` candidates per row contain the global top ``k``;
2. an all-reduce of the row maximum and of ``sum(exp(z - max))`` gives the normaliser of the
   **full** softmax, so a candidate's probability is exact;
3. the nucleus is cut on the sorted candidates; the draw is an inverse-CDF look-up with one
   uniform number per row from a generator seeded identically on every rank, so that every rank
   picks the same token without another exchange.

The result equals :func:`sample_reference` (single-device top-k / top-p on the full logits with the
same uniform numbers) whenever the kept set fits in the candidates: always for ``top_k <= k``, and
for nucleus sampling as long as the nucleus has at most ``k`` tokens per shard; if a row's nucleus
is not complete within the candidates the call repeats with a four times larger ``k`` (bounded by
the shard size, at which point all logits are candidates).
"""
from __future__ import annotations

import torch

from .backend import Group


def _inverse_cdf_pick(probs: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """Row-wise: the first index whose cumulative probability exceeds ``u * total``."""
    c = probs.cumsum(-1)
    idx = (c <= (u * c[:, -1:])).sum(-1)
    return idx.clamp(max=probs.shape[-1] - 1)


def _keep_mask(sorted_probs: torch.Tensor, top_k: int, top_p: float) -> torch.Tensor:
    """Which entries of rows sorted by descending probability survive top-k then top-p (the token
    that crosses the threshold is kept, as in ``filter_top_k_top_p``)."""
    keep = torch.ones_like(sorted_probs, dtype=torch.bool)
    if top_k:
        keep[:, top_k:] = False
    if top_p < 1.0:
        p = sorted_probs * keep
        if top_k:
            p = p / p.sum(-1, keepdim=True)             # top-p acts on the distribution left by top-k
        # without top-k the entries are probabilities of the full softmax already (a candidate list
        # does not sum to one and must not be renormalised)
        keep &= (p.cumsum(-1) - p) <= top_p
    return keep


def sample_reference(logits: torch.Tensor, u: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    """Single-device oracle: full ``logits [B, V]``, one uniform ``u [B, 1]`` per row."""
    z = logits.float() / temperature
    srt, idx = z.sort(dim=-1, descending=True, stable=True)
    probs = srt.softmax(-1)
    keep = _keep_mask(probs, top_k, top_p)
    pick = _inverse_cdf_pick(probs * keep, u)
    return idx.gather(1, pick[:, None])[:, 0]


def sample_vocab_parallel(local_logits: torch.Tensor, group: Group, vocab_offset: int, u: torch.Tensor, temperature: float = 1.0,
                          top_k: int = 0, top_p: float = 1.0, candidates: int = 64, valid: int | None = None) -> torch.Tensor:
    """``local_logits [B, V_loc]``: this rank's vocabulary shard (global ids ``vocab_offset ..``;
    only the first ``valid`` columns are real when the last shard is padded).  ``u [B, 1]`` uniform
    numbers, the same on every rank.  Returns the sampled global token ids ``[B]`` (the same on
    every rank).  ``temperature == 0`` is greedy."""
    z = local_logits.float()
    if valid is not None and valid < z.shape[1]:
        z = z.clone()
        z[:, valid:] = float("-inf")
    B, Vl = z.shape
    W = group.world_size
    if temperature == 0.0:
        temperature, top_k = 1.0, 1
    z = z / temperature
    # the normaliser of the full softmax
    m = z.max(-1).values
    gm = group.all_gather(m[None]).max(0).values if W > 1 else m
    se = torch.exp(z - gm[:, None]).sum(-1)
    if W > 1:
        se = group.all_reduce(se.clone(), "sum")
    k = min(Vl, max(candidates, top_k))
    if not top_k and top_p >= 1.0:
        k = Vl                                      # unrestricted sampling needs every logit
    while True:
        val, idx = z.topk(k, -1)
        pair = torch.stack([val, (idx + vocab_offset).to(val.dtype)], 0)                    # [2, B, k]
        gathered = group.all_gather(pair[None]) if W > 1 else pair[None]                     # [W, 2, B, k]
        cval = gathered[:, 0].permute(1, 0, 2).reshape(B, W * k)
        cid = gathered[:, 1].permute(1, 0, 2).reshape(B, W * k).long()
        # one global order: by value, ties by the lower token id (what a stable sort of the full row gives)
        order = torch.argsort(cid, dim=-1, stable=True)
        cval, cid = cval.gather(1, order), cid.gather(1, order)
        order = torch.argsort(cval, dim=-1, descending=True, stable=True)
        cval, cid = cval.gather(1, order), cid.gather(1, order)
        probs = torch.exp(cval - gm[:, None]) / se[:, None]
        keep = _keep_mask(probs, top_k, top_p)
        if k >= Vl or top_p >= 1.0 or top_k:
            break       # all logits are candidates / the global top-k (and a nucleus inside it) is always among them
        # Every token strictly better than the weakest candidate of some shard is a candidate, so that
        # prefix of the sorted candidates is the true global order with exact probabilities; the
        # nucleus is right if it is cut inside that prefix.
        floor = gathered[:, 0, :, -1].max(0).values                                          # [B]
        safe = (cval > floor[:, None]).sum(-1)
        if bool((keep.sum(-1) <= safe).all()):
            break
        k = min(Vl, 4 * k)
    pick = _inverse_cdf_pick(probs * keep, u)
    return cid.gather(1, pick[:, None])[:, 0]


def shared_uniform(batch: int, seed: int, step: int, device="cpu") -> torch.Tensor:
    """``[batch, 1]`` uniform numbers that every rank reproduces from ``(seed, step)``."""
    g = torch.Generator().manual_seed((int(seed) * 1_000_003 + int(step)) & 0x7FFFFFFFFFFFFFFF)
    return torch.rand((batch, 1), generator=g).to(device)
