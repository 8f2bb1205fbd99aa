"""Speculative sampling (Leviathan et al., "Fast Inference from Transformers via Speculative
Decoding", algorithm 1): a cheap draft model proposes ``K`` tokens, the target model scores the
whole proposal in **one** forward pass, and a rejection step keeps a prefix such that the emitted
tokens are distributed exactly as if the target model had sampled them one by one.

The reference implements this over a small model interface (ferrotorch-llama/src/spec_decode.rs:
``ModelHandle`` :40-99 with ``forward_ids`` / ``forward_ids_all_positions`` / ``vocab_size``,
``LlamaHandle`` :101-163, ``SpecDecodeConfig`` :167-215, ``SpecDecodeOutput`` :218-238,
``speculative_decode`` :264): draft token ``x_j ~ q_j`` is accepted with probability
``min(1, p_j(x_j) / q_j(x_j))``; at the first rejection a token is drawn from the residual
``norm(max(0, p_j - q_j))`` and the round ends; if all ``K`` are accepted a bonus token is drawn from
``p_K``.  The greedy special case (keep the longest prefix on which the arg-maxes agree) lives in
:func:`ferrotorch_b200.models.generation.speculative_decode`.

Everything random comes from one seeded generator, so a ``(prompt, weights, seed)`` triple always
gives the same tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch

DEFAULT_SEED = 0xDEADBEEFCAFEBABE & 0x7FFFFFFFFFFFFFFF


class ModelHandle:
    """What speculative sampling needs from a model.  ``forward_ids(ids)`` returns the logits after
    the last position, ``forward_ids_all_positions(ids)`` the logits after every position in one
    pass (the default calls ``forward_ids`` per prefix: correct, quadratic)."""

    def forward_ids(self, ids: Sequence[int]) -> torch.Tensor:
        raise NotImplementedError

    def forward_ids_all_positions(self, ids: Sequence[int]) -> torch.Tensor:
        return torch.stack([self.forward_ids(ids[:j]) for j in range(1, len(ids) + 1)])

    def vocab_size(self) -> int:
        raise NotImplementedError


class LlamaHandle(ModelHandle):
    """A causal language model (``model(ids [1, S]) -> logits [1, S, V]``) as a :class:`ModelHandle`;
    all positions come from a single forward pass."""

    def __init__(self, model):
        self.model = model

    @torch.no_grad()
    def forward_ids_all_positions(self, ids):
        dev = next(self.model.parameters()).device
        t = torch.as_tensor(list(ids), dtype=torch.long, device=dev)[None]
        out = self.model(t)
        if out.dim() != 3 or out.shape[0] != 1 or out.shape[1] != t.shape[1]:
            raise ValueError("expected logits [1, %d, V], got %s" % (t.shape[1], tuple(out.shape)))
        return out[0].double()

    def forward_ids(self, ids):
        return self.forward_ids_all_positions(ids)[-1]

    def vocab_size(self) -> int:
        cfg = getattr(self.model, "config", None)
        return int(cfg.vocab_size) if cfg is not None else int(self.forward_ids([0]).shape[-1])


class FunctionHandle(ModelHandle):
    """``fn(ids) -> logits [V]`` as a handle (tests, n-gram or table drafts)."""

    def __init__(self, fn: Callable[[Sequence[int]], torch.Tensor], vocab: int):
        self.fn, self.vocab = fn, vocab

    def forward_ids(self, ids):
        return torch.as_tensor(self.fn(list(ids)), dtype=torch.float64)

    def vocab_size(self) -> int:
        return self.vocab


@dataclass
class SpecSamplingConfig:
    draft_k: int = 4                      # draft tokens proposed per target pass
    max_new_tokens: int = 64
    seed: int | None = None               # None = a fixed default, so that runs repeat
    eos_token_ids: list[int] = field(default_factory=list)
    temperature: float = 1.0              # applied to both models' logits

    def validate(self) -> None:
        if self.draft_k < 1:
            raise ValueError("SpecSamplingConfig: draft_k must be >= 1")
        if self.max_new_tokens < 1:
            raise ValueError("SpecSamplingConfig: max_new_tokens must be >= 1")
        if not self.temperature > 0:
            raise ValueError("SpecSamplingConfig: temperature must be > 0")


@dataclass
class SpecSamplingOutput:
    tokens: list[int]                     # generated ids, prompt excluded
    accepted_count: int
    proposed_count: int
    target_calls: int = 0

    def acceptance_rate(self) -> float:
        return self.accepted_count / self.proposed_count if self.proposed_count else 1.0


def _probs(logits: torch.Tensor, vocab: int, temperature: float, who: str) -> torch.Tensor:
    if logits.shape[-1] != vocab:
        raise ValueError("%s model returned %d logits, vocabulary is %d" % (who, logits.shape[-1], vocab))
    return torch.softmax(logits.double() / temperature, -1)


def _draw(probs: torch.Tensor, gen: torch.Generator) -> int:
    return int(torch.multinomial(probs, 1, generator=gen))


def residual_distribution(p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """``norm(max(0, p - q))``; when ``p == q`` everywhere (nothing left) the target's ``p``."""
    r = (p - q).clamp_min(0)
    s = r.sum()
    return r / s if float(s) > 0 else p


def speculative_sample(target: ModelHandle, draft: ModelHandle, prompt: Sequence[int], config: SpecSamplingConfig | None = None
                       ) -> SpecSamplingOutput:
    cfg = config or SpecSamplingConfig()
    cfg.validate()
    if len(prompt) == 0:
        raise ValueError("speculative_sample: empty prompt")
    V = target.vocab_size()
    if draft.vocab_size() != V:
        raise ValueError("target and draft vocabularies differ: %d vs %d" % (V, draft.vocab_size()))
    gen = torch.Generator().manual_seed((DEFAULT_SEED if cfg.seed is None else int(cfg.seed)) & 0x7FFFFFFFFFFFFFFF)
    ctx, out = list(prompt), []
    accepted = proposed = calls = 0
    stop = set(cfg.eos_token_ids)
    while len(out) < cfg.max_new_tokens:
        k = min(cfg.draft_k, cfg.max_new_tokens - len(out))
        drafted, q = [], []
        for _ in range(k):
            qj = _probs(draft.forward_ids(ctx + drafted), V, cfg.temperature, "draft")
            q.append(qj)
            drafted.append(_draw(qj, gen))
        allp = target.forward_ids_all_positions(ctx + drafted)
        calls += 1
        p = _probs(allp[len(ctx) - 1:], V, cfg.temperature, "target")          # p_0 .. p_k
        proposed += k
        emitted = []
        for j, x in enumerate(drafted):
            ratio = float(p[j, x] / q[j][x]) if float(q[j][x]) > 0 else 0.0
            if float(torch.rand((), generator=gen, dtype=torch.float64)) < min(1.0, ratio):
                emitted.append(x)
                accepted += 1
            else:
                emitted.append(_draw(residual_distribution(p[j], q[j]), gen))
                break
        else:
            emitted.append(_draw(p[k], gen))                                   # all accepted: one more for free
        for t in emitted:
            out.append(t)
            ctx.append(t)
            if t in stop or len(out) >= cfg.max_new_tokens:
                return SpecSamplingOutput(out, accepted, proposed, calls)
    return SpecSamplingOutput(out, accepted, proposed, calls)
