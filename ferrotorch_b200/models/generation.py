"""Text generation: sampling (greedy / temperature / top-k / top-p / repetition penalty), streaming,
beam search and speculative decoding over any causal LM with per-layer KV caches.

Reference: ``GenerationConfig`` and ``generate_with_streamer`` (ferrotorch-llama/src/generation.rs:20-49,
145-228: repetition penalty -> temperature -> top-k -> top-p -> sample), ``beam_search``
(generation.rs:404), ``speculative_decode`` (spec_decode.rs:101-264).  The reference's ``generate``
re-runs the whole sequence every step; here prefill fills the KV caches once and each step feeds
one token (``forward_one_with_cache``, model.rs:284).  Sampling runs on the logits' device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass
class GenerationConfig:
    max_new_tokens: int = 32
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    do_sample: bool = False
    eos_token_id: int | None = None
    seed: int | None = None
    eos_token_ids: tuple = ()          # any of these ends a sequence (generation.rs:39-41)

    # named constructors of the reference (generation.rs:65-92)
    @classmethod
    def greedy(cls, max_new_tokens: int) -> "GenerationConfig":
        return cls(max_new_tokens=max_new_tokens, temperature=0.0)

    @classmethod
    def sampling(cls, max_new_tokens: int, temperature: float) -> "GenerationConfig":
        return cls(max_new_tokens=max_new_tokens, temperature=temperature, do_sample=temperature > 0)

    @classmethod
    def nucleus(cls, max_new_tokens: int, top_p: float, temperature: float) -> "GenerationConfig":
        return cls(max_new_tokens=max_new_tokens, temperature=temperature, top_p=top_p, do_sample=temperature > 0)

    def stop_ids(self) -> list[int]:
        ids = list(self.eos_token_ids)
        if self.eos_token_id is not None and self.eos_token_id not in ids:
            ids.append(self.eos_token_id)
        return ids

    def validate(self) -> None:
        """The argument checks of generation.rs:108-135."""
        if self.temperature < 0.0:
            raise ValueError("generate: temperature must be >= 0, got %r" % (self.temperature,))
        if not 0.0 <= self.top_p <= 1.0:
            raise ValueError("generate: top_p must be in [0, 1], got %r" % (self.top_p,))
        if self.repetition_penalty <= 0.0:
            raise ValueError("generate: repetition_penalty must be > 0, got %r" % (self.repetition_penalty,))


def apply_repetition_penalty(logits: torch.Tensor, prev_tokens: torch.Tensor, penalty: float) -> torch.Tensor:
    """Divide positive / multiply negative logits of already generated tokens by ``penalty``."""
    if penalty == 1.0 or prev_tokens.numel() == 0:
        return logits
    picked = logits.gather(-1, prev_tokens)
    picked = torch.where(picked > 0, picked / penalty, picked * penalty)
    return logits.scatter(-1, prev_tokens, picked)


def filter_top_k_top_p(logits: torch.Tensor, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    if top_k and top_k < logits.shape[-1]:
        kth = logits.topk(top_k, dim=-1).values[..., -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p < 1.0:
        srt, idx = logits.sort(dim=-1, descending=True)
        probs = srt.softmax(-1)
        remove = probs.cumsum(-1) - probs > top_p      # keep the token that crosses the threshold
        srt = srt.masked_fill(remove, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return logits


def sample_next(logits: torch.Tensor, cfg: GenerationConfig, prev_tokens: torch.Tensor | None = None,
                generator: torch.Generator | None = None) -> torch.Tensor:
    """``logits [B, V]`` -> token ids ``[B]``."""
    logits = logits.float()
    if prev_tokens is not None:
        logits = apply_repetition_penalty(logits, prev_tokens, cfg.repetition_penalty)
    if not cfg.do_sample or cfg.temperature == 0.0:
        return logits.argmax(-1)
    logits = filter_top_k_top_p(logits / cfg.temperature, cfg.top_k, cfg.top_p)
    return torch.multinomial(logits.softmax(-1), 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, cfg: GenerationConfig | None = None,
             streamer: Callable[[torch.Tensor], None] | None = None,
             logits_processor: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] | None = None) -> torch.Tensor:
    """``input_ids [B, S]`` -> ``[B, S + new]``.  ``model(ids, caches=..., last_token_only=True)`` must
    return logits and append to the caches it is given (``model.make_caches``).
    ``logits_processor(generated_ids [B, n], logits [B, V]) -> logits`` runs before sampling, e.g. a
    :class:`GrammarLogitsProcessor` for grammar-constrained decoding
    (ferrotorch-llama/src/gpu_gguf.rs:444 ``apply_grammar_mask_gpu`` masks the logits the same way)."""
    cfg = cfg or GenerationConfig()
    cfg.validate()
    if input_ids.dim() != 2 or input_ids.shape[1] == 0:
        raise ValueError("generate: input_ids must be [B, S] with S >= 1")
    B, S = input_ids.shape
    dev = input_ids.device
    stops = cfg.stop_ids()
    stop_t = torch.tensor(stops, device=dev, dtype=input_ids.dtype) if stops else None
    gen = None
    if cfg.seed is not None:
        gen = torch.Generator(device=dev).manual_seed(cfg.seed)
    caches = model.make_caches(B, S + cfg.max_new_tokens, device=dev, dtype=next(model.parameters()).dtype)
    logits = model(input_ids, caches=caches, last_token_only=True)[:, -1]
    out = input_ids
    done = torch.zeros(B, dtype=torch.bool, device=dev)
    for _ in range(cfg.max_new_tokens):
        if logits_processor is not None:
            logits = logits_processor(out[:, S:], logits.float())
        tok = sample_next(logits, cfg, out, gen)
        if stop_t is not None:
            tok = torch.where(done, torch.full_like(tok, stops[0]), tok)   # finished rows are padded with a stop id
            done |= (tok[:, None] == stop_t[None]).any(-1)
        out = torch.cat([out, tok[:, None]], dim=1)
        if streamer is not None and streamer(tok) is False:     # a streamer that returns False stops the run
            break
        if stop_t is not None and bool(done.all()):
            break
        logits = model(tok[:, None], caches=caches, last_token_only=True)[:, -1]
    return out


# ---- the sampling primitives under the reference's names (generation.rs:230-345), on tensors
def apply_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    if temperature <= 0:
        raise ValueError("apply_temperature: temperature must be > 0 (use argmax for greedy decoding)")
    return logits / temperature


def top_k_filter(logits: torch.Tensor, k: int) -> torch.Tensor:
    return filter_top_k_top_p(logits, top_k=k)


def top_p_filter(logits: torch.Tensor, p: float) -> torch.Tensor:
    return filter_top_k_top_p(logits, top_p=p)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    return logits.argmax(-1)


def sample_softmax(logits: torch.Tensor, generator: torch.Generator | None = None) -> torch.Tensor:
    return torch.multinomial(logits.float().softmax(-1), 1, generator=generator).squeeze(-1)


def generate_with_streamer(model, input_ids: torch.Tensor, cfg: GenerationConfig | None, streamer, **kw) -> torch.Tensor:
    """:func:`generate` with the streamer as a required argument: it sees every new token ``[B]``
    and stops the run by returning ``False``."""
    return generate(model, input_ids, cfg, streamer=streamer, **kw)


@dataclass
class SpecDecodeConfig:
    max_new_tokens: int = 32
    gamma: int = 4                       # draft tokens proposed per target pass
    eos_token_id: int | None = None

    def validate(self) -> None:
        if self.gamma < 1:
            raise ValueError("SpecDecodeConfig: gamma (draft tokens per pass) must be >= 1")
        if self.max_new_tokens < 1:
            raise ValueError("SpecDecodeConfig: max_new_tokens must be >= 1")


@dataclass
class SpecDecodeOutput:
    tokens: torch.Tensor
    proposed: int
    accepted: int
    target_calls: int

    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0


def speculative_decode_with_config(target, draft, input_ids: torch.Tensor, cfg: SpecDecodeConfig) -> SpecDecodeOutput:
    cfg.validate()
    ids, st = speculative_decode(target, draft, input_ids, cfg.max_new_tokens, cfg.gamma, cfg.eos_token_id)
    return SpecDecodeOutput(ids, st["proposed"], st["accepted"], st["target_calls"])


class GrammarLogitsProcessor:
    """Mask the logits so that every sequence stays a valid prefix of the grammar (and may only
    end once it is complete).  ``vocab[i]`` is the text of token ``i``; the per-step mask is built
    on the host from the grammar state and applied on the logits' device."""

    def __init__(self, grammar, vocab: list[str], eos_token_id: int | None = None):
        self.grammar, self.vocab, self.eos = grammar, vocab, eos_token_id

    def __call__(self, generated: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        from ..utils.text import apply_token_mask, token_mask

        rows = []
        for ids in generated.tolist():
            text = "".join(self.vocab[t] for t in ids if t != self.eos)
            rows.append(token_mask(self.grammar, text, self.vocab, self.eos))
        return apply_token_mask(logits, torch.stack(rows))


@torch.no_grad()
def beam_search(model, input_ids: torch.Tensor, num_beams: int = 4, max_new_tokens: int = 16,
                length_penalty: float = 1.0, eos_token_id: int | None = None) -> torch.Tensor:
    """Beam search for one prompt ``[1, S]``; returns the best sequence ``[1, S + n]``.  Hypotheses
    are re-scored by re-running the prefix (simple and exact; beams are few)."""
    assert input_ids.shape[0] == 1
    beams = [(0.0, input_ids, False)]
    for _ in range(max_new_tokens):
        cand = []
        for score, ids, fin in beams:
            if fin:
                cand.append((score, ids, True))
                continue
            logp = model(ids, last_token_only=True)[:, -1].float().log_softmax(-1)[0]
            top = logp.topk(num_beams)
            for lp, t in zip(top.values.tolist(), top.indices.tolist()):
                cand.append((score + lp, torch.cat([ids, ids.new_tensor([[t]])], 1), t == eos_token_id))
        n0 = input_ids.shape[1]
        cand.sort(key=lambda c: -c[0] / max(1, c[1].shape[1] - n0) ** length_penalty)
        beams = cand[:num_beams]
        if all(f for _, _, f in beams):
            break
    return beams[0][1]


@torch.no_grad()
def speculative_decode(target, draft, input_ids: torch.Tensor, max_new_tokens: int = 32, gamma: int = 4,
                       eos_token_id: int | None = None) -> tuple[torch.Tensor, dict]:
    """Greedy speculative decoding for one prompt: the draft proposes ``gamma`` tokens, the target
    scores them in one pass and keeps the longest agreeing prefix plus its own next token.  The
    output equals the target's greedy output.  Returns ``(ids, {"proposed", "accepted", "target_calls"})``."""
    assert input_ids.shape[0] == 1
    ids = input_ids
    n0 = ids.shape[1]
    stats = {"proposed": 0, "accepted": 0, "target_calls": 0}
    while ids.shape[1] - n0 < max_new_tokens:
        d = ids
        for _ in range(gamma):
            nxt = draft(d, last_token_only=True)[:, -1].float().argmax(-1)
            d = torch.cat([d, nxt[:, None]], 1)
        proposal = d[:, ids.shape[1]:]
        logits = target(d)[:, ids.shape[1] - 1:].float()      # one target pass over prefix + proposal
        stats["target_calls"] += 1
        choice = logits.argmax(-1)                            # target's token after each position
        agree = (choice[:, :gamma] == proposal)[0].long()
        n_ok = int(agree.cumprod(0).sum())
        stats["proposed"] += gamma
        stats["accepted"] += n_ok
        ids = torch.cat([ids, proposal[:, :n_ok], choice[:, n_ok:n_ok + 1]], 1)
        if eos_token_id is not None and bool((ids[0, n0:] == eos_token_id).any()):
            break
    return ids[:, : n0 + max_new_tokens], stats
