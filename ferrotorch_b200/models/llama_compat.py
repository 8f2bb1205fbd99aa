"""Names of the reference's ``ferrotorch-llama`` surface that this package spells differently
(ferrotorch-llama/src/lib.rs re-exports): the layer classes, the activation enum, 4-bit checkpoint
containers (quant_loaders.rs:41-670), the grammar-masked greedy loop (gpu_gguf.rs:510-560)."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Callable, Sequence

import torch

from ..nn.layers import GQAAttention as LlamaAttention, SwiGLU as LlamaMLP  # noqa: F401
from ..serialize.gguf import gguf_key_to_hf, gguf_to_hf_state_dict  # noqa: F401
from ..serialize import quant_loaders as _q
from .llama import LlamaDecoderLayer as LlamaGpuLayer  # noqa: F401  (one layer class serves host and device)


class LlamaActivation(str, enum.Enum):
    Silu = "silu"
    Relu = "relu"
    FatRelu = "fatrelu"

    def __str__(self) -> str:
        return self.value


@dataclass
class GptqQ4:
    """AutoGPTQ 4-bit linear: ``qweight [in/8, out]`` int32, ``qzeros [in/group, out/8]`` int32,
    ``scales [in/group, out]``, optional ``g_idx [in]``."""
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    g_idx: torch.Tensor | None = None
    group_size: int = 128

    @property
    def in_features(self) -> int:
        return self.qweight.shape[0] * 8

    @property
    def out_features(self) -> int:
        return self.qweight.shape[1]

    def dequantize(self) -> torch.Tensor:
        """``[out, in]`` float weights."""
        return _q.dequantize_gptq(self.qweight, self.qzeros, self.scales, self.g_idx, self.group_size)

    def to_q4_0(self):
        return _q.to_q4_linear(self.dequantize())


@dataclass
class AwqQ4:
    """AutoAWQ 4-bit linear: ``qweight [in, out/8]`` int32 (interleaved nibble order), ``qzeros
    [in/group, out/8]``, ``scales [in/group, out]``."""
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    group_size: int = 128

    @property
    def in_features(self) -> int:
        return self.qweight.shape[0]

    @property
    def out_features(self) -> int:
        return self.qweight.shape[1] * 8

    def dequantize(self) -> torch.Tensor:
        return _q.dequantize_awq(self.qweight, self.qzeros, self.scales, self.group_size)

    def to_q4_0(self):
        return _q.to_q4_linear(self.dequantize())


@dataclass
class HqqQ4Axis1:
    """HQQ 4-bit linear quantised along the input axis: packed ``w_q``, per-group ``scale`` / ``zero``."""
    w_q: torch.Tensor
    scale: torch.Tensor
    zero: torch.Tensor
    out_features: int
    in_features: int
    group_size: int = 64

    def dequantize(self) -> torch.Tensor:
        return _q.dequantize_hqq(self.w_q, self.scale, self.zero, (self.out_features, self.in_features), self.group_size)

    def to_q4_0(self):
        return _q.to_q4_linear(self.dequantize())


@dataclass
class ProfiledForwardResult:
    """Logits plus wall time per named phase, as returned by a profiled forward."""
    logits: torch.Tensor
    phase_ms: dict

    def total_ms(self) -> float:
        return float(sum(self.phase_ms.values()))


def apply_grammar_mask_gpu(logits: torch.Tensor, allow, device_ordinal: int | None = None) -> torch.Tensor:
    """Logits with every disallowed token at -inf.  ``allow``: a ``TokenMask``, a bool tensor /
    sequence, or packed mask words; CUDA logits go through the packed-mask kernel."""
    from ..utils.grammar import TokenMask, apply_packed_mask_

    out = logits.clone()
    rows = out.reshape(-1, out.shape[-1])                        # a view: the kernel works on [rows, V]
    if isinstance(allow, TokenMask):
        allow.apply_(rows)
        return out
    allow = torch.as_tensor(allow)
    if allow.dtype in (torch.int32, torch.int64) and allow.numel() != out.shape[-1]:
        apply_packed_mask_(rows, allow.reshape(-1, allow.shape[-1]).to(out.device))
        return out
    return out.masked_fill_(~allow.to(out.device, torch.bool), float("-inf"))


def masked_decode_loop(next_logits: Callable[[Sequence[int]], torch.Tensor], grammar, prompt: Sequence[int],
                       max_new_tokens: int, device_ordinal: int | None = None) -> list:
    """Greedy decode under an optional grammar: stop once the grammar is complete, otherwise mask
    the logits, take the argmax and advance the grammar with it.  ``next_logits(ids)`` returns the
    logits of the next position for the ids so far."""
    ids, generated = list(prompt), []
    for _ in range(max_new_tokens):
        if grammar is not None and grammar.is_complete():
            break
        logits = torch.as_tensor(next_logits(ids)).reshape(-1)
        if grammar is not None:
            nxt = int(apply_grammar_mask_gpu(logits, grammar.compute_mask(), device_ordinal).argmax())
            try:
                grammar.step_token(nxt)
            except Exception as e:  # noqa: BLE001
                raise ValueError("masked_decode_loop: grammar rejected greedily-chosen token %d "
                                 "(mask/grammar inconsistency): %s" % (nxt, e)) from e
        else:
            nxt = int(logits.argmax())
        generated.append(nxt)
        ids.append(nxt)
    return generated
