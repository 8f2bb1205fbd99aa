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


@dataclass(frozen=True)
class LayerKvCache:
    """One layer's keys (after RoPE) and values, ``[num_kv_heads, seq_len, head_dim]``, as a value:
    ``append`` returns a new cache and leaves this one untouched (ferrotorch-llama/src/kv_cache.rs:
    37-150).  The pre-allocated in-place cache that the models use is ``nn.layers.KVCache``; the
    paged one ``nn.paged``; this is the reference's functional form, for code written against it."""
    k: torch.Tensor
    v: torch.Tensor

    def __post_init__(self):
        if self.k.dim() != 3 or self.k.shape != self.v.shape:
            raise ValueError("LayerKvCache: k and v must both be [num_kv_heads, seq_len, head_dim], got %s and %s"
                             % (tuple(self.k.shape), tuple(self.v.shape)))

    def seq_len(self) -> int:
        return int(self.k.shape[1])

    def append(self, new_k: torch.Tensor, new_v: torch.Tensor) -> "LayerKvCache":
        if new_k.dim() != 3 or new_k.shape != new_v.shape or new_k.shape[0] != self.k.shape[0] or new_k.shape[2] != self.k.shape[2]:
            raise ValueError("LayerKvCache.append: new block %s does not extend %s" % (tuple(new_k.shape), tuple(self.k.shape)))
        return LayerKvCache(torch.cat([self.k, new_k], 1), torch.cat([self.v, new_v], 1))

    @classmethod
    def from_single_token(cls, new_k: torch.Tensor, new_v: torch.Tensor) -> "LayerKvCache":
        return cls(new_k, new_v)


@dataclass(frozen=True)
class LlamaKvCache:
    """One :class:`LayerKvCache` per decoder layer (kv_cache.rs:157-260); ``extend`` appends one
    ``(k, v)`` block per layer and returns the longer cache."""
    layers: tuple = ()
    seq_len: int = 0

    @classmethod
    def empty(cls) -> "LlamaKvCache":
        return cls()

    def __len__(self) -> int:
        return self.seq_len

    def len(self) -> int:
        return self.seq_len

    def is_empty(self) -> bool:
        return self.seq_len == 0

    def extend(self, new_layer_kv) -> "LlamaKvCache":
        new_layer_kv = list(new_layer_kv)
        if self.layers and len(new_layer_kv) != len(self.layers):
            raise ValueError("LlamaKvCache.extend: %d layers given, cache has %d" % (len(new_layer_kv), len(self.layers)))
        if not new_layer_kv:
            raise ValueError("LlamaKvCache.extend: no layers given")
        if self.layers:
            layers = tuple(c.append(k, v) for c, (k, v) in zip(self.layers, new_layer_kv))
        else:
            layers = tuple(LayerKvCache.from_single_token(k, v) for k, v in new_layer_kv)
        lens = {c.seq_len() for c in layers}
        if len(lens) != 1:
            raise ValueError("LlamaKvCache.extend: layers disagree on the sequence length: %s" % sorted(lens))
        return LlamaKvCache(layers, lens.pop())


class _GrowingLayerCache:
    """The cache protocol of the attention layer (``len``, ``append(k, v) -> all keys, all values``
    on ``[1, S, Hkv, D]``) on top of a :class:`LayerKvCache` value (``[Hkv, S, D]``)."""

    def __init__(self, layer: LayerKvCache | None):
        self.k = layer.k.transpose(0, 1)[None] if layer is not None else None
        self.v = layer.v.transpose(0, 1)[None] if layer is not None else None
        self.len = layer.seq_len() if layer is not None else 0

    def append(self, k: torch.Tensor, v: torch.Tensor):
        self.k = k if self.k is None else torch.cat([self.k.to(k.dtype), k], 1)
        self.v = v if self.v is None else torch.cat([self.v.to(v.dtype), v], 1)
        self.len = self.k.shape[1]
        return self.k, self.v

    def as_layer(self) -> LayerKvCache:
        return LayerKvCache(self.k[0].transpose(0, 1).contiguous(), self.v[0].transpose(0, 1).contiguous())


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
