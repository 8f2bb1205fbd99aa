"""Layers of the reference's ``ferrotorch-nn`` that ``torch.nn`` does not ship: ``LoRALinear``
(lora.rs:76-220), ``SqueezeExcitation`` (se.rs:79-200) and ``HookedModule`` (hooks.rs:73-200)."""
from __future__ import annotations

import math

import torch
from torch import nn


class LoRALinear(nn.Module):
    """``base(x) + (alpha / rank) * dropout(x) A^T B^T`` with the base layer frozen, ``A [r, in]``
    drawn from N(0, 1/sqrt(r)) and ``B [out, r]`` zero, so training starts at the base model.
    ``merge()`` folds the update into the base weight and re-initialises the adapters."""

    def __init__(self, base: nn.Linear, rank: int, alpha: float = 1.0, dropout_p: float = 0.0):
        super().__init__()
        if rank <= 0:
            raise ValueError("LoRALinear: rank must be > 0")
        if not 0.0 <= dropout_p < 1.0:
            raise ValueError("LoRALinear: dropout_p must be in [0, 1)")
        self.base_layer, self.rank_, self.alpha_ = base, rank, float(alpha)
        for p in base.parameters():
            p.requires_grad_(False)
        w = base.weight
        self.lora_a = nn.Parameter(torch.empty(rank, base.in_features, device=w.device, dtype=w.dtype))
        self.lora_b = nn.Parameter(torch.zeros(base.out_features, rank, device=w.device, dtype=w.dtype))
        self.dropout = nn.Dropout(dropout_p) if dropout_p > 0 else None
        self._reset()

    def _reset(self) -> None:
        with torch.no_grad():
            self.lora_a.normal_(0.0, 1.0 / math.sqrt(self.rank_))
            self.lora_b.zero_()

    def rank(self) -> int:
        return self.rank_

    def alpha(self) -> float:
        return self.alpha_

    def base(self) -> nn.Linear:
        return self.base_layer

    def into_base(self) -> nn.Linear:
        return self.base_layer

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = x if self.dropout is None else self.dropout(x)
        return self.base_layer(x) + (h @ self.lora_a.t() @ self.lora_b.t()) * (self.alpha_ / self.rank_)

    @torch.no_grad()
    def merge(self) -> None:
        self.base_layer.weight.add_((self.lora_b @ self.lora_a) * (self.alpha_ / self.rank_))
        self._reset()


class SqueezeExcitation(nn.Module):
    """Channel gate of SENet / EfficientNet: global average pool, 1x1 conv down, activation, 1x1
    conv up, scale activation, multiply (parameter names ``fc1`` / ``fc2`` as in torchvision)."""

    def __init__(self, input_channels: int, squeeze_channels: int, activation=nn.ReLU, scale_activation=nn.Sigmoid):
        super().__init__()
        if input_channels <= 0 or squeeze_channels <= 0:
            raise ValueError("SqueezeExcitation: input_channels and squeeze_channels must be > 0 (got %d, %d)"
                             % (input_channels, squeeze_channels))
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc1 = nn.Conv2d(input_channels, squeeze_channels, 1)
        self.fc2 = nn.Conv2d(squeeze_channels, input_channels, 1)
        self.activation = activation() if isinstance(activation, type) else activation
        self.scale_activation = scale_activation() if isinstance(scale_activation, type) else scale_activation

    @classmethod
    def new_with_activations(cls, input_channels: int, squeeze_channels: int, activation, scale_activation) -> "SqueezeExcitation":
        """EfficientNet uses SiLU / sigmoid, MobileNetV3 ReLU / hard-sigmoid."""
        return cls(input_channels, squeeze_channels, activation, scale_activation)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * self.scale_activation(self.fc2(self.activation(self.fc1(self.avgpool(x)))))


class HookHandle:
    def __init__(self, hid: int, registry: dict):
        self._id, self._registry = hid, registry

    def id(self) -> int:
        return self._id

    def remove(self) -> None:
        self._registry.pop(self._id, None)


class HookedModule(nn.Module):
    """Wrap any module with removable hooks: pre-hooks may replace the input, forward hooks may
    replace the output, backward hooks see (and may replace) the gradient of the output."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module
        self._pre, self._fwd, self._bwd, self._next = {}, {}, {}, 0

    def _register(self, table: dict, hook) -> HookHandle:
        hid, self._next = self._next, self._next + 1
        table[hid] = hook
        return HookHandle(hid, table)

    def register_forward_pre_hook(self, hook) -> HookHandle:       # hook(input) -> None | new input
        return self._register(self._pre, hook)

    def register_forward_hook(self, hook) -> HookHandle:           # hook(input, output) -> None | new output
        return self._register(self._fwd, hook)

    def register_backward_hook(self, hook) -> HookHandle:          # hook(grad_output) -> None | new grad
        return self._register(self._bwd, hook)

    def inner(self) -> nn.Module:
        return self.module

    inner_mut = into_inner = inner

    def forward(self, x):
        for h in list(self._pre.values()):
            r = h(x)
            x = x if r is None else r
        y = self.module(x)
        for h in list(self._fwd.values()):
            r = h(x, y)
            y = y if r is None else r
        if self._bwd and isinstance(y, torch.Tensor) and y.requires_grad:
            def run(g):
                for h in list(self._bwd.values()):
                    r = h(g)
                    g = g if r is None else r
                return g
            y.register_hook(run)
        return y


# --------------------------------------------------------------------------- tiled attention on any device
def _check_attn(q, k, v, block_size):
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("attention: expected [B, N, d] tensors")
    if q.shape[0] != k.shape[0] or k.shape[0] != v.shape[0] or q.shape[2] != k.shape[2] or k.shape[1] != v.shape[1]:
        raise ValueError("attention: incompatible shapes %s %s %s" % (tuple(q.shape), tuple(k.shape), tuple(v.shape)))
    if block_size <= 0:
        raise ValueError("attention: block_size must be positive")


def standard_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """``softmax(Q K^T / sqrt(d)) V`` with the whole score matrix in memory; ``causal`` hides keys
    ``j > i`` (ferrotorch-nn/src/flash_attention.rs:647)."""
    _check_attn(query, key, value, 1)
    s = query @ key.transpose(1, 2) / math.sqrt(query.shape[2])
    if causal:
        i = torch.arange(query.shape[1], device=query.device)[:, None]
        j = torch.arange(key.shape[1], device=query.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    return torch.softmax(s, dim=-1) @ value


class _TiledAttention(torch.autograd.Function):
    """Online-softmax attention over key blocks: memory O(N block) instead of O(N^2); the backward
    recomputes each block's probabilities from the saved row log-sum-exp."""

    @staticmethod
    def forward(ctx, q, k, v, causal, block):
        B, Nq, d = q.shape
        scale = 1.0 / math.sqrt(d)
        out = torch.zeros(B, Nq, v.shape[2], dtype=torch.float32, device=q.device)
        m = torch.full((B, Nq), float("-inf"), dtype=torch.float32, device=q.device)
        l = torch.zeros(B, Nq, dtype=torch.float32, device=q.device)
        rows = torch.arange(Nq, device=q.device)[:, None]
        for j0 in range(0, k.shape[1], block):
            kb, vb = k[:, j0:j0 + block].float(), v[:, j0:j0 + block].float()
            s = q.float() @ kb.transpose(1, 2) * scale
            if causal:
                cols = torch.arange(j0, j0 + kb.shape[1], device=q.device)[None, :]
                s = s.masked_fill(cols > rows, float("-inf"))
            m_new = torch.maximum(m, s.amax(-1))
            safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)      # rows that have seen no key yet
            p = torch.exp(s - safe[..., None])
            alpha = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - safe))
            l = alpha * l + p.sum(-1)
            out = alpha[..., None] * out + p @ vb
            m = m_new
        out = out / l[..., None]
        lse = torch.where(torch.isinf(m), m, m + torch.log(l))
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.block = causal, block
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        scale = 1.0 / math.sqrt(q.shape[2])
        dq, dk, dv = torch.zeros_like(q, dtype=torch.float32), torch.zeros_like(k, dtype=torch.float32), torch.zeros_like(v, dtype=torch.float32)
        do = dout.float()
        delta = (do * out).sum(-1)                          # rowsum(dO * O)
        rows = torch.arange(q.shape[1], device=q.device)[:, None]
        for j0 in range(0, k.shape[1], ctx.block):
            kb, vb = k[:, j0:j0 + ctx.block].float(), v[:, j0:j0 + ctx.block].float()
            s = q.float() @ kb.transpose(1, 2) * scale
            if ctx.causal:
                cols = torch.arange(j0, j0 + kb.shape[1], device=q.device)[None, :]
                s = s.masked_fill(cols > rows, float("-inf"))
            p = torch.exp(s - lse[..., None])
            dv[:, j0:j0 + ctx.block] = p.transpose(1, 2) @ do
            ds = p * (do @ vb.transpose(1, 2) - delta[..., None]) * scale
            dq += ds @ kb
            dk[:, j0:j0 + ctx.block] = ds.transpose(1, 2) @ q.float()
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None, None


def flash_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, causal: bool = False,
                    block_size: int = 64) -> torch.Tensor:
    """Tiled attention with forward and backward on ``[B, N, d]`` tensors of any device
    (ferrotorch-nn/src/flash_attention.rs:59-640).  The GPU kernels for bf16 multi-head inputs
    are :func:`ferrotorch_b200.ops.functional.flash_attention` / ``packed_attention``."""
    _check_attn(query, key, value, block_size)
    return _TiledAttention.apply(query, key, value, causal, block_size)
