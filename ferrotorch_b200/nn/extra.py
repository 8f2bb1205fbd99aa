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
