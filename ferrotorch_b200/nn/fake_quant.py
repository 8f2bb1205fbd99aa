"""Observers, fake quantisation and quantisation-aware training (QAT).

Reference: ``MinMaxObserver`` / ``MovingAverageObserver`` / per-channel observers and INT8 / INT4
post-training quantisation (ferrotorch-core/src/quantize.rs:36-627), ``prepare_qat`` and the
fake-quantised ``QatLinear`` with a straight-through estimator (ferrotorch-nn/src/qat.rs:182).
"""
from __future__ import annotations

import torch
from torch import nn


class MinMaxObserver(nn.Module):
    """Running min / max of everything seen (per tensor, or per channel along ``ch_axis``)."""

    def __init__(self, bits: int = 8, symmetric: bool = True, ch_axis: int | None = None, momentum: float | None = None):
        super().__init__()
        self.bits, self.symmetric, self.ch_axis, self.momentum = bits, symmetric, ch_axis, momentum
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.ch_axis is None:
            lo, hi = x.amin(), x.amax()
        else:
            dims = [d for d in range(x.dim()) if d != self.ch_axis % x.dim()]
            lo, hi = x.amin(dims), x.amax(dims)
        lo, hi = lo.float(), hi.float()
        if torch.isinf(self.min_val).any() or self.min_val.shape != lo.shape:
            self.min_val, self.max_val = lo.clone(), hi.clone()
        elif self.momentum is None:
            self.min_val, self.max_val = torch.minimum(self.min_val, lo), torch.maximum(self.max_val, hi)
        else:
            m = self.momentum
            self.min_val, self.max_val = (1 - m) * self.min_val + m * lo, (1 - m) * self.max_val + m * hi
        return x

    def qparams(self) -> tuple[torch.Tensor, torch.Tensor, int, int]:
        """``(scale, zero_point, qmin, qmax)``."""
        if self.symmetric:
            qmax = 2 ** (self.bits - 1) - 1
            scale = (torch.maximum(self.max_val.abs(), self.min_val.abs()) / qmax).clamp_min(1e-12)
            return scale, torch.zeros_like(scale), -qmax - 1, qmax
        qmin, qmax = 0, 2 ** self.bits - 1
        lo, hi = torch.minimum(self.min_val, torch.zeros_like(self.min_val)), torch.maximum(self.max_val, torch.zeros_like(self.max_val))
        scale = ((hi - lo) / (qmax - qmin)).clamp_min(1e-12)
        return scale, (qmin - lo / scale).round().clamp(qmin, qmax), qmin, qmax


def MovingAverageObserver(bits: int = 8, symmetric: bool = True, ch_axis: int | None = None, momentum: float = 0.01):
    return MinMaxObserver(bits, symmetric, ch_axis, momentum)


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zero, qmin, qmax):
        q = (x / scale + zero).round()
        ctx.save_for_backward((q >= qmin) & (q <= qmax))
        return ((q.clamp(qmin, qmax) - zero) * scale).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        (inside,) = ctx.saved_tensors
        return dy * inside.to(dy.dtype), None, None, None, None


class FakeQuantize(nn.Module):
    """Observe, then quantise-dequantise with a straight-through gradient (zero outside the range)."""

    def __init__(self, bits: int = 8, symmetric: bool = True, ch_axis: int | None = None, momentum: float | None = None):
        super().__init__()
        self.observer = MinMaxObserver(bits, symmetric, ch_axis, momentum)
        self.observe, self.enabled = True, True

    # ---- torch / reference switches (quantize.rs ``FakeQuantize``)
    def enable_observer(self) -> "FakeQuantize":
        self.observe = True
        return self

    def disable_observer(self) -> "FakeQuantize":
        """Freeze the range: later batches are quantised with the statistics gathered so far."""
        self.observe = False
        return self

    def enable_fake_quant(self) -> "FakeQuantize":
        self.enabled = True
        return self

    def disable_fake_quant(self) -> "FakeQuantize":
        """Pass values through unchanged (the observer may keep collecting)."""
        self.enabled = False
        return self

    def calculate_qparams(self):
        """``(scale, zero_point)`` from the observed range."""
        scale, zero, _, _ = self.observer.qparams()
        return scale, zero

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.observe and self.training:
            self.observer(x.detach())
        if not self.enabled or torch.isinf(self.observer.min_val).any():
            return x
        scale, zero, qmin, qmax = self.observer.qparams()
        if self.observer.ch_axis is not None:
            shape = [1] * x.dim()
            shape[self.observer.ch_axis % x.dim()] = -1
            scale, zero = scale.view(shape), zero.view(shape)
        return _FakeQuantSTE.apply(x, scale.to(x.device), zero.to(x.device), qmin, qmax)


class QatLinear(nn.Linear):
    """``nn.Linear`` with fake-quantised weight (per output channel) and input activation."""

    def __init__(self, in_features, out_features, bias=True, weight_bits: int = 8, act_bits: int = 8, **kw):
        super().__init__(in_features, out_features, bias, **kw)
        self.weight_fq = FakeQuantize(weight_bits, True, ch_axis=0)
        self.act_fq = FakeQuantize(act_bits, False, momentum=0.01)

    @classmethod
    def from_float(cls, lin: nn.Linear, weight_bits: int = 8, act_bits: int = 8) -> "QatLinear":
        q = cls(lin.in_features, lin.out_features, lin.bias is not None, weight_bits, act_bits,
                device=lin.weight.device, dtype=lin.weight.dtype)
        q.weight, q.bias = lin.weight, lin.bias
        return q

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return nn.functional.linear(self.act_fq(x), self.weight_fq(self.weight), self.bias)

    def to_quantized(self):
        """``(int weight [N, K], scale [N], bias)`` for the integer matmul path."""
        scale, _, qmin, qmax = self.weight_fq.observer.qparams()
        q = (self.weight.detach().float() / scale[:, None]).round().clamp(qmin, qmax).to(torch.int8)
        return q, scale, self.bias


def prepare_qat(model: nn.Module, weight_bits: int = 8, act_bits: int = 8, skip: tuple[str, ...] = ()) -> nn.Module:
    """Swap every ``nn.Linear`` (except names in ``skip``) for a :class:`QatLinear`, in place."""
    for name, child in list(model.named_children()):
        if name in skip:
            continue
        if type(child) is nn.Linear or (isinstance(child, nn.Linear) and not isinstance(child, QatLinear)):
            setattr(model, name, QatLinear.from_float(child, weight_bits, act_bits))
        else:
            prepare_qat(child, weight_bits, act_bits, skip)
    return model


def convert(model: nn.Module) -> dict[str, tuple]:
    """Integer weights + scales of every :class:`QatLinear`, keyed by module name."""
    return {n: m.to_quantized() for n, m in model.named_modules() if isinstance(m, QatLinear)}
