"""Post-training quantisation: affine INT8 / INT4 / UINT8 tensors per tensor or per channel,
observers for calibration, integer matmul (ferrotorch-core/src/quantize.rs:36-1100).

Conventions follow the reference (which follows PyTorch): the quantised range always contains
zero, ``scale = (max - min) / (qmax - qmin)`` floored at float epsilon,
``zero_point = clamp(qmin - round_half_even(min / scale))``, values round half to even.  INT4 values
live one per int8 (range -8..7); packing two per byte is a storage concern of the file formats
(``serialize.quant_loaders``, the Q4_0 planes of ``ops.quant``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch

_EPS = float(torch.finfo(torch.float32).eps)


class QuantDtype(enum.Enum):
    Int8 = (-128, 127)
    Int4 = (-8, 7)
    Uint8 = (0, 255)

    @property
    def qmin(self) -> int:
        return self.value[0]

    @property
    def qmax(self) -> int:
        return self.value[1]

    @property
    def storage(self) -> torch.dtype:
        return torch.uint8 if self is QuantDtype.Uint8 else torch.int8


@dataclass(frozen=True)
class QuantScheme:
    """``QuantScheme.per_tensor()`` or ``QuantScheme.per_channel(axis)``."""
    axis: int | None = None

    @classmethod
    def per_tensor(cls) -> "QuantScheme":
        return cls(None)

    @classmethod
    def per_channel(cls, axis: int) -> "QuantScheme":
        return cls(int(axis))

    PerTensor = None          # filled in below


QuantScheme.PerTensor = QuantScheme(None)


@dataclass
class QParams:
    scale: torch.Tensor          # float32, one entry per tensor / per channel
    zero_point: torch.Tensor     # int32

    @classmethod
    def symmetric(cls, max_abs, dtype: QuantDtype = QuantDtype.Int8) -> "QParams":
        m = torch.as_tensor(max_abs, dtype=torch.float32).reshape(-1)
        scale = (m / ((dtype.qmax - dtype.qmin) / 2.0)).clamp_min(_EPS)
        zp = torch.full_like(scale, 128 if dtype is QuantDtype.Uint8 else 0, dtype=torch.int32)
        return cls(scale, zp)

    @classmethod
    def asymmetric(cls, min_val, max_val, dtype: QuantDtype = QuantDtype.Int8) -> "QParams":
        lo = torch.as_tensor(min_val, dtype=torch.float32).reshape(-1)
        hi = torch.as_tensor(max_val, dtype=torch.float32).reshape(-1)
        empty = torch.isinf(lo) & (lo > 0) & torch.isinf(hi) & (hi < 0)        # nothing observed yet
        lo, hi = lo.clamp_max(0.0), hi.clamp_min(0.0)                           # the range must contain zero
        scale = ((hi - lo) / (dtype.qmax - dtype.qmin)).clamp_min(_EPS)
        zp = (dtype.qmin - torch.round(lo / scale)).clamp(dtype.qmin, dtype.qmax).to(torch.int32)
        scale = torch.where(empty, torch.ones_like(scale), scale)
        zp = torch.where(empty, torch.zeros_like(zp), zp)
        return cls(scale, zp)


@dataclass
class QuantizedTensor:
    data: torch.Tensor           # int8 (uint8 for Uint8) with the logical shape
    scale: torch.Tensor
    zero_point: torch.Tensor
    scheme: QuantScheme
    qdtype: QuantDtype

    def numel(self) -> int:
        return self.data.numel()

    @property
    def shape(self) -> tuple:
        return tuple(self.data.shape)

    def _expand(self, t: torch.Tensor) -> torch.Tensor:
        if self.scheme.axis is None:
            return t.reshape(())
        view = [1] * self.data.dim()
        view[self.scheme.axis] = -1
        return t.reshape(view)

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return ((self.data.to(torch.float32) - self._expand(self.zero_point).float()) * self._expand(self.scale)).to(dtype)


def quantize(tensor: torch.Tensor, scheme: QuantScheme = QuantScheme.PerTensor, dtype: QuantDtype = QuantDtype.Int8,
             symmetric: bool = False, qparams: QParams | None = None) -> QuantizedTensor:
    """Affine quantisation of a float tensor; ``qparams`` (e.g. from an observer) overrides the
    min / max of the tensor itself."""
    x = tensor.detach().float()
    axis = scheme.axis
    if axis is not None and not -x.dim() <= axis < x.dim():
        raise ValueError("quantize: axis %d outside a tensor of rank %d" % (axis, x.dim()))
    if not bool(torch.isfinite(x).all()):
        raise ValueError("quantize: the tensor holds non-finite values")
    if qparams is None:
        if axis is None:
            lo, hi = (x.min(), x.max()) if x.numel() else (torch.tensor(0.0), torch.tensor(0.0))
        else:
            red = [d for d in range(x.dim()) if d != axis % x.dim()]
            lo, hi = x.amin(dim=red), x.amax(dim=red)
        qparams = QParams.symmetric(torch.maximum(lo.abs(), hi.abs()), dtype) if symmetric else QParams.asymmetric(lo, hi, dtype)
    scheme = QuantScheme(None if axis is None else axis % x.dim())
    holder = QuantizedTensor(torch.empty(0), qparams.scale, qparams.zero_point, scheme, dtype)
    holder.data = x                                               # only for _expand's rank
    q = torch.round(x / holder._expand(qparams.scale)) + holder._expand(qparams.zero_point).float()
    holder.data = q.clamp(dtype.qmin, dtype.qmax).to(dtype.storage)
    return holder


def dequantize(q: QuantizedTensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return q.dequantize(dtype)


def quantized_matmul(a: QuantizedTensor, b: QuantizedTensor) -> torch.Tensor:
    """``dequantize(a) @ dequantize(b)`` computed on the integers: ``a [M, K]`` per tensor,
    ``b [K, N]`` per tensor or per output column (``per_channel(1)``); int32 accumulation, one
    float rescale at the end (quantize.rs:627)."""
    if a.data.dim() != 2 or b.data.dim() != 2 or a.data.shape[1] != b.data.shape[0]:
        raise ValueError("quantized_matmul: shapes %s and %s do not multiply" % (a.shape, b.shape))
    if a.scheme.axis is not None or b.scheme.axis not in (None, 1):
        raise ValueError("quantized_matmul: a must be per-tensor, b per-tensor or per-channel along its columns")
    ai = a.data.to(torch.int32) - a.zero_point.to(torch.int32).reshape(())
    bz = b.zero_point.to(torch.int32).reshape(1, -1) if b.scheme.axis == 1 else b.zero_point.to(torch.int32).reshape(())
    acc = (ai.to(torch.int64) @ (b.data.to(torch.int32) - bz).to(torch.int64)).to(torch.float32)   # exact for int8 x int8 sums
    return acc * (a.scale.reshape(()) * (b.scale.reshape(1, -1) if b.scheme.axis == 1 else b.scale.reshape(())))


def quantize_named_tensors(tensors: dict, scheme: QuantScheme = QuantScheme.PerTensor, dtype: QuantDtype = QuantDtype.Int8,
                           symmetric: bool = False) -> dict:
    """Quantise every floating tensor of a state dict (others pass through unchanged)."""
    return {k: quantize(v, scheme if (scheme.axis is None or v.dim() > scheme.axis) else QuantScheme.PerTensor, dtype, symmetric)
            if isinstance(v, torch.Tensor) and v.is_floating_point() else v for k, v in tensors.items()}


# --------------------------------------------------------------------------- observers
class MinMaxObserver:
    """Running minimum / maximum over everything observed."""

    def __init__(self):
        self.reset()

    def reset(self) -> None:
        self.min, self.max = float("inf"), float("-inf")

    def observe(self, data: torch.Tensor) -> None:
        if data.numel():
            if not bool(torch.isfinite(data).all()):
                raise ValueError("observer: non-finite values")
            self.min, self.max = min(self.min, float(data.min())), max(self.max, float(data.max()))

    def calculate_qparams(self, dtype: QuantDtype = QuantDtype.Int8) -> QParams:
        return QParams.asymmetric(self.min, self.max, dtype)


class PerChannelMinMaxObserver:
    def __init__(self, num_channels: int, axis: int = 0):
        if num_channels <= 0:
            raise ValueError("PerChannelMinMaxObserver: num_channels must be positive")
        self.n, self.axis = num_channels, axis
        self.reset()

    def reset(self) -> None:
        self.min = torch.full((self.n,), float("inf"))
        self.max = torch.full((self.n,), float("-inf"))

    def observe(self, data: torch.Tensor) -> None:
        if data.shape[self.axis] != self.n:
            raise ValueError("observer: %d channels along axis %d, expected %d" % (data.shape[self.axis], self.axis, self.n))
        red = [d for d in range(data.dim()) if d != self.axis % data.dim()]
        self.min = torch.minimum(self.min, data.float().amin(dim=red).cpu())
        self.max = torch.maximum(self.max, data.float().amax(dim=red).cpu())

    observe_with_shape = observe

    def calculate_qparams(self, dtype: QuantDtype = QuantDtype.Int8) -> QParams:
        return QParams.asymmetric(self.min, self.max, dtype)


class HistogramObserver:
    """Histogram of the observed values (re-binned when the range grows); the quantisation range
    is the narrowest interval that keeps ``coverage`` of the mass, which shrugs off outliers that a
    min / max observer would spend the whole range on (quantize.rs:1088-1460)."""

    def __init__(self, num_bins: int = 2048, coverage: float = 0.9999):
        if num_bins <= 0 or not 0 < coverage <= 1:
            raise ValueError("HistogramObserver: need bins > 0 and 0 < coverage <= 1")
        self.bins, self.coverage = num_bins, coverage
        self.reset()

    def reset(self) -> None:
        self.hist, self.lo, self.hi = None, 0.0, 0.0

    def observe(self, data: torch.Tensor) -> None:
        x = data.detach().float().reshape(-1).cpu()
        if not x.numel():
            return
        if not bool(torch.isfinite(x).all()):
            raise ValueError("observer: non-finite values")
        lo, hi = float(x.min()), float(x.max())
        if self.hist is None:
            self.lo, self.hi = (lo, hi) if hi > lo else (lo - 0.5, hi + 0.5)
            self.hist = torch.histc(x, self.bins, self.lo, self.hi)
            return
        nlo, nhi = min(lo, self.lo), max(hi, self.hi)
        if (nlo, nhi) != (self.lo, self.hi):                      # spread the old counts over the wider grid
            centers = self.lo + (torch.arange(self.bins) + 0.5) * (self.hi - self.lo) / self.bins
            idx = ((centers - nlo) / (nhi - nlo) * self.bins).long().clamp(0, self.bins - 1)
            self.hist = torch.zeros(self.bins).index_add_(0, idx, self.hist)
            self.lo, self.hi = nlo, nhi
        self.hist += torch.histc(x, self.bins, self.lo, self.hi)

    def range(self) -> tuple:
        if self.hist is None:
            return float("inf"), float("-inf")
        total = float(self.hist.sum())
        drop = total * (1.0 - self.coverage) / 2.0
        c = torch.cumsum(self.hist, 0)
        first = int(torch.searchsorted(c, torch.tensor(drop), right=True))
        last = int(torch.searchsorted(c, torch.tensor(total - drop), right=False))
        width = (self.hi - self.lo) / self.bins
        return self.lo + min(first, self.bins - 1) * width, self.lo + (min(last, self.bins - 1) + 1) * width

    def calculate_qparams(self, dtype: QuantDtype = QuantDtype.Int8) -> QParams:
        return QParams.asymmetric(*self.range(), dtype)
