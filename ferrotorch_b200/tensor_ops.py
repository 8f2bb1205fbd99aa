"""The reference's free-function tensor API over torch (ferrotorch-core/src/lib.rs re-exports:
creation.rs, ops/*, grad_fns/*, fft.rs, special.rs, masked.rs, pruning.rs, autograd/forward_ad.rs).

torch already has most of these under the same name; this module holds the ones the reference
spells or shapes differently -- ``sum_dim(x, dim, keepdim)``, ``*_with_dim`` pairs, the
``*_norm`` FFT variants, ``clamp_opt``, masked reductions, ``dual_*`` forward-mode ops -- plus type
names (``DType``, ``FerrotorchError`` ...).  Every function is differentiable wherever torch's is
(the reference's ``*_differentiable`` twins are therefore the same functions).  The package root
resolves unknown attributes here first and in ``torch`` second, so ``ferrotorch_b200.zeros`` and
``ferrotorch_b200.sum_dim`` both work.
"""
from __future__ import annotations

import enum
import math
from typing import Sequence

import torch
from torch import Tensor

from . import autograd as _ag

# --------------------------------------------------------------------------- type vocabulary
DType = torch.dtype
Generator = torch.Generator
TensorStorage = torch.UntypedStorage
StorageBuffer = torch.UntypedStorage
GradFn = torch.autograd.graph.Node
HookHandle = torch.utils.hooks.RemovableHandle
TensorId = int                                     # ``id(tensor)``: identity of a tensor object
Float = (torch.float32, torch.float64, torch.bfloat16, torch.float16)     # dtypes the float ops take
IntElement = (torch.int32, torch.int64)
Element = Float + IntElement + (torch.bool,)
FerrotorchResult = object                          # results are returned, errors are raised


class FerrotorchError(RuntimeError):
    """Base of the errors this package raises on its own account; torch's errors pass through."""


class AnomalyMode:
    """``with AnomalyMode(): ...`` -- ``torch.autograd.detect_anomaly`` (autograd/anomaly.rs:74)."""

    def __init__(self, check_nan: bool = True):
        self._cm = torch.autograd.detect_anomaly(check_nan=check_nan)

    def __enter__(self):
        self._cm.__enter__()
        return self

    def __exit__(self, *exc):
        return self._cm.__exit__(*exc)

    @staticmethod
    def is_enabled() -> bool:
        return torch.is_anomaly_enabled()

    @staticmethod
    def enable(check_nan: bool = True) -> None:
        """Switch anomaly detection on for the rest of the process (the context-manager form restores it)."""
        torch.autograd.set_detect_anomaly(True, check_nan=check_nan)

    @staticmethod
    def disable() -> None:
        torch.autograd.set_detect_anomaly(False)


class ForwardBacktrace(list):
    """The forward-pass stack that anomaly mode records on an autograd node (anomaly.rs): a list
    of formatted frames, empty when the node was created outside anomaly mode."""

    @classmethod
    def of(cls, tensor_or_node) -> "ForwardBacktrace":
        node = getattr(tensor_or_node, "grad_fn", tensor_or_node)
        meta = getattr(node, "metadata", None) or {}
        return cls(meta.get("traceback_", []))

    @classmethod
    def capture_if_enabled(cls, tensor_or_node=None) -> "ForwardBacktrace | None":
        """The recorded stack of a node when anomaly mode is on (the current Python stack when no node
        is given), ``None`` when it is off."""
        if not torch.is_anomaly_enabled():
            return None
        if tensor_or_node is not None:
            return cls.of(tensor_or_node)
        import traceback

        return cls(traceback.format_stack()[:-1])

    def trace(self) -> str:
        return "".join(self)


def check_gradient_anomaly(t: Tensor, what: str = "gradient") -> None:
    """Raise when ``t`` holds NaN or Inf (what anomaly mode checks after every backward node)."""
    if not bool(torch.isfinite(t).all()):
        raise FerrotorchError("%s contains NaN or Inf" % what)


class AutocastDtype(enum.Enum):
    F16 = torch.float16
    BF16 = torch.bfloat16


def autocast_dtype(device_type: str = "cuda") -> torch.dtype:
    return torch.get_autocast_dtype(device_type)


def autocast_guard(dtype=AutocastDtype.BF16, device_type: str = "cuda", enabled: bool = True):
    """Context manager form of ``autocast`` (autograd/autocast.rs:151)."""
    return _ag.autocast(device_type, dtype=dtype.value if isinstance(dtype, AutocastDtype) else dtype, enabled=enabled)


class FftNorm(str, enum.Enum):
    Backward = "backward"
    Forward = "forward"
    Ortho = "ortho"

    def __str__(self) -> str:
        return self.value


class GeluApproximate(str, enum.Enum):
    NoApproximation = "none"
    Tanh = "tanh"

    def __str__(self) -> str:
        return self.value


class MeshIndexing(str, enum.Enum):
    Ij = "ij"
    Xy = "xy"

    def __str__(self) -> str:
        return self.value


class EinopsReduction(str, enum.Enum):
    Sum = "sum"; Mean = "mean"; Max = "max"; Min = "min"; Prod = "prod"  # noqa: E702

    def __str__(self) -> str:
        return self.value


class DispatchKey(enum.IntEnum):
    """Dispatch keys from lowest to highest priority (ferrotorch-core/src/dispatch.rs:70-124): the three
    back-end keys, the tensor-kind keys, then the layers that wrap an op (autocast, autograd, vmap,
    profiler, tracer).  The value is the priority and the bit position in a :class:`DispatchKeySet`."""
    Cpu = 0
    Cuda = 1
    Meta = 2
    Sparse = 3
    Quantized = 4
    Nested = 5
    Autocast = 6
    Autograd = 7
    Vmap = 8
    Profiler = 9
    Tracer = 10

    def priority(self) -> int:
        return int(self)


class DispatchKeySet:
    """A set of keys as a bit mask; iteration and ``highest`` go from the highest priority down
    (dispatch.rs:137-251).  Values are immutable: ``insert`` / ``remove`` return a new set."""

    def __init__(self, keys=()):
        bits = 0
        for k in keys:
            bits |= 1 << int(DispatchKey(k))
        self.bits = bits

    @classmethod
    def from_keys(cls, keys) -> "DispatchKeySet":
        return cls(keys)

    @classmethod
    def all(cls) -> "DispatchKeySet":
        return cls(DispatchKey)

    def insert(self, key) -> "DispatchKeySet":
        out = DispatchKeySet()
        out.bits = self.bits | (1 << int(DispatchKey(key)))
        return out

    def remove(self, key) -> "DispatchKeySet":
        out = DispatchKeySet()
        out.bits = self.bits & ~(1 << int(DispatchKey(key)))
        return out

    def contains(self, key) -> bool:
        return bool(self.bits >> int(DispatchKey(key)) & 1)

    def union(self, other: "DispatchKeySet") -> "DispatchKeySet":
        out = DispatchKeySet()
        out.bits = self.bits | other.bits
        return out

    def intersection(self, other: "DispatchKeySet") -> "DispatchKeySet":
        out = DispatchKeySet()
        out.bits = self.bits & other.bits
        return out

    __or__, __and__ = union, intersection

    __contains__ = contains

    def is_empty(self) -> bool:
        return self.bits == 0

    def len(self) -> int:
        return bin(self.bits).count("1")

    __len__ = len

    def highest(self):
        return DispatchKey(self.bits.bit_length() - 1) if self.bits else None

    def iter_desc(self):
        return (k for k in sorted(DispatchKey, reverse=True) if self.contains(k))

    __iter__ = iter_desc

    def __eq__(self, other) -> bool:
        return isinstance(other, DispatchKeySet) and other.bits == self.bits

    def __hash__(self) -> int:
        return hash(self.bits)

    def __repr__(self) -> str:
        return "DispatchKeySet(%s)" % ", ".join(k.name for k in self.iter_desc())


class Dispatcher:
    """A table ``(op name, key) -> kernel`` with priority resolution (dispatch.rs:298-400): ``call`` runs
    the kernel of the highest-priority key of ``keyset`` that has one for the op and hands it the whole
    key set, so that a wrapping layer (autocast, autograd, a profiler) can take its own key out and
    call again.  torch's dispatcher routes this package's kernels; this table is for code that layers
    Python-level behaviour the same way the reference's users do."""

    def __init__(self):
        self._kernels: dict = {}

    def register(self, op_name: str, key, kernel) -> None:
        self._kernels[(str(op_name), DispatchKey(key))] = kernel

    def has_kernel(self, op_name: str, key) -> bool:
        return (str(op_name), DispatchKey(key)) in self._kernels

    def kernel_count(self) -> int:
        return len(self._kernels)

    def call(self, op_name: str, inputs, keyset: DispatchKeySet):
        if keyset.is_empty():
            raise FerrotorchError("Dispatcher.call(%r): the key set is empty" % op_name)
        for key in keyset.iter_desc():
            kernel = self._kernels.get((str(op_name), key))
            if kernel is not None:
                return kernel(inputs, keyset)
        raise FerrotorchError("Dispatcher.call(%r): no kernel for any key of %r" % (op_name, keyset))

    def call_direct(self, op_name: str, key, inputs, keyset: DispatchKeySet | None = None):
        kernel = self._kernels.get((str(op_name), DispatchKey(key)))
        if kernel is None:
            raise FerrotorchError("Dispatcher.call_direct(%r): no kernel for %s" % (op_name, DispatchKey(key).name))
        return kernel(inputs, keyset if keyset is not None else DispatchKeySet([key]))


Kernel = object


# --------------------------------------------------------------------------- creation
def scalar(value, dtype=None) -> Tensor:
    return torch.tensor(value, dtype=dtype)


def from_slice(data: Sequence, shape: Sequence[int], dtype=torch.float32) -> Tensor:
    t = torch.as_tensor(list(data), dtype=dtype)
    if t.numel() != math.prod(shape):
        raise FerrotorchError("from_slice: %d values for shape %s" % (t.numel(), tuple(shape)))
    return t.reshape(tuple(shape))


from_vec = from_slice


def rand_on_device(shape, device, dtype=torch.float32, generator=None) -> Tensor:
    return torch.rand(tuple(shape), device=device, dtype=dtype, generator=generator)


def randn_on_device(shape, device, dtype=torch.float32, generator=None) -> Tensor:
    return torch.randn(tuple(shape), device=device, dtype=dtype, generator=generator)


def fftfreq_on_device(n: int, d: float = 1.0, device=None) -> Tensor:
    return torch.fft.fftfreq(n, d, device=device)


def rfftfreq_on_device(n: int, d: float = 1.0, device=None) -> Tensor:
    return torch.fft.rfftfreq(n, d, device=device)


def meshgrid_indexing(tensors, indexing=MeshIndexing.Ij):
    return torch.meshgrid(*tensors, indexing=str(indexing))


def meshgrid(*tensors, indexing=MeshIndexing.Ij):
    if len(tensors) == 1 and isinstance(tensors[0], (list, tuple)):
        tensors = tuple(tensors[0])
    return torch.meshgrid(*tensors, indexing=str(indexing))


def normalize_axis(axis: int, ndim: int) -> int:
    if not -ndim <= axis < max(ndim, 1):
        raise FerrotorchError("axis %d out of range for %d dimensions" % (axis, ndim))
    return axis % ndim if ndim else 0


# --------------------------------------------------------------------------- shape ops under the reference's ``_t`` names
def view_t(x: Tensor, shape) -> Tensor:
    return x.view(*shape)


def permute_t(x: Tensor, dims) -> Tensor:
    return x.permute(*dims)


def contiguous_t(x: Tensor) -> Tensor:
    return x.contiguous()


def chunk_t(x: Tensor, chunks: int, dim: int = 0):
    return list(torch.chunk(x, chunks, dim))


def split_t(x: Tensor, split_size_or_sections, dim: int = 0):
    return list(torch.split(x, split_size_or_sections, dim))


def expand(x: Tensor, shape) -> Tensor:
    return x.expand(*shape)


def expand_as(x: Tensor, other: Tensor) -> Tensor:
    return x.expand_as(other)


def as_strided_copy(x: Tensor, size, stride, storage_offset: int = 0) -> Tensor:
    return torch.as_strided(x, size, stride, storage_offset).clone()


AsStridedBackward = "AsStridedBackward0"           # the autograd node's name, for graph inspection


def select(x: Tensor, dim: int, index: int) -> Tensor:
    return torch.select(x, dim, index)


# --------------------------------------------------------------------------- reductions with the dimension spelled out
def sum_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.sum(dim, keepdim)


def sum_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False) -> Tensor:
    return x.sum(tuple(dims), keepdim) if len(dims) else x.clone()


def mean_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.mean(dim, keepdim)


def mean_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False) -> Tensor:
    return x.mean(tuple(dims), keepdim) if len(dims) else x.clone()


def std_dim(x: Tensor, dim: int, keepdim: bool = False, correction: int = 1) -> Tensor:
    return x.std(dim, correction=correction, keepdim=keepdim)


def std_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False, correction: int = 1) -> Tensor:
    return x.std(tuple(dims), correction=correction, keepdim=keepdim)


def var_dim(x: Tensor, dim: int, keepdim: bool = False, correction: int = 1) -> Tensor:
    return x.var(dim, correction=correction, keepdim=keepdim)


def var_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False, correction: int = 1) -> Tensor:
    return x.var(tuple(dims), correction=correction, keepdim=keepdim)


def nansum_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.nansum(dim, keepdim)


def nansum_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False) -> Tensor:
    return x.nansum(tuple(dims), keepdim)


def nanmean_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.nanmean(dim, keepdim)


def nanmean_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False) -> Tensor:
    return x.nanmean(tuple(dims), keepdim)


def logsumexp_dims(x: Tensor, dims: Sequence[int], keepdim: bool = False) -> Tensor:
    return torch.logsumexp(x, tuple(dims), keepdim)


def max_with_dim(x: Tensor, dim: int, keepdim: bool = False):
    """``(values, indices)`` along ``dim``."""
    r = x.max(dim, keepdim)
    return r.values, r.indices


def min_with_dim(x: Tensor, dim: int, keepdim: bool = False):
    r = x.min(dim, keepdim)
    return r.values, r.indices


def median_with_dim(x: Tensor, dim: int, keepdim: bool = False):
    r = x.median(dim, keepdim)
    return r.values, r.indices


def nanmedian_with_dim(x: Tensor, dim: int, keepdim: bool = False):
    r = x.nanmedian(dim, keepdim)
    return r.values, r.indices


def norm_with_dim(x: Tensor, p: float = 2.0, dim=None, keepdim: bool = False) -> Tensor:
    return torch.linalg.vector_norm(x, p, dim, keepdim)


def topk_dim(x: Tensor, k: int, dim: int = -1, largest: bool = True):
    r = torch.topk(x, k, dim, largest, True)
    return r.values, r.indices


def topk_dim_sorted(x: Tensor, k: int, dim: int = -1, largest: bool = True, sorted: bool = True):  # noqa: A002
    r = torch.topk(x, k, dim, largest, sorted)
    return r.values, r.indices


class CumExtremeResult(tuple):
    """``(values, indices)`` of ``cummax`` / ``cummin``."""

    @property
    def values(self) -> Tensor:
        return self[0]

    @property
    def indices(self) -> Tensor:
        return self[1]

    def indices_host(self) -> list:
        """The indices as a (nested) Python list on the host."""
        return self[1].cpu().tolist()


def cummax(x: Tensor, dim: int) -> CumExtremeResult:
    r = torch.cummax(x, dim)
    return CumExtremeResult((r.values, r.indices))


def cummin(x: Tensor, dim: int) -> CumExtremeResult:
    r = torch.cummin(x, dim)
    return CumExtremeResult((r.values, r.indices))


# --------------------------------------------------------------------------- clamp family
def clamp_opt(x: Tensor, min=None, max=None) -> Tensor:  # noqa: A002
    if min is None and max is None:
        raise FerrotorchError("clamp_opt: at least one of 'min' or 'max' must not be None")
    return torch.clamp(x, min, max)


def clamp_min_tensor(x: Tensor, min: Tensor) -> Tensor:  # noqa: A002
    return torch.clamp(x, min=min)


def clamp_max_tensor(x: Tensor, max: Tensor) -> Tensor:  # noqa: A002
    return torch.clamp(x, max=max)


def clamp_tensor(x: Tensor, min: Tensor | None = None, max: Tensor | None = None) -> Tensor:  # noqa: A002
    return clamp_opt(x, min, max)


clip_opt, clip_tensor = clamp_opt, clamp_tensor


def gelu_with(x: Tensor, approximate=GeluApproximate.NoApproximation) -> Tensor:
    return torch.nn.functional.gelu(x, approximate=str(approximate))


gelu = torch.nn.functional.gelu


def where_cond(condition, x: Tensor, y: Tensor) -> Tensor:
    """``condition``: a bool sequence / tensor of ``x``'s size (flat) or shape."""
    c = torch.as_tensor(condition, dtype=torch.bool, device=x.device)
    if c.shape != x.shape:
        if c.numel() != x.numel():
            raise FerrotorchError("where_cond: condition has %d elements, x has %d" % (c.numel(), x.numel()))
        c = c.reshape(x.shape)
    return torch.where(c, x, y)


def where_cond_bt(cond: Tensor, x: Tensor, y: Tensor) -> Tensor:
    """Broadcasting form over a bool tensor."""
    return torch.where(cond.bool(), x, y)


def scatter_add_segments(src: Tensor, index, dim_size: int) -> Tensor:
    """``out[index[i]] += src[i]`` over rows: ``src [E, ...]`` -> ``[dim_size, ...]`` (the message
    aggregation of graph layers, ops/scatter.rs:183)."""
    idx = torch.as_tensor(index, dtype=torch.int64, device=src.device)
    if idx.numel() != src.shape[0]:
        raise FerrotorchError("scatter_add_segments: %d indices for %d rows" % (idx.numel(), src.shape[0]))
    if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= dim_size):
        raise FerrotorchError("scatter_add_segments: index out of range for %d segments" % dim_size)
    return torch.zeros((dim_size,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device).index_add_(0, idx, src)


def einsum_differentiable(equation: str, *operands: Tensor) -> Tensor:
    return torch.einsum(equation, *operands)


def rearrange_with(tensor: Tensor, pattern: str, axes: dict | None = None) -> Tensor:
    from .core import rearrange

    return rearrange(tensor, pattern, **(axes or {}))


def vmap2(fn, in_dims=(0, 0), out_dims=0):
    """``vmap`` over two arguments."""
    return torch.vmap(fn, in_dims=in_dims, out_dims=out_dims)


def manual_seed(seed: int) -> None:
    torch.manual_seed(seed)


def nested_scaled_dot_product_attention(q, k, v, is_causal: bool = False):
    """Attention over nested (ragged) batches: one call per sequence, results re-nested."""
    qs, ks, vs = (t.unbind() if t.is_nested else list(t) for t in (q, k, v))
    outs = [torch.nn.functional.scaled_dot_product_attention(a[None], b[None], c[None], is_causal=is_causal)[0]
            for a, b, c in zip(qs, ks, vs)]
    return torch.nested.nested_tensor(outs)


# --------------------------------------------------------------------------- FFT family
# ``name(x, ...)`` is torch.fft's; ``name_norm(x, ..., norm)`` takes the normalisation as a
# trailing argument; the ``_differentiable`` spellings are the same functions (torch.fft has autograd).
def _fft_family():
    g = globals()
    for base in ("fft", "ifft", "rfft", "irfft", "hfft", "ihfft", "fft2", "ifft2", "rfft2", "irfft2", "hfft2", "ihfft2",
                 "fftn", "ifftn", "rfftn", "irfftn", "hfftn", "ihfftn"):
        fn = getattr(torch.fft, base)

        def with_norm(x, *args, norm=FftNorm.Backward, _fn=fn, **kw):
            return _fn(x, *args, norm=str(norm), **kw)

        with_norm.__name__ = base + "_norm"
        with_norm.__doc__ = "``torch.fft.%s`` with ``norm`` one of ``FftNorm`` (default backward)." % base
        g[base] = fn
        g[base + "_norm"] = with_norm
        g[base + "_differentiable"] = fn
        g[base + "_differentiable_norm"] = with_norm
    for name in ("fftfreq", "rfftfreq", "fftshift", "ifftshift"):
        g[name] = getattr(torch.fft, name)


_fft_family()


# --------------------------------------------------------------------------- special functions
airy_ai, digamma, entr, erf, erfc, erfinv = (torch.special.airy_ai, torch.special.digamma, torch.special.entr,
                                             torch.special.erf, torch.special.erfc, torch.special.erfinv)
expm1, log1p, gammaln, lgamma, gammainc, gammaincc = (torch.special.expm1, torch.special.log1p, torch.special.gammaln,
                                                     torch.lgamma, torch.special.gammainc, torch.special.gammaincc)
i0, i0e, i1, i1e, ndtr, ndtri = (torch.special.i0, torch.special.i0e, torch.special.i1, torch.special.i1e,
                                 torch.special.ndtr, torch.special.ndtri)
sinc, xlogy, zeta, multigammaln = torch.special.sinc, torch.special.xlogy, torch.special.zeta, torch.special.multigammaln
mvlgamma = torch.special.multigammaln
modified_bessel_k0, modified_bessel_k1 = torch.special.modified_bessel_k0, torch.special.modified_bessel_k1
scaled_modified_bessel_k0, scaled_modified_bessel_k1 = (torch.special.scaled_modified_bessel_k0,
                                                        torch.special.scaled_modified_bessel_k1)
spherical_bessel_j0 = torch.special.spherical_bessel_j0


def log_beta(a: Tensor, b: Tensor) -> Tensor:
    return torch.lgamma(a) + torch.lgamma(b) - torch.lgamma(a + b)


def beta(a: Tensor, b: Tensor) -> Tensor:
    return torch.exp(log_beta(a, b))


def gammaln_sign(x: Tensor) -> Tensor:
    """Sign of Gamma(x): +1 for x > 0, alternating between the negative integers, NaN at the poles."""
    neg = x < 0
    fl = torch.floor(x)
    sign = torch.where(neg & (torch.remainder(fl, 2) != 0), -torch.ones_like(x), torch.ones_like(x))
    return torch.where((x <= 0) & (x == fl), torch.full_like(x, float("nan")), sign)


# --------------------------------------------------------------------------- masked tensors
class MaskedTensor:
    """Data plus a validity mask (True = valid), masked.rs."""

    def __init__(self, data: Tensor, mask: Tensor):
        if mask.shape != data.shape:
            raise FerrotorchError("MaskedTensor: mask shape %s != data shape %s" % (tuple(mask.shape), tuple(data.shape)))
        self.data, self.mask = data, mask.bool()

    def filled(self, value=None) -> Tensor:
        value = self._fill if value is None else value
        return torch.where(self.mask, self.data, torch.full_like(self.data, value))

    # ---- masked.rs accessors
    _fill = 0.0

    @classmethod
    def from_data(cls, data: Tensor, mask: Tensor) -> "MaskedTensor":
        return cls(data, mask)

    def with_fill_value(self, value) -> "MaskedTensor":
        out = MaskedTensor(self.data, self.mask)
        out._fill = value
        return out

    def fill_value(self):
        return self._fill

    def count_valid(self) -> int:
        return int(self.mask.sum())

    def count_masked(self) -> int:
        return self.mask.numel() - self.count_valid()

    def numel(self) -> int:
        return self.data.numel()

    @property
    def shape(self):
        return tuple(self.data.shape)

    def to_tensor(self) -> Tensor:
        """The data with the fill value where the mask is off."""
        return self.filled()

    def to_ferray(self):
        """A ``numpy.ma`` masked array (numpy's mask marks the *invalid* entries)."""
        import numpy as np

        return np.ma.array(self.data.detach().cpu().numpy(), mask=(~self.mask).cpu().numpy(), fill_value=self._fill)


def masked_where(data: Tensor, condition) -> MaskedTensor:
    """Mask out (invalidate) where ``condition`` holds."""
    c = torch.as_tensor(condition, dtype=torch.bool, device=data.device)
    if c.numel() != data.numel():
        raise FerrotorchError("masked_where: condition has %d elements, data has %d" % (c.numel(), data.numel()))
    return MaskedTensor(data, ~c.reshape(data.shape))


def masked_invalid(data: Tensor) -> MaskedTensor:
    return MaskedTensor(data, torch.isfinite(data))


def masked_equal(data: Tensor, value) -> MaskedTensor:
    return MaskedTensor(data, data != value)


def masked_sum(mt: MaskedTensor) -> Tensor:
    return mt.filled(0.0).sum()


def masked_count(mt: MaskedTensor) -> Tensor:
    return mt.mask.sum().to(mt.data.dtype)


def masked_mean(mt: MaskedTensor) -> Tensor:
    return masked_sum(mt) / masked_count(mt)


def masked_min(mt: MaskedTensor) -> Tensor:
    return mt.filled(float("inf")).min()


def masked_max(mt: MaskedTensor) -> Tensor:
    return mt.filled(float("-inf")).max()


masked_select = torch.masked_select


# --------------------------------------------------------------------------- forward-mode ops on dual tensors
def _dual(fn_name):
    def op(a: "_ag.DualTensor", *rest):
        return getattr(a, fn_name)(*rest)
    op.__name__ = "dual_" + fn_name.strip("_")
    return op


dual_add, dual_sub, dual_mul, dual_div, dual_matmul, dual_neg = (_dual("__add__"), _dual("__sub__"), _dual("__mul__"),
                                                                 _dual("__truediv__"), _dual("__matmul__"), _dual("__neg__"))
dual_exp, dual_log, dual_sin, dual_cos, dual_tanh, dual_relu = (_dual("exp"), _dual("log"), _dual("sin"), _dual("cos"),
                                                                _dual("tanh"), _dual("relu"))


def dual_sigmoid(a: "_ag.DualTensor") -> "_ag.DualTensor":
    return a.apply(torch.sigmoid)


# --------------------------------------------------------------------------- pruning, sparsity, quantisation names
def magnitude_prune(weights: Tensor, sparsity: float) -> Tensor:
    """Zero the ``sparsity`` fraction of smallest magnitudes (pruning.rs:72)."""
    if not 0.0 <= sparsity < 1.0:
        raise FerrotorchError("sparsity must be in [0, 1), got %r" % sparsity)
    k = int(weights.numel() * sparsity)
    if k == 0:
        return weights.clone()
    thresh = weights.abs().flatten().kthvalue(k).values
    return torch.where(weights.abs() <= thresh, torch.zeros_like(weights), weights)


def sparsity_ratio(t: Tensor) -> float:
    return float((t == 0).sum()) / max(1, t.numel())


def CooTensor(indices: Tensor, values: Tensor, size) -> Tensor:
    return torch.sparse_coo_tensor(indices, values, tuple(size))


def CsrTensor(crow_indices: Tensor, col_indices: Tensor, values: Tensor, size) -> Tensor:
    return torch.sparse_csr_tensor(crow_indices, col_indices, values, tuple(size))


def CscTensor(ccol_indices: Tensor, row_indices: Tensor, values: Tensor, size) -> Tensor:
    return torch.sparse_csc_tensor(ccol_indices, row_indices, values, tuple(size))


SparseGrad = torch.Tensor            # a sparse COO gradient, as ``nn.Embedding(sparse=True)`` produces


class SemiStructuredSparseTensor:
    """2:4-compressed matrix: kept values ``[N, K/2]`` and 2-bit positions ``[N, K/8]`` bytes, the
    form this framework's sparse GEMM reads (``ops.quant.pack_2_4``)."""

    def __init__(self, values: Tensor, meta: Tensor, shape):
        self.values, self.meta, self.shape = values, meta, tuple(shape)

    @classmethod
    def from_dense(cls, w: Tensor) -> "SemiStructuredSparseTensor":
        from .ops.quant import apply_2_4_mask, pack_2_4

        values, meta = pack_2_4(apply_2_4_mask(w))
        return cls(values, meta, w.shape)

    def linear(self, x: Tensor, bias: Tensor | None = None) -> Tensor:
        from .ops.quant import sparse24_linear

        return sparse24_linear(x, self.values, self.meta, bias)

    def to_dense(self) -> Tensor:
        from .ops.quant import unpack_2_4

        return unpack_2_4(self.values, self.meta)

    # ---- sparse.rs ``SemiStructuredSparseTensor`` / ``CudaSemiStructuredSparseTensor`` accessors
    @classmethod
    def compress(cls, dense: Tensor) -> "SemiStructuredSparseTensor":
        """Keep the two largest magnitudes of every group of four along the last dimension."""
        if dense.dim() != 2 or dense.shape[1] % 8:
            raise FerrotorchError("2:4 compression needs a matrix whose second dimension is a multiple of 8, got %s" % (tuple(dense.shape),))
        return cls.from_dense(dense)

    decompress = to_dense

    def num_groups(self) -> int:
        return self.shape[0] * self.shape[1] // 4

    def compression_ratio(self) -> float:
        """Dense bytes over compressed bytes (values + position bits)."""
        dense = self.shape[0] * self.shape[1] * self.values.element_size()
        return dense / (self.values.numel() * self.values.element_size() + self.meta.numel() * self.meta.element_size())

    def mask(self) -> Tensor:
        """Which dense positions are kept (exactly two per group of four)."""
        ones = SemiStructuredSparseTensor(torch.ones_like(self.values), self.meta, self.shape)
        return ones.to_dense() != 0

    def group_mask(self, group: int) -> list:
        """The four keep flags of group ``group`` (row-major over the groups)."""
        if not 0 <= group < self.num_groups():
            raise FerrotorchError("group %d of %d" % (group, self.num_groups()))
        r, c = divmod(group, self.shape[1] // 4)
        return self.mask()[r, 4 * c:4 * c + 4].tolist()

    backend = "expand-gemm"             # one implementation here: the compressed weight is expanded inside the GEMM

    @property
    def packed(self) -> Tensor:
        return self.values

    @property
    def indices(self) -> Tensor:
        return self.meta

    def values_shape(self) -> tuple:
        return tuple(self.values.shape)

    def indices_shape(self) -> tuple:
        return tuple(self.meta.shape)


CudaSemiStructuredSparseTensor = SemiStructuredSparseTensor
to_sparse_semi_structured = SemiStructuredSparseTensor.from_dense
to_sparse_semi_structured_cutlass = to_sparse_semi_structured_cusparselt = SemiStructuredSparseTensor.from_dense


class SemiStructuredSparseBackend(enum.Enum):
    """One implementation here (this framework's expand-GEMM); the names remain for callers that pass one."""
    Cutlass = "cutlass"
    CuSparseLt = "cusparselt"

    def as_str(self) -> str:
        return self.value


def sparse_matmul_24(a: Tensor, b: SemiStructuredSparseTensor) -> Tensor:
    """``a [M, K] @ dense(b)[N, K].T``."""
    return b.linear(a)


def PackedNestedTensor(tensors) -> Tensor:
    return torch.nested.nested_tensor(list(tensors), layout=torch.jagged)


def fake_quantize_differentiable(x: Tensor, scale: float, zero_point: int, qmin: int = -128, qmax: int = 127) -> Tensor:
    """Quantise-dequantise with a straight-through gradient inside the representable range."""
    return torch.fake_quantize_per_tensor_affine(x, float(scale), int(zero_point), qmin, qmax)


def __getattr__(name):
    """QAT / observer names live in ``nn``; loaded on demand to keep this module light."""
    if name in ("FakeQuantize", "QatModel", "prepare_qat", "QatLayer", "Observer", "cuda_rng"):
        if name == "cuda_rng":
            from .utils import philox

            return philox
        from . import nn

        return {"QatLayer": nn.QatLinear, "Observer": nn.MinMaxObserver}.get(name) or getattr(nn, name)
    raise AttributeError(name)
