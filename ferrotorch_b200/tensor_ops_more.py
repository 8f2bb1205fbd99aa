"""The rest of the reference core crate's free functions (``ferrotorch-core/src/{ops,linalg,signal,shape,
stride_tricks,meta_propagate,vmap,special}``): per-dimension reductions, differentiable linear-algebra
spellings, window functions that torch does not ship, stride arithmetic, meta-tensor constructors,
broadcasting helpers.  Names that torch already has under the same spelling (``torch.linalg``,
``torch.special``, ``torch.nn.functional``, ``torch.signal.windows``) are found by the package root's
fallback chain and are not repeated here.
"""
from __future__ import annotations

import math
from typing import Callable, Sequence

import torch
from torch import Tensor

from .tensor_ops import FerrotorchError


# --------------------------------------------------------------------------- reductions along one dimension
def all_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.all(dim, keepdim)


def any_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.any(dim, keepdim)


def amax_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.amax(dim, keepdim)


def amin_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.amin(dim, keepdim)


def argmax_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.argmax(dim, keepdim)


def argmin_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.argmin(dim, keepdim)


def prod_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return x.prod(dim, keepdim)


def count_nonzero_dim(x: Tensor, dim: int) -> Tensor:
    return torch.count_nonzero(x, dim)


def logsumexp_dim(x: Tensor, dim: int, keepdim: bool = False) -> Tensor:
    return torch.logsumexp(x, dim, keepdim)


def sum_axis(x: Tensor, axis: int, keepdim: bool = False) -> Tensor:
    return x.sum(axis, keepdim)


def std_with_correction(x: Tensor, dim=None, correction: int = 1, keepdim: bool = False) -> Tensor:
    return torch.std(x, dim, correction=correction, keepdim=keepdim)


def var_with_correction(x: Tensor, dim=None, correction: int = 1, keepdim: bool = False) -> Tensor:
    return torch.var(x, dim, correction=correction, keepdim=keepdim)


def reduce_all(x: Tensor, op: str = "sum") -> Tensor:
    """``op``: sum, prod, max, min, mean."""
    return {"sum": x.sum, "prod": x.prod, "max": x.max, "min": x.min, "mean": x.mean}[op]()


def reduce_dim(x: Tensor, dim: int, op: str = "sum", keepdim: bool = False) -> Tensor:
    fn = {"sum": torch.sum, "prod": torch.prod, "max": torch.amax, "min": torch.amin, "mean": torch.mean}[op]
    return fn(x, dim, keepdim=keepdim)


def sum_f32(x: Tensor) -> float:
    return float(x.float().sum())


def sum_f64(x: Tensor) -> float:
    return float(x.double().sum())


def l2_norm_f32_torch(x: Tensor) -> float:
    return float(torch.linalg.vector_norm(x.float()))


def reverse_cumsum(x: Tensor, dim: int) -> Tensor:
    """``out[i] = sum(x[i:])`` along ``dim``."""
    return x.flip(dim).cumsum(dim).flip(dim)


cumsum_forward, cumprod_forward = torch.cumsum, torch.cumprod
logcumsumexp_forward = torch.logcumsumexp


def cummax_forward(x: Tensor, dim: int):
    r = torch.cummax(x, dim)
    return r.values, r.indices


def cummin_forward(x: Tensor, dim: int):
    r = torch.cummin(x, dim)
    return r.values, r.indices


# --------------------------------------------------------------------------- scaled sums, out-variants, maps
def add_scaled(a: Tensor, b: Tensor, alpha: float) -> Tensor:
    return torch.add(a, b, alpha=alpha)


def sub_scaled(a: Tensor, b: Tensor, alpha: float) -> Tensor:
    return torch.sub(a, b, alpha=alpha)


def add_out(a: Tensor, b: Tensor, out: Tensor) -> Tensor:
    return torch.add(a, b, out=out)


def add_scaled_out(a: Tensor, b: Tensor, alpha: float, out: Tensor) -> Tensor:
    return torch.add(a, b, alpha=alpha, out=out)


def unary_map(x: Tensor, f: Callable[[Tensor], Tensor]) -> Tensor:
    """``f`` applied to the whole tensor at once (the reference maps a scalar closure element by element)."""
    out = f(x)
    if out.shape != x.shape:
        raise FerrotorchError("unary_map: the function changed the shape from %s to %s" % (tuple(x.shape), tuple(out.shape)))
    return out


unary_same_shape = scalar_map = unary_map


def unary_map_named(x: Tensor, name: str) -> Tensor:
    """A unary operator by name (``"exp"``, ``"relu"``, ``"erf"`` ...)."""
    for home in (torch, torch.special, torch.nn.functional):
        if hasattr(home, name):
            return getattr(home, name)(x)
    raise FerrotorchError("unary_map_named: no unary operator called %r" % name)


def binary_map(a: Tensor, b: Tensor, f: Callable[[Tensor, Tensor], Tensor]) -> Tensor:
    if a.shape != b.shape:
        raise FerrotorchError("binary_map: shapes %s and %s differ (use binary_broadcast)" % (tuple(a.shape), tuple(b.shape)))
    return f(a, b)


def binary_broadcast(a: Tensor, b: Tensor, f: Callable[[Tensor, Tensor], Tensor]) -> Tensor:
    a, b = torch.broadcast_tensors(a, b)
    return f(a, b)


def ternary_broadcast(a: Tensor, b: Tensor, c: Tensor, f: Callable[[Tensor, Tensor, Tensor], Tensor]) -> Tensor:
    a, b, c = torch.broadcast_tensors(a, b, c)
    return f(a, b, c)


def check_shapes_match(a: Tensor, b: Tensor, what: str = "operands") -> None:
    if a.shape != b.shape:
        raise FerrotorchError("%s: shape %s does not match %s" % (what, tuple(a.shape), tuple(b.shape)))


def where_(cond: Tensor, a: Tensor, b: Tensor) -> Tensor:
    return torch.where(cond, a, b)


where_bt = where_cond_bcast = where_


def masked_fill_bcast(x: Tensor, mask: Tensor, value) -> Tensor:
    """``mask`` broadcasts against ``x``."""
    return x.masked_fill(mask.expand_as(x) if mask.shape != x.shape else mask, value)


masked_fill_bt = masked_fill_bcast


def masked_select_bcast(x: Tensor, mask: Tensor) -> Tensor:
    x, mask = torch.broadcast_tensors(x, mask)
    return x.masked_select(mask)


def scatter_value(x: Tensor, dim: int, index: Tensor, value) -> Tensor:
    return x.scatter(dim, index, value)


def index_select_dim(x: Tensor, dim: int, index: Tensor) -> Tensor:
    return x.index_select(dim, index)


def index_select_1d(x: Tensor, index: Tensor) -> Tensor:
    if x.dim() != 1:
        raise FerrotorchError("index_select_1d: expected a vector, got %d dimensions" % x.dim())
    return x.index_select(0, index)


def index_select_1d_it(x: Tensor, indices) -> Tensor:
    return index_select_1d(x, torch.as_tensor(list(indices), dtype=torch.long, device=x.device))


def transpose_2d(x: Tensor) -> Tensor:
    if x.dim() != 2:
        raise FerrotorchError("transpose_2d: expected a matrix, got %d dimensions" % x.dim())
    return x.t().contiguous()


def permute_0213(x: Tensor) -> Tensor:
    return x.permute(0, 2, 1, 3).contiguous()


def cast(x: Tensor, dtype: torch.dtype) -> Tensor:
    return x.to(dtype)


def is_f32(x: Tensor) -> bool:
    return x.dtype == torch.float32


def is_f64(x: Tensor) -> bool:
    return x.dtype == torch.float64


def is_f16(x: Tensor) -> bool:
    return x.dtype == torch.float16


def is_bf16(x: Tensor) -> bool:
    return x.dtype == torch.bfloat16


# elementwise spellings whose fast / SIMD paths are torch's vectorised kernels
fast_add, fast_sub, fast_mul, fast_div = torch.add, torch.sub, torch.mul, torch.div
fast_exp, fast_log, fast_sin, fast_cos, fast_tanh, fast_sigmoid = torch.exp, torch.log, torch.sin, torch.cos, torch.tanh, torch.sigmoid
simd_add_f32 = simd_add_f64 = torch.add
simd_mul_f32 = simd_mul_f64 = torch.mul
simd_exp_f32 = simd_exp_f64 = torch.exp
simd_log_f32, simd_sqrt_f32 = torch.log, torch.sqrt


def hardtanh_with(x: Tensor, min_val: float, max_val: float) -> Tensor:
    return torch.nn.functional.hardtanh(x, min_val, max_val)


# --------------------------------------------------------------------------- linear algebra: differentiable spellings
# torch's operators are differentiable as they are; the reference keeps a raw and a recorded form of each.
matmul_differentiable = mm_differentiable = mm_raw = torch.matmul
bmm_differentiable, mv_differentiable, dot_differentiable, outer_differentiable = torch.bmm, torch.mv, torch.dot, torch.outer
det_differentiable, inv_differentiable, trace_differentiable = torch.linalg.det, torch.linalg.inv, torch.trace
cholesky_differentiable, qr_differentiable, solve_differentiable = torch.linalg.cholesky, torch.linalg.qr, torch.linalg.solve
slogdet_differentiable, matrix_exp_differentiable = torch.linalg.slogdet, torch.linalg.matrix_exp
solve_triangular_differentiable = torch.linalg.solve_triangular


def mm_bt_differentiable(a: Tensor, b: Tensor) -> Tensor:
    """``a @ b.T`` (the layout of a linear layer's weight)."""
    return a @ b.transpose(-1, -2)


mm_raw_bt = mm_bt_differentiable


def mm_raw_at(a: Tensor, b: Tensor) -> Tensor:
    return a.transpose(-1, -2) @ b


def linear_fused(x: Tensor, weight: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x @ weight.T + bias`` in one call (grad_fns/linalg.rs:1600); bf16 CUDA operands go to this package's GEMM."""
    from . import nn

    return nn.functional.linear(x, weight, bias) if not (x.is_cuda and x.dtype == torch.bfloat16) else \
        __import__("ferrotorch_b200.ops.functional", fromlist=["linear"]).linear(x, weight, bias)


def matrix_norm_ord(x: Tensor, ord="fro", dim=(-2, -1), keepdim: bool = False) -> Tensor:  # noqa: A002
    return torch.linalg.matrix_norm(x, ord, dim, keepdim)


def matrix_rank_atol_rtol(x: Tensor, atol: float | None = None, rtol: float | None = None, hermitian: bool = False) -> Tensor:
    return torch.linalg.matrix_rank(x, atol=atol, rtol=rtol, hermitian=hermitian)


matrix_rank_atol_rtol_tensors = matrix_rank_with_options = matrix_rank_atol_rtol


def matrix_rank_tol_tensor(x: Tensor, tol: Tensor | float) -> Tensor:
    return torch.linalg.matrix_rank(x, tol=float(tol))


def lstsq_solve(a: Tensor, b: Tensor) -> Tensor:
    return torch.linalg.lstsq(a, b).solution


def lstsq_with_driver(a: Tensor, b: Tensor, driver: str = "gelsd"):
    return torch.linalg.lstsq(a, b, driver=driver)


def lu_factor_ex_with_options(a: Tensor, pivot: bool = True, check_errors: bool = False):
    return torch.linalg.lu_factor_ex(a, pivot=pivot, check_errors=check_errors)


def ldl_solve(ld: Tensor, pivots: Tensor, b: Tensor, hermitian: bool = False) -> Tensor:
    return torch.linalg.ldl_solve(ld, pivots, b, hermitian=hermitian)


def householder_product_full(v: Tensor, tau: Tensor) -> Tensor:
    """The full square orthogonal factor of the reflectors in ``v [m, k]``: ``v`` is padded with unit columns
    whose coefficient is zero (identity reflectors)."""
    m, k = v.shape[-2], v.shape[-1]
    if k >= m:
        return torch.linalg.householder_product(v, tau)
    pad_v = torch.cat([v, torch.zeros(*v.shape[:-1], m - k, dtype=v.dtype, device=v.device)], -1)
    pad_t = torch.cat([tau, torch.zeros(*tau.shape[:-1], m - k, dtype=tau.dtype, device=tau.device)], -1)
    return torch.linalg.householder_product(pad_v, pad_t)


# --------------------------------------------------------------------------- windows torch does not have
def _window_positions(n: int, sym: bool, dtype) -> tuple[Tensor, int]:
    m = n if sym else n + 1
    return torch.arange(n, dtype=dtype), m


def hanning(n: int, sym: bool = True, dtype=torch.float32) -> Tensor:
    """numpy's name for the Hann window."""
    return torch.signal.windows.hann(n, sym=sym, dtype=dtype)


def parzen(n: int, sym: bool = True, dtype=torch.float32) -> Tensor:
    """Piecewise-cubic B-spline window (four-fold convolution of a rectangle)."""
    if n <= 1:
        return torch.ones(max(n, 0), dtype=dtype)
    k, m = _window_positions(n, sym, torch.float64)
    x = (k - (m - 1) / 2.0).abs() / (m / 2.0)
    w = torch.where(x <= 0.5, 1 - 6 * x ** 2 * (1 - x), 2 * (1 - x) ** 3)
    return w.to(dtype)


def tukey(n: int, alpha: float = 0.5, sym: bool = True, dtype=torch.float32) -> Tensor:
    """Flat top with cosine tapers over a fraction ``alpha`` of the window (0: rectangular, 1: Hann)."""
    if n <= 1:
        return torch.ones(max(n, 0), dtype=dtype)
    if alpha <= 0:
        return torch.ones(n, dtype=dtype)
    if alpha >= 1:
        return torch.signal.windows.hann(n, sym=sym, dtype=dtype)
    k, m = _window_positions(n, sym, torch.float64)
    width = alpha * (m - 1) / 2.0
    w = torch.ones(n, dtype=torch.float64)
    left, right = k < width, k > (m - 1) - width
    w[left] = 0.5 * (1 + torch.cos(math.pi * (k[left] / width - 1)))
    w[right] = 0.5 * (1 + torch.cos(math.pi * ((k[right] - (m - 1)) / width + 1)))
    return w.to(dtype)


def taylor(n: int, nbar: int = 4, sll: float = 30.0, norm: bool = True, sym: bool = True, dtype=torch.float32) -> Tensor:
    """Taylor window: ``nbar`` nearly constant side lobes ``sll`` dB below the main lobe (radar weighting)."""
    if n <= 1:
        return torch.ones(max(n, 0), dtype=dtype)
    k, m = _window_positions(n, sym, torch.float64)
    b = 10 ** (sll / 20.0)
    a = math.acosh(b) / math.pi
    s2 = nbar ** 2 / (a ** 2 + (nbar - 0.5) ** 2)
    ma = torch.arange(1, nbar, dtype=torch.float64)
    fm = torch.empty(nbar - 1, dtype=torch.float64)
    signs = torch.tensor([(-1.0) ** (i + 1) for i in range(1, nbar)], dtype=torch.float64)
    for i, mi in enumerate(ma.tolist()):
        numer = signs[i] * torch.prod(1 - mi ** 2 / s2 / (a ** 2 + (ma - 0.5) ** 2))
        others = torch.cat([ma[:i], ma[i + 1:]])
        denom = 2 * torch.prod(1 - mi ** 2 / others ** 2)
        fm[i] = numer / denom

    def w_of(pos: Tensor) -> Tensor:
        return 1 + 2 * (fm[None, :] * torch.cos(2 * math.pi * ma[None, :] * (pos[:, None] - m / 2.0 + 0.5) / m)).sum(-1)

    w = w_of(k)
    if norm:
        w = w / w_of(torch.tensor([(m - 1) / 2.0], dtype=torch.float64))
    return w.to(dtype)


# --------------------------------------------------------------------------- stride arithmetic (stride_tricks.rs, shape.rs)
def checked_numel(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        if d < 0:
            raise FerrotorchError("negative extent %d in shape %s" % (d, tuple(shape)))
        n *= int(d)
    if n > 2 ** 63 - 1:
        raise FerrotorchError("shape %s has more than 2^63 - 1 elements" % (tuple(shape),))
    return n


def checked_byte_count(shape: Sequence[int], itemsize: int) -> int:
    n = checked_numel(shape) * int(itemsize)
    if n > 2 ** 63 - 1:
        raise FerrotorchError("shape %s with %d-byte elements overflows a signed 64-bit byte count" % (tuple(shape), itemsize))
    return n


def c_contiguous_strides(shape: Sequence[int]) -> tuple:
    strides, acc = [], 1
    for d in reversed(tuple(shape)):
        strides.append(acc)
        acc *= max(int(d), 1)
    return tuple(reversed(strides))


def channels_last_strides(shape: Sequence[int]) -> tuple:
    """Strides of an ``[N, C, H, W]`` tensor stored as N, H, W, C."""
    if len(shape) != 4:
        raise FerrotorchError("channels_last_strides: expected 4 dimensions, got %d" % len(shape))
    n, c, h, w = (max(int(d), 1) for d in shape)
    return (h * w * c, 1, w * c, c)


def channels_last_3d_strides(shape: Sequence[int]) -> tuple:
    if len(shape) != 5:
        raise FerrotorchError("channels_last_3d_strides: expected 5 dimensions, got %d" % len(shape))
    n, c, d, h, w = (max(int(v), 1) for v in shape)
    return (d * h * w * c, 1, h * w * c, w * c, c)


def checked_c_contiguous_strides(shape: Sequence[int]) -> tuple:
    checked_numel(shape)
    return c_contiguous_strides(shape)


def checked_channels_last_strides(shape: Sequence[int]) -> tuple:
    checked_numel(shape)
    return channels_last_strides(shape)


def checked_channels_last_3d_strides(shape: Sequence[int]) -> tuple:
    checked_numel(shape)
    return channels_last_3d_strides(shape)


# --------------------------------------------------------------------------- meta tensors (meta_propagate.rs)
def zeros_meta(shape, dtype=torch.float32) -> Tensor:
    return torch.zeros(tuple(shape), dtype=dtype, device="meta")


def ones_meta(shape, dtype=torch.float32) -> Tensor:
    return torch.ones(tuple(shape), dtype=dtype, device="meta")


def full_meta(shape, value, dtype=torch.float32) -> Tensor:
    return torch.full(tuple(shape), value, dtype=dtype, device="meta")


def meta_like(x: Tensor) -> Tensor:
    return torch.empty_like(x, device="meta")


# --------------------------------------------------------------------------- batching helpers (vmap.rs)
def vmap_many(f: Callable, in_dims=0, out_dims=0) -> Callable:
    """``torch.vmap`` over any number of inputs."""
    return torch.vmap(f, in_dims=in_dims, out_dims=out_dims)


vmap_multi_output = vmap_many


def vmap3(f: Callable, a: Tensor, b: Tensor, c: Tensor) -> Tensor:
    return torch.vmap(f)(a, b, c)


def per_sample_grad(f: Callable[[Tensor, Tensor], Tensor], params: Tensor, inputs: Tensor) -> Tensor:
    """Gradient of ``f(params, x)`` with respect to ``params`` for every row ``x`` of ``inputs``: ``[B, *params.shape]``."""
    return torch.vmap(torch.func.grad(f), in_dims=(None, 0))(params, inputs)


# --------------------------------------------------------------------------- host buffer pool statistics (cpu_pool.rs)
def cpu_pool_stats() -> dict:
    """torch's host allocator keeps no reuse pool for pageable memory; pinned memory is cached by its own
    allocator, whose counters these are."""
    st = torch.cuda.host_memory_stats() if hasattr(torch.cuda, "host_memory_stats") and torch.cuda.is_available() else {}
    return {"hits": 0, "misses": 0, "pinned_allocated_bytes": st.get("allocated_bytes.current", 0)}


def reset_cpu_pool_stats() -> None:
    if hasattr(torch.cuda, "reset_peak_host_memory_stats") and torch.cuda.is_available():
        torch.cuda.reset_peak_host_memory_stats()


def empty_cpu_pool() -> None:
    if hasattr(torch._C, "_host_emptyCache"):
        torch._C._host_emptyCache()


def fft_norm_from_str(norm: str | None) -> str:
    """``None`` / ``"backward"`` / ``"forward"`` / ``"ortho"`` checked and normalised."""
    n = "backward" if norm in (None, "") else str(norm).lower()
    if n not in ("backward", "forward", "ortho"):
        raise FerrotorchError("fft norm must be backward, forward or ortho, got %r" % (norm,))
    return n


# --------------------------------------------------------------------------- autograd / autocast / profiler plumbing under its reference names
def checkpoint_multi(fn: Callable, *inputs):
    """Activation checkpointing of a function with several inputs and outputs (autograd/checkpoint.rs)."""
    from torch.utils.checkpoint import checkpoint

    return checkpoint(fn, *inputs, use_reentrant=False)


def fake_quantize_per_tensor_affine_tensor_qparams(x: Tensor, scale: Tensor, zero_point: Tensor, quant_min: int, quant_max: int) -> Tensor:
    """Fake quantisation whose scale and zero point are one-element tensors on ``x``'s device (they may be learnt)."""
    if scale.numel() != 1 or zero_point.numel() != 1:
        raise FerrotorchError("fake_quantize_per_tensor_affine_tensor_qparams: scale and zero_point must hold one element each")
    if scale.device != x.device or zero_point.device != x.device:
        raise FerrotorchError("fake_quantize_per_tensor_affine_tensor_qparams: scale / zero_point must be on %s" % x.device)
    return torch.fake_quantize_per_tensor_affine(x, scale.reshape(()).float(), zero_point.reshape(()).to(torch.int32), quant_min, quant_max)


_AUTOCAST_REDUCED = {"matmul", "mm", "bmm", "linear", "conv1d", "conv2d", "conv3d", "addmm", "baddbmm", "einsum", "attention"}
_AUTOCAST_FULL = {"softmax", "log_softmax", "layer_norm", "group_norm", "batch_norm", "cross_entropy", "mse_loss", "exp", "log", "pow",
                  "sum", "mean", "prod", "norm", "cumsum", "rsqrt", "reciprocal"}


def autocast_log(op_name: str, device_type: str = "cuda"):
    """The autocast category of an op when autocast is active on ``device_type`` (``"reduced"``: runs in the
    autocast dtype; ``"full"``: kept in fp32; ``"keep"``: takes its inputs' dtype), else ``None``
    (autograd/autocast_ops.rs:42-110)."""
    if not torch.is_autocast_enabled(device_type):
        return None
    return "reduced" if op_name in _AUTOCAST_REDUCED else "full" if op_name in _AUTOCAST_FULL else "keep"


def current_autocast_snapshot() -> dict:
    """The autocast state of this thread for every device type, to carry into a worker thread."""
    return {d: (torch.is_autocast_enabled(d), torch.get_autocast_dtype(d)) for d in ("cpu", "cuda")}


class with_autocast_state:
    """``with with_autocast_state(snapshot): ...`` re-creates a snapshot taken on another thread."""

    def __init__(self, snapshot: dict):
        self._cms = [torch.autocast(d, dtype=dt, enabled=en) for d, (en, dt) in snapshot.items()]

    def __enter__(self):
        for cm in self._cms:
            cm.__enter__()
        return self

    def __exit__(self, *exc):
        for cm in reversed(self._cms):
            cm.__exit__(*exc)
        return False


_saved_hooks: list = []


class _TrackedSavedTensorsHooks(torch.autograd.graph.saved_tensors_hooks):
    """``saved_tensors_hooks`` that this module can see, for ``has_saved_tensor_hooks`` / ``pack_saved_tensor``."""

    def __init__(self, pack, unpack):
        super().__init__(pack, unpack)
        self._pair = (pack, unpack)

    def __enter__(self):
        _saved_hooks.append(self._pair)
        return super().__enter__()

    def __exit__(self, *exc):
        _saved_hooks.pop()
        return super().__exit__(*exc)


tracked_saved_tensors_hooks = _TrackedSavedTensorsHooks


def has_saved_tensor_hooks() -> bool:
    """Whether a :class:`tracked_saved_tensors_hooks` scope is open on this thread."""
    return bool(_saved_hooks)


def pack_saved_tensor(t: Tensor):
    """What the innermost open hook pair would store for ``t`` (``t`` itself without one)."""
    return _saved_hooks[-1][0](t) if _saved_hooks else t


def unpack_saved_tensor(packed):
    return _saved_hooks[-1][1](packed) if _saved_hooks else packed


_current_profiler: list = [None]


def set_current(profiler) -> None:
    """Install (or, with ``None``, clear) the profiler that :func:`profile_op_scope` reports to (profiler_hook.rs:69)."""
    _current_profiler[0] = profiler


def current():
    return _current_profiler[0]


def profile_op_scope(name: str, category: str = "op", shapes=()):
    """A context manager timing one op on the current profiler; does nothing when none is installed."""
    import contextlib

    p = _current_profiler[0]
    return p.scope(name, category, shapes) if p is not None else contextlib.nullcontext()


def with_thread_rng(f: Callable):
    """Run ``f(generator)`` on the process-wide default CPU generator (the one ``rand`` / ``randn`` and the
    initialisers use when none is given)."""
    return f(torch.default_generator)


def with_default_rng_test_lock(f: Callable):
    """Run ``f()`` with the default generator's state saved before and restored after, so that tests do not
    perturb one another's random streams."""
    state = torch.get_rng_state()
    try:
        return f()
    finally:
        torch.set_rng_state(state)


def has_gpu_backend() -> bool:
    return torch.cuda.is_available()


def gpu_backend():
    """The device back-end object (``cuda.CudaBackendImpl``) when a GPU is present, else ``None``."""
    if not torch.cuda.is_available():
        return None
    from . import cuda

    return cuda.CudaBackendImpl(torch.cuda.current_device())


def register_gpu_backend(backend) -> None:
    raise FerrotorchError("register_gpu_backend: this package has one device back-end, bound when it is imported; "
                          "custom kernels are registered with torch.library")


def pool_alloc_cpu(n: int, dtype=torch.float32) -> Tensor:
    """A zeroed host buffer of ``n`` elements (cpu_pool.rs:141); torch's allocator does the recycling."""
    return torch.zeros(n, dtype=dtype)


def pool_alloc_cpu_uninit_f32(n: int) -> Tensor:
    return torch.empty(n, dtype=torch.float32)


def pool_alloc_cpu_uninit_f64(n: int) -> Tensor:
    return torch.empty(n, dtype=torch.float64)


def pool_return_cpu(buffer: Tensor) -> None:
    """Hand a buffer back: dropping the last reference returns it to the allocator."""
    buffer.set_()
