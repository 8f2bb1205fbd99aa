"""Autograd surface under the reference's names (ferrotorch-core/src/autograd/mod.rs:10-45).

PyTorch's engine does the differentiation; this module gives its pieces the names a ferrotorch
user knows (``backward``, ``grad``, ``no_grad``, ``inference_mode``, ``detect_anomaly``,
``checkpoint``, ``saved_tensors_hooks``, ``jvp`` / ``vjp`` / ``jacobian`` / ``hessian`` / ``jacfwd``,
``gradcheck``, ``autocast``) and adds what torch has no single call for:

* :func:`fixed_point` -- differentiate through the solution of ``x = f(x, p)`` with the implicit
  function theorem instead of unrolling the iteration (fixed_point.rs:79-330);
* :func:`grad_norm`, :func:`gradient_penalty` (grad_penalty.rs);
* :func:`cond`, :func:`scan` (ops/higher_order.rs);
* :class:`DualTensor` -- forward-mode values as (primal, tangent) pairs (forward_ad.rs).
"""
from __future__ import annotations

import math
from typing import Callable, Sequence

import torch
from torch.autograd import grad, gradcheck  # noqa: F401
from torch.autograd.graph import saved_tensors_hooks  # noqa: F401
from torch.func import hessian, jacfwd, jacrev, vmap  # noqa: F401
from torch.utils.checkpoint import checkpoint as _torch_checkpoint

no_grad, enable_grad, inference_mode, set_grad_enabled = (torch.no_grad, torch.enable_grad, torch.inference_mode,
                                                          torch.set_grad_enabled)
is_grad_enabled, is_inference_mode = torch.is_grad_enabled, torch.is_inference_mode_enabled
detect_anomaly = torch.autograd.detect_anomaly
jacobian = torch.autograd.functional.jacobian


def backward(tensor: torch.Tensor, retain_graph: bool = False) -> None:
    """Reverse pass from a scalar (graph.rs:262 ``backward``)."""
    if tensor.numel() != 1:
        raise ValueError("backward: the root must hold one element; use backward_with_grad for others")
    tensor.backward(retain_graph=retain_graph)


def backward_with_grad(tensor: torch.Tensor, grad_output: torch.Tensor, retain_graph: bool = False) -> None:
    tensor.backward(grad_output, retain_graph=retain_graph)


def backward_parallel(tensor: torch.Tensor, grad_output: torch.Tensor | None = None, retain_graph: bool = False) -> None:
    """Reverse pass with independent branches run concurrently (graph.rs:415).  torch's engine
    already runs one worker thread per device and overlaps ready nodes across them, so this is
    ``backward`` with the optional seed gradient; it exists so that callers of the reference
    keep their call."""
    if grad_output is None and tensor.numel() != 1:
        raise ValueError("backward_parallel: a root with more than one element needs grad_output")
    tensor.backward(grad_output, retain_graph=retain_graph)


def checkpoint(fn: Callable, *args, preserve_rng_state: bool = True, **kw):
    """Recompute ``fn`` in backward instead of keeping its activations; CPU / CUDA RNG state and the
    autocast state at call time are restored for the recomputation (checkpoint.rs:76-121)."""
    return _torch_checkpoint(fn, *args, use_reentrant=False, preserve_rng_state=preserve_rng_state, **kw)


def jvp(fn: Callable, primals, tangents):
    """``(fn(primals), J . tangents)`` by forward-mode AD."""
    single = isinstance(primals, torch.Tensor)
    out, tan = torch.func.jvp(fn, (primals,) if single else tuple(primals), (tangents,) if single else tuple(tangents))
    return out, tan


jvp_exact = jvp


def vjp(fn: Callable, primals, cotangent):
    """``(fn(primals), cotangent . J)`` by reverse-mode AD; one tensor in gives one tensor back."""
    single = isinstance(primals, torch.Tensor)
    out, pull = torch.func.vjp(fn, *((primals,) if single else tuple(primals)))
    grads = pull(cotangent)
    return out, (grads[0] if single else grads)


def grad_norm(outputs: torch.Tensor, inputs: Sequence[torch.Tensor] | torch.Tensor, create_graph: bool = True) -> torch.Tensor:
    """L2 norm of ``d outputs / d inputs`` over all inputs, itself differentiable by default."""
    inputs = [inputs] if isinstance(inputs, torch.Tensor) else list(inputs)
    gs = torch.autograd.grad(outputs, inputs, torch.ones_like(outputs), create_graph=create_graph)
    return torch.sqrt(sum((g ** 2).sum() for g in gs))


def gradient_penalty(outputs: torch.Tensor, inputs: torch.Tensor, target: float = 1.0, weight: float = 1.0) -> torch.Tensor:
    """WGAN-GP term ``weight * mean((||d out / d in||_2 per sample - target)^2)``."""
    (g,) = torch.autograd.grad(outputs, inputs, torch.ones_like(outputs), create_graph=True)
    per_sample = g.flatten(1).norm(dim=1) if g.dim() > 1 else g.abs()
    return weight * ((per_sample - target) ** 2).mean()


def cond(pred, true_fn: Callable, false_fn: Callable, operands: Sequence = ()):
    """Run one of two branches; both must produce the same shapes and dtypes
    (``validate_cond_branches`` of the reference checks that up front, so does this)."""
    validate_cond_branches(true_fn, false_fn, operands)
    take_true = bool(pred.item()) if isinstance(pred, torch.Tensor) else bool(pred)
    return (true_fn if take_true else false_fn)(*operands)


def validate_cond_branches(true_fn: Callable, false_fn: Callable, operands: Sequence = ()) -> None:
    with torch.no_grad():
        a, b = true_fn(*operands), false_fn(*operands)
    fa, fb = (a if isinstance(a, (tuple, list)) else [a]), (b if isinstance(b, (tuple, list)) else [b])
    if len(fa) != len(fb) or any(x.shape != y.shape or x.dtype != y.dtype for x, y in zip(fa, fb)):
        raise ValueError("cond: the branches disagree on the shape or dtype of their results")


def scan(fn: Callable, init, xs: torch.Tensor):
    """``carry, y_t = fn(carry, xs[t])`` over the leading dimension; returns ``(carry, stacked ys)``."""
    carry, ys = init, []
    for t in range(xs.shape[0]):
        carry, y = fn(carry, xs[t])
        ys.append(y)
    return carry, (torch.stack(ys) if ys else xs.new_empty((0,)))


# --------------------------------------------------------------------------- implicit differentiation
class _FixedPoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f, x_star, max_iter, tol, *params):
        ctx.f, ctx.max_iter, ctx.tol = f, max_iter, tol
        ctx.save_for_backward(x_star, *params)
        return x_star.clone()

    @staticmethod
    def backward(ctx, grad_out):
        x_star, *params = ctx.saved_tensors
        with torch.enable_grad():
            x = x_star.detach().requires_grad_(True)
            ps = [p.detach().requires_grad_(p.requires_grad) for p in params]
            y = ctx.f(x, ps)
        # v = (I - J_x^T)^-1 g as the limit of v <- g + J_x^T v (the Neumann series, summed term by
        # term); it converges because f is contractive at the fixed point.
        v = grad_out
        for _ in range(ctx.max_iter):
            (jt_v,) = torch.autograd.grad(y, x, v, retain_graph=True, allow_unused=True)
            nxt = grad_out if jt_v is None else grad_out + jt_v
            done = float((nxt - v).abs().sum()) <= ctx.tol
            v = nxt
            if done or jt_v is None:
                break
        need = [p for p in ps if p.requires_grad]
        gs = torch.autograd.grad(y, need, v, allow_unused=True) if need else ()
        it = iter(gs)
        grads = [next(it) if p.requires_grad else None for p in ps]
        return (None, None, None, None, *grads)


def fixed_point(f: Callable, x0: torch.Tensor, params: Sequence[torch.Tensor], max_iter: int = 1000,
                tol: float = 1e-8) -> torch.Tensor:
    """Solve ``x* = f(x*, params)`` by iteration (no graph is kept) and return ``x*`` with a backward
    that applies the implicit function theorem: ``dL/dp = (df/dp)^T (I - (df/dx)^T)^-1 dL/dx*``.
    ``f(x, params) -> x_next`` must be contractive.  Raises when the iteration does not reach
    ``sum |x_next - x| <= tol`` within ``max_iter`` steps or produces a non-finite value."""
    if max_iter <= 0 or not (tol > 0 and math.isfinite(tol)):
        raise ValueError("fixed_point: max_iter must be positive and tol a positive finite number")
    params = list(params)
    with torch.no_grad():
        x, residual = x0, float("inf")
        for _ in range(max_iter):
            nxt = f(x, params)
            if nxt.shape != x.shape or nxt.dtype != x.dtype:
                raise ValueError("fixed_point forward: f changed the shape or dtype of the iterate")
            residual = float((nxt - x).abs().sum())
            if not math.isfinite(residual):
                raise ValueError("fixed_point forward: the residual became non-finite")
            x = nxt
            if residual <= tol:
                break
        else:
            raise RuntimeError("fixed_point forward: no convergence in %d iterations (residual %.3e > tol %.3e)"
                               % (max_iter, residual, tol))
    if not any(p.requires_grad for p in params) or not torch.is_grad_enabled():
        return x
    return _FixedPoint.apply(f, x, max_iter, tol, *params)


# --------------------------------------------------------------------------- forward-mode values
class DualTensor:
    """A (primal, tangent) pair with arithmetic that pushes the tangent forward (forward_ad.rs).
    For whole functions use :func:`jvp` / :func:`jacfwd`; this is the value-level view."""

    def __init__(self, primal: torch.Tensor, tangent: torch.Tensor | None = None):
        self.primal = primal
        self.tangent = torch.zeros_like(primal) if tangent is None else tangent
        if self.tangent.shape != primal.shape:
            raise ValueError("DualTensor: the tangent must have the primal's shape")

    @staticmethod
    def _lift(o) -> "DualTensor":
        return o if isinstance(o, DualTensor) else DualTensor(torch.as_tensor(o))

    @classmethod
    def constant(cls, primal: torch.Tensor) -> "DualTensor":
        """A value that does not depend on the differentiation variable: zero tangent."""
        return cls(primal)

    @property
    def shape(self):
        return tuple(self.primal.shape)

    def numel(self) -> int:
        return self.primal.numel()

    def __add__(self, o):
        o = self._lift(o)
        return DualTensor(self.primal + o.primal, self.tangent + o.tangent)

    __radd__ = __add__

    def __sub__(self, o):
        o = self._lift(o)
        return DualTensor(self.primal - o.primal, self.tangent - o.tangent)

    def __neg__(self):
        return DualTensor(-self.primal, -self.tangent)

    def __mul__(self, o):
        o = self._lift(o)
        return DualTensor(self.primal * o.primal, self.tangent * o.primal + self.primal * o.tangent)

    __rmul__ = __mul__

    def __truediv__(self, o):
        o = self._lift(o)
        return DualTensor(self.primal / o.primal, (self.tangent * o.primal - self.primal * o.tangent) / (o.primal ** 2))

    def __matmul__(self, o):
        o = self._lift(o)
        return DualTensor(self.primal @ o.primal, self.tangent @ o.primal + self.primal @ o.tangent)

    def apply(self, fn: Callable) -> "DualTensor":
        """Any differentiable ``fn`` of one tensor, through ``torch.func.jvp``."""
        out, tan = torch.func.jvp(fn, (self.primal,), (self.tangent,))
        return DualTensor(out, tan)

    def exp(self):
        return self.apply(torch.exp)

    def log(self):
        return self.apply(torch.log)

    def sin(self):
        return self.apply(torch.sin)

    def cos(self):
        return self.apply(torch.cos)

    def tanh(self):
        return self.apply(torch.tanh)

    def relu(self):
        return self.apply(torch.relu)

    def sum(self):
        return DualTensor(self.primal.sum(), self.tangent.sum())


# --------------------------------------------------------------------------- autocast policy and debug events
_autocast_depth = 0


class autocast(torch.autocast):
    """``torch.autocast`` that also tells the debug recorder when a region is active (inside a
    dispatch-mode handler torch reports autocast as off, so the recorder cannot ask torch)."""

    def __enter__(self):
        global _autocast_depth
        r = super().__enter__()
        if self._enabled:
            _autocast_depth += 1
        return r

    def __exit__(self, *exc):
        global _autocast_depth
        if self._enabled:
            _autocast_depth -= 1
        return super().__exit__(*exc)


class AutocastCategory:
    """How an op treats its inputs under autocast (autocast_ops.rs:30-58)."""
    ReducedPrecision, FullPrecision, Passthrough = "reduced_precision", "full_precision", "passthrough"


_REDUCED = {"mm", "matmul", "bmm", "linear", "conv1d", "conv2d", "conv3d", "conv_transpose2d", "addmm", "einsum",
            "scaled_dot_product_attention"}
_FULL = {"sum", "mean", "prod", "softmax", "log_softmax", "layer_norm", "batch_norm", "group_norm", "rms_norm",
         "cross_entropy", "mse_loss", "bce_with_logits", "exp", "log", "pow"}


def autocast_category(op_name: str) -> str:
    """The policy table: GEMM-shaped ops run in the autocast dtype, reductions / normalisations /
    losses stay in fp32, everything else follows its inputs."""
    op_name = op_name.lstrip("_")              # ATen spells some of them "_softmax", "_log_softmax"
    if op_name in _REDUCED:
        return AutocastCategory.ReducedPrecision
    if op_name in _FULL:
        return AutocastCategory.FullPrecision
    return AutocastCategory.Passthrough


def is_autocast_enabled(device_type: str | None = None) -> bool:
    if device_type is not None:
        return torch.is_autocast_enabled(device_type)
    return torch.is_autocast_enabled("cuda") or torch.is_autocast_enabled("cpu")


def should_cast_to_reduced(op_name: str) -> bool:
    return is_autocast_enabled() and autocast_category(op_name) == AutocastCategory.ReducedPrecision


def should_keep_full_precision(op_name: str) -> bool:
    return is_autocast_enabled() and autocast_category(op_name) == AutocastCategory.FullPrecision


_autocast_debug = False
_autocast_events: list = []
_autocast_mode = None


class _AutocastRecorder(torch.utils._python_dispatch.TorchDispatchMode):
    """Sees every ATen call below autocast: records the op with the dtypes that reached it."""

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        out = func(*args, **(kwargs or {}))
        if _autocast_depth > 0:
            name = func.overloadpacket.__name__
            ins = [str(a.dtype).replace("torch.", "") for a in torch.utils._pytree.tree_flatten((args, kwargs or {}))[0]
                   if isinstance(a, torch.Tensor)]
            o = out if isinstance(out, torch.Tensor) else None
            _autocast_events.append({"op": name, "category": autocast_category(name), "inputs": ins,
                                     "output": str(o.dtype).replace("torch.", "") if o is not None else None})
        return out


def set_autocast_debug(on: bool) -> None:
    """While on, every op executed inside an ``autocast`` region is logged with its policy category
    and the dtypes it actually ran in; :func:`drain_autocast_events` returns and clears the log
    (autocast_ops.rs:86-132)."""
    global _autocast_debug, _autocast_mode
    if on and not _autocast_debug:
        _autocast_mode = _AutocastRecorder()
        _autocast_mode.__enter__()
    elif not on and _autocast_debug and _autocast_mode is not None:
        _autocast_mode.__exit__(None, None, None)
        _autocast_mode = None
    _autocast_debug = bool(on)


def is_autocast_debug() -> bool:
    return _autocast_debug


def drain_autocast_events() -> list:
    out = list(_autocast_events)
    _autocast_events.clear()
    return out
