"""Optimizers and helpers torch does not ship (reference: ferrotorch-optim/src/{muon,adafactor,
natural_gradient,ema,swa}.rs, grad_accumulator, scheduler/warmup.rs)."""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR


QUINTIC_NS = (3.4445, -4.7750, 2.0315)      # Keller Jordan's Muon coefficients (torch/optim/_muon.py)
CUBIC_NS = (1.5, -0.5, 0.0)                  # G (3 I - G^T G) / 2, the reference's historic default (muon.rs)


def _newton_schulz(g: torch.Tensor, steps: int = 5, coefficients=QUINTIC_NS) -> torch.Tensor:
    """Newton-Schulz iteration ``X <- a X + b (X X^T) X + c (X X^T)^2 X`` that drives the singular
    values of a matrix towards one (Muon's orthogonalisation)."""
    a, b, c = coefficients
    x = g.float()
    transposed = x.shape[0] > x.shape[1]
    if transposed:
        x = x.t()
    x = x / (x.norm() + 1e-7)
    for _ in range(steps):
        s = x @ x.t()
        x = a * x + (b * s + c * s @ s) @ x
    return (x.t() if transposed else x).to(g.dtype)


class Muon(Optimizer):
    """Momentum + orthogonalised update for 2-D parameters (ferrotorch-optim/src/muon.rs).

    ``ns_coefficients``: the polynomial of the Newton-Schulz step (quintic by default; the
    reference's default is the cubic ``CUBIC_NS``).  ``decoupled_weight_decay``: shrink the weights by
    ``1 - lr * wd`` (default, as torch's Muon) or, when false, fold ``wd * p`` into the gradient before
    the orthogonalisation (the reference's default).  ``strict_2d``: refuse parameters that are not
    matrices instead of giving them plain momentum SGD.  ``maximize`` negates the gradient."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0, maximize=False,
                 ns_coefficients=QUINTIC_NS, decoupled_weight_decay=True, strict_2d=False):
        if len(tuple(ns_coefficients)) != 3:
            raise ValueError("Muon: ns_coefficients must be three numbers (a, b, c)")
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay, maximize=maximize, ns_coefficients=tuple(ns_coefficients),
                                      decoupled_weight_decay=decoupled_weight_decay, strict_2d=strict_2d))
        for g in self.param_groups:
            if g["strict_2d"]:
                bad = [tuple(p.shape) for p in g["params"] if p.dim() != 2]
                if bad:
                    raise ValueError("Muon only supports 2D parameters with strict_2d; got shapes %s" % bad)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = -p.grad if g["maximize"] else p.grad
                if g["weight_decay"] and not g["decoupled_weight_decay"]:
                    grad = grad.add(p, alpha=g["weight_decay"])
                st = self.state[p]
                buf = st.setdefault("momentum_buffer", torch.zeros_like(p))
                buf.mul_(g["momentum"]).add_(grad)
                upd = grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                if p.dim() == 2:
                    upd = _newton_schulz(upd, g["ns_steps"], g["ns_coefficients"]) * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                if g["weight_decay"] and g["decoupled_weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd, alpha=-g["lr"])
        return loss


class Adafactor(Optimizer):
    """Factored second moments for matrices (row / column statistics), Adam-style otherwise
    (ferrotorch-optim/src/adafactor.rs).  ``beta1`` adds a first moment of the clipped update;
    ``relative_step`` replaces ``lr`` by ``min(cap, 1 / sqrt(step)) * max(eps[1], rms(p))`` with
    ``cap = 1e-2``, or ``1e-6 * step`` under ``warmup_init`` (Shazeer & Stern, section 8)."""

    def __init__(self, params, lr=1e-3, beta2_decay=-0.8, eps=(1e-30, 1e-3), clip_threshold=1.0, weight_decay=0.0,
                 beta1=None, relative_step=False, warmup_init=False):
        if lr is None:
            relative_step = True
        super().__init__(params, dict(lr=lr, beta2_decay=beta2_decay, eps=eps, clip_threshold=clip_threshold,
                                      weight_decay=weight_decay, beta1=beta1, relative_step=relative_step, warmup_init=warmup_init))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float()
                st = self.state[p]
                st["step"] = st.get("step", 0) + 1
                beta2 = 1.0 - st["step"] ** g["beta2_decay"]
                sq = grad * grad + g["eps"][0]
                if grad.dim() >= 2:
                    r = st.setdefault("row", torch.zeros(grad.shape[:-1], device=grad.device))
                    c = st.setdefault("col", torch.zeros(grad.shape[:-2] + grad.shape[-1:], device=grad.device))
                    r.mul_(beta2).add_(sq.mean(-1), alpha=1 - beta2)
                    c.mul_(beta2).add_(sq.mean(-2), alpha=1 - beta2)
                    v = (r / r.mean(-1, keepdim=True)).unsqueeze(-1) * c.unsqueeze(-2)
                else:
                    v = st.setdefault("v", torch.zeros_like(grad))
                    v.mul_(beta2).add_(sq, alpha=1 - beta2)
                u = grad / v.sqrt()
                u = u / max(1.0, float(u.pow(2).mean().sqrt()) / g["clip_threshold"])
                if g["beta1"] is not None:
                    m = st.setdefault("exp_avg", torch.zeros_like(u))
                    m.mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                    u = m
                lr = g["lr"]
                if g["relative_step"]:
                    cap = 1e-6 * st["step"] if g["warmup_init"] else 1e-2
                    lr = min(cap, 1.0 / math.sqrt(st["step"])) * max(g["eps"][1], float(p.float().pow(2).mean().sqrt()))
                if g["weight_decay"]:
                    p.mul_(1 - lr * g["weight_decay"])
                p.add_(u.to(p.dtype), alpha=-lr)
        return loss


class NaturalGradient(Optimizer):
    """Diagonal-Fisher natural gradient (a K-FAC-style preconditioner reduced to its diagonal):
    ``p -= lr * g / (ema(g^2) + damping)``."""

    def __init__(self, params, lr=1e-2, decay=0.95, damping=1e-3):
        super().__init__(params, dict(lr=lr, decay=decay, damping=damping))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                f = self.state[p].setdefault("fisher", torch.zeros_like(p))
                f.mul_(g["decay"]).addcmul_(p.grad, p.grad, value=1 - g["decay"])
                p.addcdiv_(p.grad, f + g["damping"], value=-g["lr"])
        return loss


class Kfac(Optimizer):
    """K-FAC natural gradient for dense layers (Martens & Grosse 2015; ferrotorch-optim/src/natural_gradient.rs:
    92-700).  The Fisher block of a weight ``W [out, in]`` is approximated by ``A (x) G`` with
    ``A = E[a a^T]`` over the layer's inputs and ``G = E[g g^T]`` over the gradients of its outputs, so the
    preconditioned gradient is ``(G + damping I)^-1 grad (A + damping I)^-1``.

    Curvature comes in through :meth:`update_factors` (``weight``, inputs ``[batch, in]``, output
    gradients ``[batch, out]``) or, automatically, from hooks installed by :meth:`watch` on every
    ``nn.Linear`` of a module.  The first update seeds a factor with the batch estimate, later ones blend
    with ``stat_decay``; inverses are recomputed every ``update_freq`` steps.  Parameters without
    factors (biases, anything not registered) get the plain gradient.  ``momentum`` acts on the
    preconditioned gradient; ``weight_decay`` is L2 (added to the gradient before preconditioning);
    ``maximize`` negates the gradient."""

    def __init__(self, params, lr=1e-3, damping=1e-3, momentum=0.9, stat_decay=0.95, update_freq=10, weight_decay=0.0,
                 maximize=False):
        if update_freq < 1:
            raise ValueError("Kfac: update_freq must be >= 1")
        super().__init__(params, dict(lr=lr, damping=damping, momentum=momentum, stat_decay=stat_decay, update_freq=update_freq,
                                      weight_decay=weight_decay, maximize=maximize))
        self._factors: dict = {}          # id(weight) -> {"A", "G", "A_inv", "G_inv"}
        self._steps = 0
        self._hooks: list = []

    def _stat_decay(self) -> float:
        return self.param_groups[0]["stat_decay"]

    @torch.no_grad()
    def update_factors(self, weight: torch.Tensor, input_activation: torch.Tensor, output_gradient: torch.Tensor) -> None:
        a, g = input_activation.detach(), output_gradient.detach()
        if a.dim() != 2 or g.dim() != 2:
            raise ValueError("update_factors expects 2-D tensors, got activation %s and gradient %s" % (tuple(a.shape), tuple(g.shape)))
        if a.shape[0] != g.shape[0] or tuple(weight.shape) != (g.shape[1], a.shape[1]):
            raise ValueError("update_factors: activation %s and gradient %s do not belong to a weight of shape %s"
                             % (tuple(a.shape), tuple(g.shape), tuple(weight.shape)))
        a, g = a.float(), g.float()
        A, G = a.t() @ a / a.shape[0], g.t() @ g / g.shape[0]
        f = self._factors.get(id(weight))
        if f is None:
            self._factors[id(weight)] = {"A": A, "G": G, "A_inv": None, "G_inv": None}
        else:
            d = self._stat_decay()
            f["A"].mul_(d).add_(A, alpha=1 - d)
            f["G"].mul_(d).add_(G, alpha=1 - d)

    def watch(self, module: torch.nn.Module) -> "Kfac":
        """Collect the factors of every ``nn.Linear`` in ``module`` during its forward and backward passes.
        Output gradients are multiplied by the batch size, which undoes the ``1 / batch`` of a mean loss
        (the convention of the K-FAC reference implementations)."""
        def pre(m, args):
            m._kfac_input = args[0].detach().reshape(-1, args[0].shape[-1])

        def back(m, grad_in, grad_out):
            g = grad_out[0].detach().reshape(-1, grad_out[0].shape[-1])
            self.update_factors(m.weight, m._kfac_input, g * g.shape[0])

        for m in module.modules():
            if isinstance(m, torch.nn.Linear):
                self._hooks += [m.register_forward_pre_hook(pre), m.register_full_backward_hook(back)]
        return self

    def unwatch(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def preconditioned(self, weight: torch.Tensor, grad: torch.Tensor, damping: float, refresh: bool = True) -> torch.Tensor:
        """``(G + damping I)^-1 grad (A + damping I)^-1`` for a registered weight (the plain gradient otherwise)."""
        f = self._factors.get(id(weight))
        if f is None or grad.dim() != 2:
            return grad
        if refresh or f["A_inv"] is None:
            eye_a = torch.eye(f["A"].shape[0], device=f["A"].device)
            eye_g = torch.eye(f["G"].shape[0], device=f["G"].device)
            f["A_inv"] = torch.linalg.solve(f["A"] + damping * eye_a, eye_a)
            f["G_inv"] = torch.linalg.solve(f["G"] + damping * eye_g, eye_g)
        return (f["G_inv"] @ grad.float() @ f["A_inv"]).to(grad.dtype)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._steps += 1
        for g in self.param_groups:
            refresh = self._steps == 1 or self._steps % g["update_freq"] == 0
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = -p.grad if g["maximize"] else p.grad
                if g["weight_decay"]:
                    grad = grad.add(p, alpha=g["weight_decay"])
                upd = self.preconditioned(p, grad, g["damping"], refresh)
                if g["momentum"] > 0:
                    st = self.state[p]
                    if "momentum_buf" not in st:
                        st["momentum_buf"] = upd.clone()
                    else:
                        st["momentum_buf"].mul_(g["momentum"]).add_(upd)
                    upd = st["momentum_buf"]
                p.add_(upd, alpha=-g["lr"])
        return loss


class EMA:
    """Exponential moving average of parameters, kept on the parameters' device and updated with
    multi-tensor ops (the reference's EMA callback pulls every parameter to the host each step,
    ferrotorch-train/src/learner.rs:625-637; its ``ExponentialMovingAverage`` is
    ferrotorch-optim/src/ema.rs:93-400, whose method names this class answers to).  Built from a
    module or from a list of parameters; the methods that take ``params`` default to the ones given
    at construction."""

    def __init__(self, module_or_params, decay: float = 0.999):
        if not 0.0 <= decay <= 1.0:
            raise ValueError("EMA decay must be in [0, 1], got %r" % (decay,))
        self.decay = decay
        ps = module_or_params.parameters() if isinstance(module_or_params, torch.nn.Module) else module_or_params
        self.params = [p for p in ps if p.requires_grad]
        self.shadow = [p.detach().clone().float() for p in self.params]
        self._backup = None
        self._n = 0
        self._warmup = False

    def with_foreach(self, params=None) -> "EMA":
        """The shadow tensors already live on the parameters' device and are updated with foreach ops."""
        return self

    def with_decay_warmup(self, use_warmup: bool = True) -> "EMA":
        """Ramp the decay as ``min(decay, (1 + n) / (10 + n))`` over the first updates."""
        self._warmup = bool(use_warmup)
        return self

    def num_updates(self) -> int:
        return self._n

    def effective_decay(self) -> float:
        return min(self.decay, (1.0 + self._n) / (10.0 + self._n)) if self._warmup else self.decay

    def _check(self, params):
        params = self.params if params is None else list(params)
        if len(params) != len(self.shadow):
            raise ValueError("EMA: %d parameters given, %d tracked" % (len(params), len(self.shadow)))
        return params

    @torch.no_grad()
    def update(self, params=None) -> None:
        params = self._check(params)
        self._n += 1
        d = self.effective_decay()
        torch._foreach_mul_(self.shadow, d)
        torch._foreach_add_(self.shadow, [p.detach().float() for p in params], alpha=1 - d)

    @torch.no_grad()
    def apply(self, params=None) -> None:
        """Swap the averaged weights in (the originals are kept for :meth:`restore`)."""
        params = self._check(params)
        self._backup = [p.detach().clone() for p in params]
        for p, s in zip(params, self.shadow):
            p.copy_(s.to(p.dtype))

    apply_shadow = apply

    @torch.no_grad()
    def restore(self, params=None) -> None:
        params = self._check(params)
        if self._backup is not None:
            for p, b in zip(params, self._backup):
                p.copy_(b)
            self._backup = None

    def shadow_params(self) -> list:
        return self.shadow

    def shadow_values(self, index: int) -> torch.Tensor:
        if not 0 <= index < len(self.shadow):
            raise IndexError("EMA.shadow_values: index %d of %d" % (index, len(self.shadow)))
        return self.shadow[index]

    def state_dict(self):
        return {"decay": self.decay, "shadow": self.shadow}

    def load_state_dict(self, sd):
        self.decay = sd["decay"]
        for s, t in zip(self.shadow, sd["shadow"]):
            s.copy_(t)


class GradientAccumulator:
    """Call ``backward`` on ``loss / steps`` and tell when to step the optimizer."""

    def __init__(self, steps: int):
        assert steps >= 1
        self.steps, self._n = steps, 0

    def backward(self, loss: torch.Tensor) -> bool:
        (loss / self.steps).backward()
        self._n += 1
        if self._n == self.steps:
            self._n = 0
            return True
        return False

    # ---- grad_accumulator.rs: the pieces of ``backward`` for loops that call ``backward`` themselves
    def accumulation_steps(self) -> int:
        return self.steps

    def current_step(self) -> int:
        return self._n

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss / self.steps

    def should_step(self) -> bool:
        """Count one micro-batch; true when the optimizer should step now (the counter starts over)."""
        self._n += 1
        if self._n >= self.steps:
            self._n = 0
            return True
        return False

    def reset(self) -> None:
        self._n = 0


class WarmupLR(LambdaLR):
    """Linear warm-up from ``start_factor`` to 1 over ``warmup_steps``."""

    def __init__(self, optimizer, warmup_steps: int, start_factor: float = 0.0):
        super().__init__(optimizer, lambda s: 1.0 if s >= warmup_steps else
                         start_factor + (1 - start_factor) * s / max(1, warmup_steps))


def cosine_warmup_scheduler(optimizer, warmup_steps: int, total_steps: int, min_ratio: float = 0.0) -> LambdaLR:
    def f(s):
        if s < warmup_steps:
            return s / max(1, warmup_steps)
        t = min(1.0, (s - warmup_steps) / max(1, total_steps - warmup_steps))
        return min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t))

    return LambdaLR(optimizer, f)



def diff_sgd_step(params, grads, lr: float):
    """One SGD step as a differentiable function of the parameters, the gradients and ``lr``:
    returns new tensors instead of updating in place, so an outer loss can be differentiated
    through the update (meta-learning; ferrotorch-optim/src/differentiable.rs)."""
    return [p - lr * g for p, g in zip(params, grads)]


def diff_sgd_momentum_step(params, grads, bufs, lr: float, momentum: float = 0.9):
    """The same with momentum: ``buf' = momentum * buf + g``, ``p' = p - lr * buf'``; returns
    ``(new_params, new_bufs)``."""
    new_bufs = [momentum * b + g for b, g in zip(bufs, grads)]
    return [p - lr * b for p, b in zip(params, new_bufs)], new_bufs



class AveragedModel(torch.optim.swa_utils.AveragedModel):
    """torch's averaged model (a deep copy whose parameters are the running average) with the
    reference's entry points on top (ferrotorch-optim/src/swa.rs:133-400): built ``from_module`` with an
    :class:`~ferrotorch_b200.optim.configs.AveragingStrategy`, updated from a module or from a parameter
    list, and written back into a module or a parameter list."""

    def __init__(self, model, device=None, avg_fn=None, multi_avg_fn=None, use_buffers=False, strategy=None, decay: float = 0.999):
        from .configs import AveragingStrategy

        if isinstance(strategy, tuple):
            strategy, decay = strategy
        if strategy is not None and multi_avg_fn is None and avg_fn is None:
            if strategy is AveragingStrategy.Ema and not 0.0 <= decay <= 1.0:
                raise ValueError("AveragedModel: EMA decay must be in [0, 1], got %r" % (decay,))
            multi_avg_fn = strategy.avg_fn(decay)
        super().__init__(model, device, avg_fn, multi_avg_fn, use_buffers)
        self._strategy = strategy if strategy is not None else AveragingStrategy.Swa

    @classmethod
    def from_module(cls, module, strategy=None, decay: float = 0.999) -> "AveragedModel":
        return cls(module, strategy=strategy, decay=decay)

    def strategy(self):
        return self._strategy

    def with_foreach(self, params=None) -> "AveragedModel":
        return self                      # the average is updated with multi-tensor ops already

    def update_parameters_from_module(self, module) -> None:
        self.update_parameters(module)

    def averaged_params(self) -> list:
        return [p.detach() for p in self.module.parameters()]

    def averaged_values(self, index: int) -> torch.Tensor:
        ps = self.averaged_params()
        if not 0 <= index < len(ps):
            raise IndexError("AveragedModel.averaged_values: index %d of %d" % (index, len(ps)))
        return ps[index]

    @torch.no_grad()
    def apply_to(self, params) -> None:
        """Copy the averaged values into ``params`` (same order as the module's parameters)."""
        params, avg = list(params), self.averaged_params()
        if len(params) != len(avg):
            raise ValueError("AveragedModel.apply_to: %d parameters given, %d averaged" % (len(params), len(avg)))
        for p, a in zip(params, avg):
            p.copy_(a.to(p.dtype))

    def apply_to_module(self, module) -> None:
        self.apply_to(module.parameters())


# --------------------------------------------------------------------------- helpers of the multi-tensor ("foreach") steps (foreach_utils.rs)
def elemwise_max(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``max(a, b)`` element by element."""
    return torch.maximum(a, b)


def scalar_on(value, device, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """A 0-d tensor holding a hyper-parameter on ``device``, so that a step never reads it from the host."""
    return torch.tensor(value, dtype=dtype, device=device)


def f64_scalar_on(value: float, device, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return scalar_on(float(value), device, dtype)
