"""Optimizers and helpers torch does not ship (reference: ferrotorch-optim/src/{muon,adafactor,
natural_gradient,ema,swa}.rs, grad_accumulator, scheduler/warmup.rs)."""
from __future__ import annotations

import math

import torch
from torch.optim import Optimizer
from torch.optim.lr_scheduler import LambdaLR


def _newton_schulz(g: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Quintic Newton-Schulz iteration that orthogonalises a matrix (Muon)."""
    a, b, c = 3.4445, -4.7750, 2.0315
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
    """Momentum + orthogonalised update for 2-D parameters; other shapes fall back to SGD-momentum."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                buf = st.setdefault("momentum_buffer", torch.zeros_like(p))
                buf.mul_(g["momentum"]).add_(p.grad)
                upd = p.grad.add(buf, alpha=g["momentum"]) if g["nesterov"] else buf
                if p.dim() == 2:
                    upd = _newton_schulz(upd, g["ns_steps"]) * max(1.0, p.shape[0] / p.shape[1]) ** 0.5
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(upd, alpha=-g["lr"])
        return loss


class Adafactor(Optimizer):
    """Factored second moments for matrices (row / column statistics), Adam-style otherwise."""

    def __init__(self, params, lr=1e-3, beta2_decay=-0.8, eps=(1e-30, 1e-3), clip_threshold=1.0, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, beta2_decay=beta2_decay, eps=eps, clip_threshold=clip_threshold,
                                      weight_decay=weight_decay))

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
                if g["weight_decay"]:
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(u.to(p.dtype), alpha=-g["lr"])
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
