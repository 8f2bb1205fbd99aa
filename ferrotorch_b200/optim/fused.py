"""torch.optim-style optimizers on the flat-arena kernels.

``FusedAdamW`` / ``FusedSGD`` keep the usual ``Optimizer`` surface of the reference
(``step, zero_grad, param_groups, add_param_group, state_dict, load_state_dict``,
ferrotorch-optim/src/optimizer.rs:93-143) but move each parameter group into one contiguous
fp32 arena (plus a gradient staging arena), so a step is: one gather of ``.grad`` into the
arena (``torch._foreach_copy_``) and one ``ft_adamw_flat`` / ``ft_sgd_flat`` launch per group.
bf16 parameters get fp32 master weights in the arena and are written back by the same kernel.
On CPU the same update rules run through :mod:`ferrotorch_b200.ops.reference`.
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from .. import _native
from ..ops import reference as ref


class _FlatGroup:
    def __init__(self, params):
        self.params = [p for p in params]
        self.device = self.params[0].device
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.numel() + 63) // 64 * 64
        self.numel = off
        self.master = torch.zeros(off, device=self.device, dtype=torch.float32)
        self.grad = torch.zeros(off, device=self.device, dtype=torch.float32)
        for p, o in zip(self.params, self.offsets):
            self.master[o:o + p.numel()].copy_(p.detach().reshape(-1))
        self.views_g = [self.grad[o:o + p.numel()].view(p.shape) for p, o in zip(self.params, self.offsets)]
        self.views_p = [self.master[o:o + p.numel()].view(p.shape) for p, o in zip(self.params, self.offsets)]
        self.state: dict[str, torch.Tensor] = {}

    def buf(self, name: str) -> torch.Tensor:
        if name not in self.state:
            self.state[name] = torch.zeros_like(self.master)
        return self.state[name]

    def gather_grads(self) -> bool:
        self.grad.zero_()
        have = [(v, p.grad) for v, p in zip(self.views_g, self.params) if p.grad is not None]
        if not have:
            return False
        torch._foreach_copy_([v for v, _ in have], [g for _, g in have])
        return True

    def scatter_params(self) -> None:
        with torch.no_grad():
            torch._foreach_copy_([p.data for p in self.params], self.views_p)


class _FusedBase(Optimizer):
    def _flat(self, group) -> _FlatGroup:
        fg = group.get("_flat")
        if fg is None or len(fg.params) != len(group["params"]):
            fg = _FlatGroup(group["params"])
            group["_flat"] = fg
        return fg

    def state_dict(self):
        groups = []
        for g in self.param_groups:
            fg = g.get("_flat")
            groups.append({**{k: v for k, v in g.items() if k not in ("params", "_flat")},
                           "flat_state": {k: v.clone() for k, v in (fg.state if fg else {}).items()},
                           "master": fg.master.clone() if fg else None})
        return {"param_groups": groups}

    def load_state_dict(self, sd):
        for g, s in zip(self.param_groups, sd["param_groups"]):
            for k, v in s.items():
                if k not in ("flat_state", "master"):
                    g[k] = v
            fg = self._flat(g)
            if s.get("master") is not None:
                fg.master.copy_(s["master"])
                fg.scatter_params()
            for k, v in s.get("flat_state", {}).items():
                fg.buf(k).copy_(v)


class FusedAdamW(_FusedBase):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, adam_l2: bool = False,
                 maximize: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, adam_l2=adam_l2,
                                      maximize=maximize, step=0))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            fg = self._flat(g)
            if not fg.gather_grads():
                continue
            if g["maximize"]:
                fg.grad.neg_()
            g["step"] += 1
            m, v = fg.buf("exp_avg"), fg.buf("exp_avg_sq")
            if fg.device.type == "cuda":
                rc = _native.kernels().ft_adamw_flat(
                    fg.master.data_ptr(), m.data_ptr(), v.data_ptr(), fg.grad.data_ptr(), None, fg.numel, 1, None,
                    g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"], g["step"], int(g["adam_l2"]),
                    fg.device.index or 0, torch.cuda.current_stream().cuda_stream)
                _native.check(rc, "ft_adamw_flat")
            else:
                ref.adamw_step(fg.master, fg.grad, m, v, lr=g["lr"], beta1=g["betas"][0], beta2=g["betas"][1],
                               eps=g["eps"], weight_decay=g["weight_decay"], step=g["step"], adam_l2=g["adam_l2"])
            fg.scatter_params()
        return loss


class FusedSGD(_FusedBase):
    def __init__(self, params, lr=1e-3, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
                 maximize: bool = False):
        if nesterov and (momentum <= 0 or dampening != 0):
            raise ValueError("Nesterov momentum requires a momentum and zero dampening")
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov, maximize=maximize, step=0))

    def set_momentum(self, momentum: float) -> None:
        for g in self.param_groups:
            g["momentum"] = momentum

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            fg = self._flat(g)
            if not fg.gather_grads():
                continue
            if g["maximize"]:
                fg.grad.neg_()
            g["step"] += 1
            buf = fg.buf("momentum_buffer") if g["momentum"] != 0 else None
            if fg.device.type == "cuda":
                rc = _native.kernels().ft_sgd_flat(
                    fg.master.data_ptr(), buf.data_ptr() if buf is not None else None, fg.grad.data_ptr(), None,
                    fg.numel, 1, None, g["lr"], g["momentum"], g["dampening"], g["weight_decay"], int(g["nesterov"]),
                    int(g["step"] == 1), fg.device.index or 0, torch.cuda.current_stream().cuda_stream)
                _native.check(rc, "ft_sgd_flat")
            else:
                ref.sgd_step(fg.master, fg.grad, buf, lr=g["lr"], momentum=g["momentum"], dampening=g["dampening"],
                             weight_decay=g["weight_decay"], nesterov=g["nesterov"], first_step=g["step"] == 1)
            fg.scatter_params()
        return loss
