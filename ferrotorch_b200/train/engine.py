"""Flat-arena mixed-precision training engine.

All parameters of a model live in one bf16 arena, their gradients in a second arena of the
same layout, and the optimizer state (fp32 master weights and moments) in three fp32 arenas.
The weight-gradient GEMMs accumulate straight into the gradient arena (``param.main_grad``),
the global gradient norm and the AdamW / SGD update each run as a single launch over the
arena, and nothing in a step synchronises with the host.

The reference's training loop (ferrotorch-train/src/learner.rs:554-619) runs
``forward -> loss.item() -> backward -> clip_grad_norm_ -> optimizer.step -> zero_grad`` with
a per-parameter op chain in the optimizer (ferrotorch-optim/src/adamw.rs:239-384); data-parallel
users then call ``ddp.sync_gradients()`` after backward (ferrotorch-distributed/src/ddp.rs:117).
Here the same sequence is: memset the gradient arena, micro-batches of forward/backward,
(data parallel: bucketed fused all-reduce + update, see ``parallel/ddp.py``), one norm launch
pair, one update launch per parameter group.
"""
from __future__ import annotations

from typing import Callable

import torch
from torch import nn

from .. import _native


def _pad(n: int, mult: int = 64) -> int:
    return (n + mult - 1) // mult * mult


class FlatArena:
    """Parameters of ``module`` re-homed into flat buffers.

    ``groups`` maps a group name to the parameters in it; each group is a contiguous range
    of the arena (so a group = one optimizer launch).  Every parameter starts on a 128-byte
    boundary."""

    def __init__(self, module: nn.Module, group_of: Callable[[str, nn.Parameter], str] | None = None,
                 grad_dtype: torch.dtype | None = None, allocator: Callable | None = None):
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        seen, uniq = set(), []
        for n, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        group_of = group_of or (lambda name, p: "decay" if p.dim() >= 2 else "no_decay")
        order: dict[str, list] = {}
        for n, p in uniq:
            order.setdefault(group_of(n, p), []).append((n, p))
        self.device = uniq[0][1].device
        self.dtype = uniq[0][1].dtype
        self.ranges: dict[str, tuple[int, int]] = {}
        self.slots: list[tuple[str, nn.Parameter, int, int]] = []
        off = 0
        for g, items in order.items():
            start = off
            for n, p in items:
                self.slots.append((n, p, off, p.numel()))
                off += _pad(p.numel())
            self.ranges[g] = (start, off)
        self.numel = off
        alloc = allocator or (lambda n, dt: torch.zeros(n, device=self.device, dtype=dt))
        grad_dtype = grad_dtype or self.dtype
        self.params = alloc(self.numel, self.dtype)
        self.grads = alloc(self.numel, grad_dtype)
        with torch.no_grad():
            for n, p, o, k in self.slots:
                view = self.params[o:o + k].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = self.grads[o:o + k].view(p.shape)
                p.arena_offset = o

    def zero_grad(self) -> None:
        self.grads.zero_()

    def fold_autograd_grads(self) -> None:
        """Add ``.grad`` produced by ops that do not write ``main_grad`` themselves."""
        for _, p, _, _ in self.slots:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None


class FlatTrainer:
    """Forward / backward / fused-update driver over a :class:`FlatArena`.

    ``optimizer``: "adamw" (decoupled decay, ferrotorch-optim/src/adamw.rs:296-334), "adam"
    (L2 decay) or "sgd" (momentum / nesterov / dampening, sgd.rs:224-330).
    ``max_grad_norm``: global L2 clip (ferrotorch-nn/src/utils.rs:148-240), applied inside the
    update kernel from a device-side coefficient.
    ``micro_batches``: the batch given to :meth:`step` is split into this many sequential
    forward/backward passes whose gradients accumulate in the arena.
    ``grad_dtype``: dtype of the gradient arena; default fp32 when ``micro_batches > 2`` (the
    weight-gradient GEMMs then add their tiles in fp32), else the parameter dtype.
    """

    def __init__(self, model: nn.Module, *, optimizer: str = "adamw", lr: float = 1e-3,
                 betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 momentum: float = 0.0, dampening: float = 0.0, nesterov: bool = False,
                 max_grad_norm: float | None = None, micro_batches: int = 1,
                 no_decay: Callable[[str, nn.Parameter], bool] | None = None,
                 loss_fn: Callable | None = None, ddp=None, allocator: Callable | None = None,
                 grad_dtype: torch.dtype | None = None):
        self.model = model
        self.kind = optimizer
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.momentum, self.dampening, self.nesterov = momentum, dampening, nesterov
        self.max_grad_norm = max_grad_norm
        self.micro_batches = micro_batches
        self.loss_fn = loss_fn
        nd = no_decay or (lambda name, p: p.dim() < 2)
        if grad_dtype is None:
            # every micro-batch adds into the arena; beyond two additions a bf16 arena would round
            # away most of a late micro-batch's contribution, so the sum is kept in fp32
            first = next(p for p in model.parameters() if p.requires_grad)
            grad_dtype = torch.float32 if micro_batches > 2 else first.dtype
        self.arena = FlatArena(model, lambda n, p: "no_decay" if nd(n, p) else "decay", allocator=allocator,
                               grad_dtype=grad_dtype)
        a = self.arena
        self.master = a.params.float()
        self.exp_avg = torch.zeros_like(self.master) if optimizer != "sgd" or momentum != 0.0 else None
        self.exp_avg_sq = torch.zeros_like(self.master) if optimizer in ("adamw", "adam") else None
        self.step_count = 0
        self.native = a.device.type == "cuda"
        self._norm_out = torch.zeros(4, device=a.device, dtype=torch.float32)
        if self.native:
            lib = _native.kernels()
            self._norm_partial = torch.empty(lib.ft_grad_norm_scratch(a.device.index or 0), device=a.device,
                                             dtype=torch.float32)
        self.ddp = ddp
        # called after the last backward and before the update (tensor parallelism sums the
        # gradients of replicated parameters here)
        self.pre_update: Callable[[], None] | None = None
        # model-parallel group whose ranks hold different shards of the "decay" parameters and
        # full copies of the "no_decay" ones: the clipping norm is then taken over the whole model
        self.model_parallel_group = None
        if ddp is not None:
            ddp.attach(self)

    # ------------------------------------------------------------------ one training step
    def forward_backward(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Accumulate gradients of the mean loss over ``inputs`` (split into micro-batches);
        returns the mean loss as a 0-dim device tensor."""
        mb = self.micro_batches
        B = inputs.shape[0]
        assert B % mb == 0, "batch %d not divisible into %d micro-batches" % (B, mb)
        per = B // mb
        total = None
        denom = targets.numel()
        for i in range(mb):
            x, y = inputs[i * per:(i + 1) * per], targets[i * per:(i + 1) * per]
            if self.ddp is not None:
                self.ddp.note_micro_batch(i, mb)
            if self.loss_fn is not None:
                loss = self.loss_fn(self.model, x, y) / mb
            else:
                loss = self.model(x, labels=y, loss_denominator=denom)
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        self.arena.fold_autograd_grads()
        return total

    def step(self, inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        self.arena.zero_grad()
        if self.ddp is not None:
            self.ddp.begin_step()
        loss = self.forward_backward(inputs, targets)
        self.optimizer_step()
        return loss

    # ------------------------------------------------------------------ update
    def grad_norm(self) -> torch.Tensor:
        """Launch the norm kernels; returns the device tensor ``[norm, clip_coef, norm^2]``."""
        a = self.arena
        if self.native:
            lib = _native.kernels()
            rc = lib.ft_grad_norm(a.grads.data_ptr(), a.numel, int(a.grads.dtype == torch.float32),
                                  self._norm_partial.data_ptr(), None, float(self.max_grad_norm or 0.0),
                                  self._norm_out.data_ptr(), a.device.index or 0,
                                  torch.cuda.current_stream().cuda_stream)
            _native.check(rc, "ft_grad_norm")
        else:
            n = a.grads.float().norm()
            self._norm_out[0] = n
            self._norm_out[1] = torch.clamp(self.max_grad_norm / (n + 1e-6), max=1.0) if self.max_grad_norm else 1.0
            self._norm_out[2] = n * n
        if self.model_parallel_group is not None:
            import torch.distributed as dist

            s, e = a.ranges.get("no_decay", (0, 0))
            rep = a.grads[s:e].float().pow(2).sum()
            sharded = self._norm_out[2] - rep
            dist.all_reduce(sharded, group=self.model_parallel_group)
            total = (sharded + rep).clamp_min(0)
            n = total.sqrt()
            self._norm_out[0] = n
            self._norm_out[1] = torch.clamp(self.max_grad_norm / (n + 1e-6), max=1.0) if self.max_grad_norm else 1.0
            self._norm_out[2] = total
        return self._norm_out

    def optimizer_step(self) -> None:
        if self.pre_update is not None:
            self.pre_update()
        if self.ddp is not None and self.ddp.fused_update:
            self.step_count += 1
            self.ddp.finish_step(self)
            return
        if self.ddp is not None:
            self.ddp.finish_step(self)
        self.step_count += 1
        scale_ptr = None
        if self.max_grad_norm:
            scale_ptr = self.grad_norm()[1:]
        self.apply_update(0, self.arena.numel, scale_ptr)

    def apply_update(self, lo: int, hi: int, scale: torch.Tensor | None, grads: torch.Tensor | None = None) -> None:
        """Update arena elements ``[lo, hi)`` (clipped per group so weight decay is right)."""
        a = self.arena
        grads = a.grads if grads is None else grads
        for g, (s, e) in a.ranges.items():
            s2, e2 = max(s, lo), min(e, hi)
            if s2 >= e2:
                continue
            wd = self.weight_decay if g == "decay" else 0.0
            self._update_range(s2, e2, wd, scale, grads)

    def _update_range(self, s: int, e: int, wd: float, scale, grads) -> None:
        a = self.arena
        n = e - s
        if self.native:
            lib = _native.kernels()
            dev, stream = a.device.index or 0, torch.cuda.current_stream().cuda_stream
            gf32 = int(grads.dtype == torch.float32)
            gptr = grads.data_ptr() + s * grads.element_size()
            plp = a.params.data_ptr() + s * a.params.element_size() if a.params.dtype == torch.bfloat16 else None
            sp = scale.data_ptr() if scale is not None else None
            if self.kind in ("adamw", "adam"):
                rc = lib.ft_adamw_flat(self.master.data_ptr() + 4 * s, self.exp_avg.data_ptr() + 4 * s,
                                       self.exp_avg_sq.data_ptr() + 4 * s, gptr, plp, n, gf32, sp, self.lr,
                                       self.betas[0], self.betas[1], self.eps, wd, self.step_count,
                                       int(self.kind == "adam"), dev, stream)
                _native.check(rc, "ft_adamw_flat")
            else:
                rc = lib.ft_sgd_flat(self.master.data_ptr() + 4 * s,
                                     self.exp_avg.data_ptr() + 4 * s if self.exp_avg is not None else None,
                                     gptr, plp, n, gf32, sp, self.lr, self.momentum, self.dampening, wd,
                                     int(self.nesterov), int(self.step_count == 1), dev, stream)
                _native.check(rc, "ft_sgd_flat")
            if a.params.dtype != torch.bfloat16:
                a.params[s:e].copy_(self.master[s:e])
            return
        # CPU path: the PyTorch restatement of the same update rules
        from ..ops import reference as ref

        g = grads[s:e].float()
        if scale is not None:
            g = g * scale[0]
        p = self.master[s:e]
        if self.kind in ("adamw", "adam"):
            ref.adamw_step(p, g, self.exp_avg[s:e], self.exp_avg_sq[s:e], lr=self.lr, beta1=self.betas[0],
                           beta2=self.betas[1], eps=self.eps, weight_decay=wd, step=self.step_count,
                           adam_l2=self.kind == "adam")
        else:
            ref.sgd_step(p, g, self.exp_avg[s:e] if self.exp_avg is not None else None, lr=self.lr,
                         momentum=self.momentum, dampening=self.dampening, weight_decay=wd,
                         nesterov=self.nesterov, first_step=self.step_count == 1)
        a.params[s:e].copy_(p.to(a.params.dtype))

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "lr": self.lr,
                "layout": [(n, o, k) for n, _, o, k in self.arena.slots]}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.lr = float(sd.get("lr", self.lr))
        self.master.copy_(sd["master"])
        for name in ("exp_avg", "exp_avg_sq"):
            if getattr(self, name) is not None and sd.get(name) is not None:
                getattr(self, name).copy_(sd[name])
        self.arena.params.copy_(self.master.to(self.arena.params.dtype))

    def set_lr(self, lr: float) -> None:
        self.lr = lr
