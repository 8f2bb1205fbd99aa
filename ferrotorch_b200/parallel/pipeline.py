"""Pipeline parallelism: micro-batched GPipe and 1F1B over point-to-point sends.

The reference's ``Pipeline`` (ferrotorch-distributed/src/pipeline.rs:50-367) has both schedule
names but runs the micro-batches sequentially per stage and sends a zero tensor upstream as the
input gradient (pipeline.rs:223-233).  Here each stage holds its sub-module, activations travel
with a small shape header like the reference's (pipeline.rs:266-346), and the backward sends the
**real** input gradient upstream.  ``schedule="gpipe"`` runs all forwards then all backwards;
``"1f1b"`` interleaves them after a warm-up of ``n_stages - stage - 1`` forwards, which bounds
the number of live activations.  Works over any :class:`~.backend.Group` (NCCL p2p on GPUs).
"""
from __future__ import annotations

import torch
from torch import nn

from .backend import Group


def _send(g: Group, t: torch.Tensor, dst: int) -> None:
    hdr = torch.zeros(8, dtype=torch.int64)
    hdr[0] = t.dim()
    hdr[1:1 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
    g.send(hdr.to(t.device) if t.is_cuda else hdr, dst)
    g.send(t.contiguous(), dst)


def _recv(g: Group, src: int, device, dtype) -> torch.Tensor:
    hdr = torch.zeros(8, dtype=torch.int64, device=device)
    g.recv(hdr, src)
    h = hdr.cpu()
    shape = [int(x) for x in h[1:1 + int(h[0])]]
    t = torch.empty(shape, device=device, dtype=dtype)
    g.recv(t, src)
    return t


class Pipeline:
    def __init__(self, stage_module: nn.Module, group: Group, n_micro: int, schedule: str = "1f1b",
                 loss_fn=None, dtype=torch.float32, device="cpu"):
        assert schedule in ("gpipe", "1f1b")
        self.m, self.g, self.n_micro, self.schedule = stage_module, group, n_micro, schedule
        self.stage, self.n_stages = group.rank, group.world_size
        self.loss_fn, self.dtype, self.device = loss_fn, dtype, torch.device(device)
        self.first, self.last = self.stage == 0, self.stage == group.world_size - 1

    def _fwd(self, x_mb):
        if self.first:
            inp = x_mb
        else:
            inp = _recv(self.g, self.stage - 1, self.device, self.dtype).requires_grad_()
        out = self.m(inp)
        if not self.last:
            _send(self.g, out.detach(), self.stage + 1)
        return inp, out

    def _bwd(self, inp, out, y_mb):
        if self.last:
            loss = self.loss_fn(out, y_mb) / self.n_micro
            loss.backward()
            val = loss.detach()
        else:
            grad = _recv(self.g, self.stage + 1, self.device, self.dtype)
            out.backward(grad)
            val = None
        if not self.first:
            _send(self.g, inp.grad, self.stage - 1)
        return val

    def train_step(self, x: torch.Tensor | None, y: torch.Tensor | None):
        """One forward/backward over ``n_micro`` micro-batches.  ``x`` is used on the first stage,
        ``y`` on the last; returns the mean loss on the last stage, ``None`` elsewhere."""
        xs = x.chunk(self.n_micro) if self.first else [None] * self.n_micro
        ys = y.chunk(self.n_micro) if self.last else [None] * self.n_micro
        live, total = [], None
        warm = self.n_micro if self.schedule == "gpipe" else min(self.n_micro, self.n_stages - self.stage - 1)
        f = b = 0
        for _ in range(warm):
            live.append(self._fwd(xs[f]))
            f += 1
        while b < self.n_micro:
            if f < self.n_micro:
                live.append(self._fwd(xs[f]))
                f += 1
            inp, out = live.pop(0)
            v = self._bwd(inp, out, ys[b])
            b += 1
            if v is not None:
                total = v if total is None else total + v
        return total
