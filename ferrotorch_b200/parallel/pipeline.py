"""Pipeline parallelism: micro-batched GPipe and 1F1B over non-blocking point-to-point transfers.

The reference's ``Pipeline`` (ferrotorch-distributed/src/pipeline.rs:50-367) has both schedule
names but runs the micro-batches sequentially per stage and sends a zero tensor upstream as the
input gradient (pipeline.rs:223-233).  Here each stage holds its sub-module and the backward sends
the **real** input gradient upstream.  ``schedule="gpipe"`` runs all forwards then all backwards;
``"1f1b"`` interleaves them after a warm-up of ``n_stages - stage - 1`` forwards, which bounds
the number of live activations.

Transfers overlap compute: every activation and every gradient leaves through ``Group.isend``
(the stage goes on with its next micro-batch while the bytes travel; NCCL p2p on its own stream
for a ``TorchGroup``), and the receive of the *next* micro-batch is posted before the current one
is computed.  Shapes travel once per step: the first micro-batch carries a small header like the
reference's (pipeline.rs:266-346), later micro-batches of the step reuse it (``x`` must split into
equal micro-batches); the gradient of an activation has the activation's shape and needs none.
Works over any :class:`~.backend.Group`.
"""
from __future__ import annotations

import torch
from torch import nn

from .backend import Group, PendingOp


class Pipeline:
    def __init__(self, stage_module: nn.Module, group: Group, n_micro: int, schedule: str = "1f1b",
                 loss_fn=None, dtype=torch.float32, device="cpu"):
        assert schedule in ("gpipe", "1f1b")
        self.m, self.g, self.n_micro, self.schedule = stage_module, group, n_micro, schedule
        self.stage, self.n_stages = group.rank, group.world_size
        self.loss_fn, self.dtype, self.device = loss_fn, dtype, torch.device(device)
        self.first, self.last = self.stage == 0, self.stage == group.world_size - 1
        self.stats = {"posted_sends": 0, "prefetched_recvs": 0}

    # ------------------------------------------------------------------ transfers
    def _post_send(self, t: torch.Tensor, dst: int, with_header: bool) -> None:
        if with_header:
            hdr = torch.zeros(8, dtype=torch.int64)
            hdr[0] = t.dim()
            hdr[1:1 + t.dim()] = torch.tensor(list(t.shape), dtype=torch.int64)
            self._sends.append(self.g.isend(hdr.to(t.device) if t.is_cuda else hdr, dst))
        self._sends.append(self.g.isend(t.contiguous(), dst))
        self.stats["posted_sends"] += 1

    def _post_recv(self, shape, src: int) -> tuple[torch.Tensor, PendingOp]:
        t = torch.empty(shape, device=self.device, dtype=self.dtype)
        return t, self.g.irecv(t, src)

    def _recv_first_input(self) -> torch.Tensor:
        """First micro-batch of a step: header, then payload (both in order on the receive lane)."""
        hdr = torch.zeros(8, dtype=torch.int64, device=self.device)
        self.g.irecv(hdr, self.stage - 1).wait()
        h = hdr.cpu()
        self._in_shape = [int(x) for x in h[1:1 + int(h[0])]]
        t, op = self._post_recv(self._in_shape, self.stage - 1)
        op.wait()
        return t

    # ------------------------------------------------------------------ one micro-batch
    def _fwd(self, i: int, x_mb):
        if self.first:
            inp = x_mb
        else:
            if i == 0:
                inp = self._recv_first_input()
            else:
                inp, op = self._next_in
                op.wait()
            if i + 1 < self.n_micro:           # the next input travels while this one is computed
                self._next_in = self._post_recv(self._in_shape, self.stage - 1)
                self.stats["prefetched_recvs"] += 1
            inp.requires_grad_()
        out = self.m(inp)
        if not self.last:
            self._post_send(out.detach(), self.stage + 1, with_header=(i == 0))
        return inp, out

    def _bwd(self, j: int, inp, out, y_mb, next_out):
        if self.last:
            loss = self.loss_fn(out, y_mb) / self.n_micro
            loss.backward()
            val = loss.detach()
        else:
            if self._next_grad is None:
                self._next_grad = self._post_recv(out.shape, self.stage + 1)
            grad, op = self._next_grad
            op.wait()
            # the gradient of the next micro-batch in line travels during this backward
            self._next_grad = self._post_recv(next_out.shape, self.stage + 1) if next_out is not None else None
            if next_out is not None:
                self.stats["prefetched_recvs"] += 1
            out.backward(grad)
            val = None
        if not self.first:
            self._post_send(inp.grad, self.stage - 1, with_header=False)
        return val

    def train_step(self, x: torch.Tensor | None, y: torch.Tensor | None):
        """One forward/backward over ``n_micro`` micro-batches.  ``x`` is used on the first stage,
        ``y`` on the last; returns the mean loss on the last stage, ``None`` elsewhere."""
        if self.first and x.shape[0] % self.n_micro:
            raise ValueError("batch of %d does not split into %d equal micro-batches" % (x.shape[0], self.n_micro))
        xs = x.chunk(self.n_micro) if self.first else [None] * self.n_micro
        ys = y.chunk(self.n_micro) if self.last else [None] * self.n_micro
        self._sends: list[PendingOp] = []
        self._next_in = self._next_grad = None
        live, total = [], None
        warm = self.n_micro if self.schedule == "gpipe" else min(self.n_micro, self.n_stages - self.stage - 1)
        f = b = 0
        for _ in range(warm):
            live.append(self._fwd(f, xs[f]))
            f += 1
        while b < self.n_micro:
            if f < self.n_micro:
                live.append(self._fwd(f, xs[f]))
                f += 1
            inp, out = live.pop(0)
            # the micro-batch whose gradient arrives after this one: the next live one, else the
            # next to be forwarded (same shape as every other micro-batch of the step)
            if b + 1 < self.n_micro:
                next_out = live[0][1] if live else out
            else:
                next_out = None
            v = self._bwd(b, inp, out, ys[b], next_out)
            b += 1
            if v is not None:
                total = v if total is None else total + v
        for op in self._sends:               # buffers stay alive until their transfer has completed
            op.wait()
        self._sends = []
        return total
