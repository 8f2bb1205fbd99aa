"""Bucketed data-parallel gradient averaging over any :class:`~.backend.Group`.

This is the reference's ``DDP`` (ferrotorch-distributed/src/ddp.rs:55-311) restated: parameters
are walked in reverse order into buckets of at most 25 MB (ddp.rs:35, 230-258); after backward
each bucket is flattened (missing gradients count as zeros), all-reduced with Mean and sliced
back into ``.grad`` (ddp.rs:265-311); ``broadcast_parameters`` copies rank ``root``'s weights
to every rank (ddp.rs:176-186).  Used for CPU ranks (gloo / native TCP / simulated) and as the
generic path for modules that do not go through the flat-arena trainer; GPU training uses
:class:`ferrotorch_b200.parallel.ddp.FusedDDP`.
"""
from __future__ import annotations


import torch
from torch import nn

from .backend import Group

DEFAULT_BUCKET_SIZE_BYTES = 25 * 1024 * 1024


def compute_buckets(params, bucket_size_bytes: int = DEFAULT_BUCKET_SIZE_BYTES) -> list[list[int]]:
    """Indices of ``params`` grouped into buckets, walking the list in reverse."""
    buckets, cur, cur_bytes = [], [], 0
    for i in reversed(range(len(params))):
        nbytes = params[i].numel() * params[i].element_size()
        if cur and cur_bytes + nbytes > bucket_size_bytes:
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(i)
        cur_bytes += nbytes
    if cur:
        buckets.append(cur)
    return buckets


class DDP(nn.Module):
    """``overlap=True`` starts a bucket's all-reduce as soon as the backward pass has produced its
    last gradient (a hook per parameter counts them down) on one worker thread, in the order the
    buckets complete, which is the same on every rank because the model and the autograd order
    are; ``sync_gradients`` then only waits for what is still in flight and handles buckets that
    never completed (parameters without a gradient).  Results are identical to the sequential
    form: the same buckets, the same flattening, the same reduction."""

    def __init__(self, module: nn.Module, group: Group, bucket_size_bytes: int = DEFAULT_BUCKET_SIZE_BYTES,
                 overlap: bool = False):
        super().__init__()
        self.module, self.group = module, group
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.buckets = compute_buckets(self.params, bucket_size_bytes)
        self.overlap, self._sync_enabled = overlap, True
        if overlap:
            from .backend import _Lane

            self._lane = _Lane()
            self._bucket_of = {i: b for b, idxs in enumerate(self.buckets) for i in idxs}
            self._left = [len(idxs) for idxs in self.buckets]
            self._ops: dict[int, object] = {}
            for i, p in enumerate(self.params):
                p.register_post_accumulate_grad_hook(lambda _p, i=i: self._grad_ready(i))

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    def no_sync(self):
        """Context manager: backward passes inside it only accumulate (gradient accumulation)."""
        ddp = self

        class _NoSync:
            def __enter__(self):
                self.prev, ddp._sync_enabled = ddp._sync_enabled, False

            def __exit__(self, *exc):
                ddp._sync_enabled = self.prev
                return False

        return _NoSync()

    def _grad_ready(self, i: int) -> None:
        if not self._sync_enabled:
            return
        b = self._bucket_of[i]
        self._left[b] -= 1
        if self._left[b] == 0:
            self._ops[b] = self._lane.post(self._sync_bucket, self.buckets[b])

    def _sync_bucket(self, idxs) -> None:
        ps = [self.params[i] for i in idxs]
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in ps])
        self.group.all_reduce(flat, "mean")
        off = 0
        for p in ps:
            n = p.numel()
            g = flat[off:off + n].view_as(p)
            if p.grad is None:
                p.grad = g.clone()
            else:
                p.grad.copy_(g)
            off += n

    def sync_gradients(self) -> None:
        """Average gradients across ranks, bucket by bucket (call after ``backward``)."""
        if not self.overlap:
            for b in self.buckets:
                self._sync_bucket(b)
            return
        # every rank posts the buckets that did not complete in the same (index) order, after the
        # ones that did; then everything is awaited
        for b in range(len(self.buckets)):
            if b not in self._ops:
                self._ops[b] = self._lane.post(self._sync_bucket, self.buckets[b])
        for b in sorted(self._ops):
            self._ops[b].wait()
        self._ops = {}
        self._left = [len(idxs) for idxs in self.buckets]

    def broadcast_parameters(self, root: int = 0) -> None:
        with torch.no_grad():
            for p in self.module.parameters():
                self.group.broadcast(p.data, root)
            for b in self.module.buffers():
                self.group.broadcast(b.data, root)
