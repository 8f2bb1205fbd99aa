"""Fully-sharded data parallelism (ZeRO) and synchronised batch norm over any Group.

``FSDP`` follows the reference (ferrotorch-distributed/src/fsdp.rs:66-900): strategies
``FULL_SHARD`` (parameters, gradients and optimizer state sharded; all-gather before forward,
reduce-scatter after backward), ``SHARD_GRAD_OP`` (parameters stay gathered between forward
and backward; gradients / optimizer state sharded), ``NO_SHARD`` (plain all-reduce) and
``HYBRID_SHARD`` (shard inside a node, replicate across nodes: reduce-scatter on the intra-node
sub-group, all-reduce of the shard on the inter-node sub-group, fsdp.rs:740-787).  Every
parameter is flattened and padded to a multiple of the shard-group size (the reference asserts
divisibility, fsdp.rs:231); the optimizer is built on ``fsdp.shard_parameters()``.

``SyncBatchNorm2d`` mirrors sync_batch_norm.rs:85-590: one all-reduce of ``[sum, sum_sq]``
(2C floats) in forward, one of ``[sum_dy, sum_dy_xhat]`` in backward.
"""
from __future__ import annotations

import enum

import torch
from torch import nn

from .backend import Group, SubGroup


class ShardingStrategy(enum.Enum):
    FULL_SHARD = "full_shard"
    SHARD_GRAD_OP = "shard_grad_op"
    NO_SHARD = "no_shard"
    HYBRID_SHARD = "hybrid_shard"


class FSDP(nn.Module):
    def __init__(self, module: nn.Module, group: Group, strategy: ShardingStrategy = ShardingStrategy.FULL_SHARD,
                 intra_node_size: int | None = None):
        super().__init__()
        self.module, self.group, self.strategy = module, group, strategy
        self.shard_group: Group = group
        self.replica_group: Group | None = None
        if strategy == ShardingStrategy.HYBRID_SHARD:
            n = intra_node_size or group.world_size
            assert group.world_size % n == 0
            node = group.rank // n
            self.shard_group = SubGroup(group, range(node * n, (node + 1) * n))
            self.replica_group = SubGroup(group, range(group.rank % n, group.world_size, n))
        W, r = self.shard_group.world_size, self.shard_group.rank
        self.params = [p for p in module.parameters() if p.requires_grad]
        self.shapes = [p.shape for p in self.params]
        self.padded = [(p.numel() + W - 1) // W * W for p in self.params]
        self.shards: list[nn.Parameter] = []
        for p, n in zip(self.params, self.padded):
            flat = torch.zeros(n, dtype=p.dtype, device=p.device)
            flat[:p.numel()] = p.detach().reshape(-1)
            self.shards.append(nn.Parameter(flat[r * (n // W):(r + 1) * (n // W)].clone()))
        self._gathered = True
        if strategy == ShardingStrategy.FULL_SHARD or strategy == ShardingStrategy.HYBRID_SHARD:
            self._free_full()

    def shard_parameters(self) -> list[nn.Parameter]:
        """The local shards (what the optimizer updates)."""
        return self.params if self.strategy == ShardingStrategy.NO_SHARD else self.shards

    def _free_full(self) -> None:
        for p in self.params:
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        self._gathered = False

    def gather_parameters(self) -> None:
        """All-gather every parameter from its shards (also what prefetching would overlap)."""
        if self.strategy == ShardingStrategy.NO_SHARD:
            return
        for p, sh, shape in zip(self.params, self.shards, self.shapes):
            full = self.shard_group.all_gather(sh.detach())
            p.data = full[: shape.numel()].view(shape)
        self._gathered = True

    def prefetch_forward_params(self):
        """Start the all-gather of every parameter on a helper thread and return the handle; the
        next ``forward`` waits for it instead of gathering itself, so the gather overlaps whatever
        the caller does in between -- the data loading of the next batch, the optimizer step of
        another module (fsdp.rs:341-368).  One collective is in flight per group at a time: do not
        issue other collectives on the shard group before the forward."""
        from .dist_checkpoint import PendingCollective

        if self.strategy == ShardingStrategy.NO_SHARD:
            return None

        def gather_all():
            return [self.shard_group.all_gather(sh.detach()) for sh in self.shards]

        self._prefetch = PendingCollective(gather_all)
        return self._prefetch

    def forward(self, *a, **kw):
        pending = getattr(self, "_prefetch", None)
        if pending is not None:
            fulls = pending.wait()
            self._prefetch = None
            for p, full, shape in zip(self.params, fulls, self.shapes):
                p.data = full[: shape.numel()].view(shape)
            self._gathered = True
        elif not self._gathered or self.strategy == ShardingStrategy.SHARD_GRAD_OP:
            self.gather_parameters()
        return self.module(*a, **kw)

    def sync_gradients(self) -> None:
        """After backward: reduce-scatter (mean) the gradients into the shards' ``.grad`` and, for
        FULL_SHARD / HYBRID_SHARD, drop the gathered parameters again."""
        if self.strategy == ShardingStrategy.NO_SHARD:
            for p in self.params:
                if p.grad is not None:
                    self.group.all_reduce(p.grad, "mean")
            return
        W = self.shard_group.world_size
        for p, sh, n in zip(self.params, self.shards, self.padded):
            g = torch.zeros(n, dtype=p.dtype, device=sh.device)
            if p.grad is not None:
                g[: p.grad.numel()] = p.grad.reshape(-1)
            part = self.shard_group.reduce_scatter(g.view(W, n // W), "mean").reshape(-1)
            if self.replica_group is not None:
                self.replica_group.all_reduce(part, "mean")
            sh.grad = part
            p.grad = None
        if self.strategy != ShardingStrategy.SHARD_GRAD_OP:
            self._free_full()
        else:
            self._gathered = False

    def full_state_dict(self) -> dict[str, torch.Tensor]:
        self.gather_parameters()
        sd = {k: v.detach().clone() for k, v in self.module.state_dict().items()}
        if self.strategy in (ShardingStrategy.FULL_SHARD, ShardingStrategy.HYBRID_SHARD):
            self._free_full()
        return sd


class _SyncBNFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, group, eps):
        C = x.shape[1]
        dims = [0] + list(range(2, x.dim()))
        n_local = x.numel() // C
        stats = torch.cat([x.sum(dims), (x * x).sum(dims), x.new_tensor([float(n_local)])])
        group.all_reduce(stats, "sum")
        n = stats[-1]
        mean = stats[:C] / n
        var = stats[C:2 * C] / n - mean * mean
        rstd = torch.rsqrt(var + eps)
        shape = [1, C] + [1] * (x.dim() - 2)
        xhat = (x - mean.view(shape)) * rstd.view(shape)
        ctx.save_for_backward(xhat, weight, rstd)
        ctx.group, ctx.n, ctx.dims, ctx.shape = group, n, dims, shape
        ctx.mark_non_differentiable(mean, var)
        return xhat * weight.view(shape) + bias.view(shape), mean, var

    @staticmethod
    def backward(ctx, dy, _dm, _dv):
        xhat, weight, rstd = ctx.saved_tensors
        C = xhat.shape[1]
        sum_dy, sum_dy_xhat = dy.sum(ctx.dims), (dy * xhat).sum(ctx.dims)
        packed = torch.cat([sum_dy, sum_dy_xhat])
        ctx.group.all_reduce(packed, "sum")
        g_dy, g_dyx = packed[:C] / ctx.n, packed[C:] / ctx.n
        sh = ctx.shape
        dx = (dy - g_dy.view(sh) - xhat * g_dyx.view(sh)) * (weight * rstd).view(sh)
        # weight / bias gradients stay local; the data-parallel wrapper averages them
        return dx, sum_dy_xhat, sum_dy, None, None


class SyncBatchNorm2d(nn.Module):
    def __init__(self, num_features: int, group: Group, eps: float = 1e-5, momentum: float = 0.1):
        super().__init__()
        self.group, self.eps, self.momentum = group, eps, momentum
        self.weight = nn.Parameter(torch.ones(num_features))
        self.bias = nn.Parameter(torch.zeros(num_features))
        self.register_buffer("running_mean", torch.zeros(num_features))
        self.register_buffer("running_var", torch.ones(num_features))
        self.register_buffer("num_batches_tracked", torch.zeros((), dtype=torch.long))

    def with_backend(self, group: Group) -> "SyncBatchNorm2d":
        """The same layer (shared parameters and statistics) synchronising over another group."""
        import copy

        out = copy.copy(self)
        out.group = group
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.training:
            return nn.functional.batch_norm(x, self.running_mean, self.running_var, self.weight, self.bias, False,
                                            0.0, self.eps)
        y, mean, var = _SyncBNFn.apply(x, self.weight, self.bias, self.group, self.eps)
        with torch.no_grad():
            self.num_batches_tracked += 1
            n = x.numel() // x.shape[1] * self.group.world_size
            self.running_mean.lerp_(mean, self.momentum)
            self.running_var.lerp_(var * n / max(n - 1, 1), self.momentum)
        return y
