"""Device meshes and a light distributed tensor with *real* redistribution.

Vocabulary from the reference: ``DeviceMesh`` with row-major rank <-> coordinate maps,
``ranks_along_dim`` / ``groups_along_dim`` (ferrotorch-distributed/src/device_mesh.rs:37-203) and
``Placement::{Replicate, Shard(dim), Partial}`` (dtensor.rs:56-67).  The reference's
``DTensor::redistribute`` only rewrites metadata (dtensor.rs:205-230); here it moves data with
the collectives of a :class:`~.backend.Group` (all-gather, reduce-scatter, all-reduce, slice).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from .backend import Group, InvalidRank, SubGroup


class DeviceMesh:
    def __init__(self, shape: Sequence[int], dim_names: Sequence[str] | None = None):
        self.shape = tuple(int(s) for s in shape)
        if not self.shape or any(s < 1 for s in self.shape):
            raise ValueError("mesh shape %r" % (shape,))
        self.dim_names = tuple(dim_names) if dim_names is not None else tuple("dim%d" % i for i in range(len(self.shape)))
        if len(self.dim_names) != len(self.shape):
            raise ValueError("one name per mesh dimension")
        self.size = 1
        for s in self.shape:
            self.size *= s

    def _dim(self, dim) -> int:
        return self.dim_names.index(dim) if isinstance(dim, str) else int(dim)

    def coords(self, rank: int) -> tuple[int, ...]:
        if not 0 <= rank < self.size:
            raise InvalidRank("rank %d outside mesh of %d" % (rank, self.size))
        out = []
        for s in reversed(self.shape):
            out.append(rank % s)
            rank //= s
        return tuple(reversed(out))

    def rank_of(self, coords: Sequence[int]) -> int:
        r = 0
        for c, s in zip(coords, self.shape):
            if not 0 <= c < s:
                raise InvalidRank("coordinate %r outside mesh %r" % (tuple(coords), self.shape))
            r = r * s + c
        return r

    def ranks_along_dim(self, rank: int, dim) -> list[int]:
        """The ranks that differ from ``rank`` only in coordinate ``dim`` (its group on that axis)."""
        d = self._dim(dim)
        c = list(self.coords(rank))
        out = []
        for i in range(self.shape[d]):
            c[d] = i
            out.append(self.rank_of(c))
        return out

    def groups_along_dim(self, dim) -> list[list[int]]:
        seen, groups = set(), []
        for r in range(self.size):
            if r not in seen:
                g = self.ranks_along_dim(r, dim)
                seen.update(g)
                groups.append(g)
        return groups

    def subgroup(self, parent: Group, dim) -> SubGroup:
        """The communication group of ``parent.rank`` along mesh axis ``dim``."""
        return SubGroup(parent, self.ranks_along_dim(parent.rank, dim))

    def torch_groups(self, dim):
        """Create ``torch.distributed`` process groups for every group on ``dim`` (collective);
        returns the one this rank belongs to."""
        import torch.distributed as dist

        mine = None
        for ranks in self.groups_along_dim(dim):
            g = dist.new_group(ranks)
            if dist.get_rank() in ranks:
                mine = g
        return mine


@dataclass(frozen=True)
class Replicate:
    pass


@dataclass(frozen=True)
class Shard:
    dim: int


@dataclass(frozen=True)
class Partial:
    op: str = "sum"


class DTensor:
    """A local shard + its placement on one mesh axis (group) + the global shape."""

    def __init__(self, local: torch.Tensor, group: Group, placement, global_shape: Sequence[int] | None = None):
        self.local, self.group, self.placement = local, group, placement
        if global_shape is None:
            gs = list(local.shape)
            if isinstance(placement, Shard):
                gs[placement.dim] *= group.world_size
            global_shape = gs
        self.global_shape = tuple(global_shape)

    @classmethod
    def from_global(cls, full: torch.Tensor, group: Group, placement) -> "DTensor":
        if isinstance(placement, Shard):
            n = full.shape[placement.dim]
            if n % group.world_size:
                raise ValueError("dim %d (%d) not divisible by %d" % (placement.dim, n, group.world_size))
            local = full.chunk(group.world_size, dim=placement.dim)[group.rank].contiguous()
        else:
            local = full.clone()
        return cls(local, group, placement, full.shape)

    def _gather(self, dim: int) -> torch.Tensor:
        t = self.local.movedim(dim, 0).contiguous()
        full = self.group.all_gather(t)
        return full.movedim(0, dim).contiguous()

    def redistribute(self, placement) -> "DTensor":
        src, g = self.placement, self.group
        if src == placement:
            return self
        if isinstance(src, Partial):
            if isinstance(placement, Replicate):
                out = g.all_reduce(self.local.clone(), src.op)
            elif isinstance(placement, Shard):
                t = self.local.movedim(placement.dim, 0).contiguous()
                out = g.reduce_scatter(t, src.op).movedim(0, placement.dim).contiguous()
            else:
                raise ValueError("Partial -> %r" % (placement,))
        elif isinstance(src, Shard):
            full = self._gather(src.dim)
            if isinstance(placement, Replicate):
                out = full
            elif isinstance(placement, Shard):
                out = full.chunk(g.world_size, dim=placement.dim)[g.rank].contiguous()
            else:
                raise ValueError("Shard -> Partial is not a data movement")
        else:  # Replicate
            if isinstance(placement, Shard):
                out = self.local.chunk(g.world_size, dim=placement.dim)[g.rank].contiguous()
            elif isinstance(placement, Partial):
                out = self.local.clone() if g.rank == 0 else torch.zeros_like(self.local)
            else:
                out = self.local
        return DTensor(out, g, placement, self.global_shape)

    def full_tensor(self) -> torch.Tensor:
        return self.redistribute(Replicate()).local
