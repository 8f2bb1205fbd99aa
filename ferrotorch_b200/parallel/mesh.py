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

    @classmethod
    def new(cls, shape: Sequence[int], world_size: int) -> "DeviceMesh":
        """Validating constructor (device_mesh.rs:48): the mesh must cover exactly ``world_size`` ranks."""
        m = cls(shape)
        if m.size != world_size:
            raise ValueError("mesh %r covers %d ranks, world size is %d" % (tuple(shape), m.size, world_size))
        return m

    @classmethod
    def new_with_names(cls, shape: Sequence[int], dim_names: Sequence[str], world_size: int) -> "DeviceMesh":
        if len(set(dim_names)) != len(tuple(dim_names)):
            raise ValueError("mesh dimension names must be distinct: %r" % (tuple(dim_names),))
        m = cls(shape, dim_names)
        if m.size != world_size:
            raise ValueError("mesh %r covers %d ranks, world size is %d" % (tuple(shape), m.size, world_size))
        return m

    @property
    def ndim(self) -> int:
        return len(self.shape)

    def dim_index(self, name: str) -> int:
        if name not in self.dim_names:
            raise ValueError("mesh has no dimension named %r (names: %r)" % (name, self.dim_names))
        return self.dim_names.index(name)

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


class _PlacementQueries:
    """The predicates of the reference's ``Placement`` enum (dtensor.rs:70-90)."""

    def is_replicate(self) -> bool:
        return isinstance(self, Replicate)

    def is_shard(self) -> bool:
        return isinstance(self, Shard)

    def is_partial(self) -> bool:
        return isinstance(self, Partial)

    def shard_dim(self):
        return self.dim if isinstance(self, Shard) else None


@dataclass(frozen=True)
class Replicate(_PlacementQueries):
    pass


@dataclass(frozen=True)
class Shard(_PlacementQueries):
    dim: int


@dataclass(frozen=True)
class Partial(_PlacementQueries):
    op: str = "sum"


class DTensor:
    """A local shard + its placement on one mesh axis (group) + the global shape."""
    mesh = None                      # the one-axis form has a group, not a mesh; ``from_local`` builds the mesh form

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

    # ---- the reference's accessors (dtensor.rs:162-190) for the one-axis form
    def to_local(self) -> torch.Tensor:
        return self.local

    @property
    def shape(self) -> tuple:
        return self.global_shape

    @property
    def placements(self) -> list:
        return [self.placement]

    def numel(self) -> int:
        n = 1
        for d in self.global_shape:
            n *= d
        return n

    @staticmethod
    def from_local(local: torch.Tensor, mesh: DeviceMesh, placements, global_shape: Sequence[int] | None = None, groups=None
                   ) -> "MeshTensor":
        """A tensor laid out over every axis of ``mesh`` (dtensor.rs:115): one placement per mesh
        dimension.  ``groups`` (one :class:`~.backend.Group` per mesh dimension, e.g.
        ``[mesh.subgroup(world, d) for d in range(mesh.ndim)]``) makes ``redistribute`` move data;
        without them it rewrites the placement list only, as the reference does."""
        return MeshTensor(local, mesh, list(placements), global_shape, groups)

    @staticmethod
    def from_local_replicated(local: torch.Tensor, mesh: DeviceMesh, groups=None) -> "MeshTensor":
        return MeshTensor(local, mesh, [Replicate()] * mesh.ndim, tuple(local.shape), groups)


class MeshTensor:
    """A local shard, a mesh, and one placement per mesh dimension (the reference's ``DTensor``,
    ferrotorch-distributed/src/dtensor.rs:88-230).  A tensor dimension may be sharded by at most one
    mesh dimension.  ``redistribute`` goes mesh dimension by mesh dimension, each step a collective
    on that dimension's group (all-gather, reduce-scatter, all-reduce or a local slice)."""

    def __init__(self, local: torch.Tensor, mesh: DeviceMesh, placements, global_shape=None, groups=None):
        if len(placements) != mesh.ndim:
            raise ValueError("DTensor.from_local: %d placements for a mesh of %d dimensions" % (len(placements), mesh.ndim))
        if groups is not None:
            groups = list(groups)
            if len(groups) != mesh.ndim or any(g.world_size != n for g, n in zip(groups, mesh.shape)):
                raise ValueError("one group per mesh dimension, sized like it: mesh %r" % (mesh.shape,))
        sharded = [p.dim for p in placements if isinstance(p, Shard)]
        if len(set(sharded)) != len(sharded):
            raise ValueError("a tensor dimension is sharded by two mesh dimensions: %r" % (placements,))
        for mi, p in enumerate(placements):
            if isinstance(p, Shard) and not 0 <= p.dim < local.dim():
                raise ValueError("mesh dim %d shards tensor dim %d of a %d-d tensor" % (mi, p.dim, local.dim()))
        if global_shape is None:
            gs = list(local.shape)
            for p, n in zip(placements, mesh.shape):
                if isinstance(p, Shard):
                    gs[p.dim] *= n
            global_shape = gs
        self.local, self.mesh, self._placements, self.global_shape, self.groups = local, mesh, list(placements), tuple(global_shape), groups

    def to_local(self) -> torch.Tensor:
        return self.local

    @property
    def shape(self) -> tuple:
        return self.global_shape

    @property
    def placements(self) -> list:
        return list(self._placements)

    def numel(self) -> int:
        n = 1
        for d in self.global_shape:
            n *= d
        return n

    def redistribute(self, target_placements) -> "MeshTensor":
        target = list(target_placements)
        if len(target) != self.mesh.ndim:
            raise ValueError("redistribute: %d placements for a mesh of %d dimensions" % (len(target), self.mesh.ndim))
        for mi, p in enumerate(target):
            if isinstance(p, Shard) and not 0 <= p.dim < len(self.global_shape):
                raise ValueError("mesh dim %d shards tensor dim %d of a %d-d tensor" % (mi, p.dim, len(self.global_shape)))
        if self.groups is None:
            return MeshTensor(self.local, self.mesh, target, self.global_shape, None)
        local, cur = self.local, list(self._placements)
        # first every step that frees a tensor dimension (to Replicate), then the ones that shard, so that a
        # tensor dimension handed from one mesh dimension to another is never sharded twice on the way
        order = [i for i in range(self.mesh.ndim) if not isinstance(target[i], Shard)] + \
                [i for i in range(self.mesh.ndim) if isinstance(target[i], Shard)]
        for mi in order:
            if cur[mi] == target[mi]:
                continue
            if isinstance(target[mi], Shard) and any(isinstance(c, Shard) and c.dim == target[mi].dim for j, c in enumerate(cur) if j != mi):
                raise ValueError("tensor dim %d would be sharded by two mesh dimensions" % target[mi].dim)
            local = DTensor(local, self.groups[mi], cur[mi]).redistribute(target[mi]).local
            cur[mi] = target[mi]
        return MeshTensor(local, self.mesh, cur, self.global_shape, self.groups)

    def full_tensor(self) -> torch.Tensor:
        return self.redistribute([Replicate()] * self.mesh.ndim).local
