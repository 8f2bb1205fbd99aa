"""Function-style collectives and the reference's type names over the group classes
(ferrotorch-distributed/src/lib.rs:181-247; collective.rs:43-744; checkpoint.rs:107-145, 478,
910; nccl_collective.rs:87-279).  Every function takes the group (the reference's ``&dyn
Backend``) as an argument; the ``*_with_timeout`` forms bound the call's point-to-point waits.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass, field

import torch

from . import backend as _b
from .backend import (BackendUnavailable, DistributedError, Group, HybridGroup, SimulatedGroup, SizeMismatch, SubGroup,
                      TcpGroup, TorchGroup)
from .dist_checkpoint import (AsyncDistributedCheckpointer, RpcAgent, load_distributed as _load_distributed, shard_sizes)

DEFAULT_COLLECTIVE_TIMEOUT = _b.DEFAULT_COLLECTIVE_TIMEOUT_S

Backend, TcpBackend, SimulatedBackend, SubBackend, HybridBackend = Group, TcpGroup, SimulatedGroup, SubGroup, HybridGroup
from .dist_checkpoint import TcpRpcBackend  # noqa: F401,E402


class ReduceOp(str, enum.Enum):
    Sum = "sum"
    Mean = "mean"

    def __str__(self) -> str:
        return self.value


class RpcError(DistributedError):
    pass


class DistCheckpointError(DistributedError):
    pass


def _op(op) -> str:
    return op.value if isinstance(op, ReduceOp) else str(op)


class _timeout:
    """Temporarily lower a group's wait limit (groups without one run unchanged)."""

    def __init__(self, group: Group, seconds: float | None):
        self.g, self.s, self.prev = group, seconds, None

    def __enter__(self):
        if self.s is not None and hasattr(self.g, "timeout"):
            self.prev = self.g.timeout
            self.g.set_timeout(self.s) if hasattr(self.g, "set_timeout") else setattr(self.g, "timeout", self.s)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            self.g.set_timeout(self.prev) if hasattr(self.g, "set_timeout") else setattr(self.g, "timeout", self.prev)
        return False


def allreduce(tensor: torch.Tensor, group: Group, op=ReduceOp.Sum) -> torch.Tensor:
    """Every rank ends with the same (bitwise identical) reduction; returns a new tensor."""
    return group.all_reduce(tensor.clone(), _op(op))


def allreduce_with_timeout(tensor, group, op=ReduceOp.Sum, timeout: float | None = None):
    with _timeout(group, timeout):
        return allreduce(tensor, group, op)


def broadcast(tensor: torch.Tensor, group: Group, root: int = 0) -> torch.Tensor:
    return group.broadcast(tensor.clone(), root)


def all_gather(tensor: torch.Tensor, group: Group) -> torch.Tensor:
    """Concatenation of every rank's tensor along dim 0."""
    return group.all_gather(tensor)


def all_gather_with_timeout(tensor, group, timeout: float | None = None):
    with _timeout(group, timeout):
        return all_gather(tensor, group)


def reduce_scatter(tensor: torch.Tensor, group: Group, op=ReduceOp.Sum) -> torch.Tensor:
    if tensor.shape[0] % group.world_size:
        raise SizeMismatch("reduce_scatter: dim 0 (%d) not divisible by world size %d" % (tensor.shape[0], group.world_size))
    return group.reduce_scatter(tensor, _op(op))


reduce_scatter_tensor = reduce_scatter


def reduce_scatter_with_timeout(tensor, group, op=ReduceOp.Sum, timeout: float | None = None):
    with _timeout(group, timeout):
        return reduce_scatter(tensor, group, op)


def all_to_all(tensor: torch.Tensor, group: Group) -> torch.Tensor:
    """Rank r's i-th chunk of dim 0 goes to rank i; the result holds the chunks received, in rank order."""
    return group.all_to_all(tensor)


def all_to_all_single_uneven(tensor: torch.Tensor, send_counts, recv_counts, group: Group) -> torch.Tensor:
    return group.all_to_all(tensor, list(send_counts), list(recv_counts))


def all_to_all_with_timeout(tensor, group, timeout: float | None = None):
    with _timeout(group, timeout):
        return all_to_all(tensor, group)


def barrier(group: Group) -> None:
    group.barrier()


# --------------------------------------------------------------------------- library back-ends
class NcclUniqueId(bytes):
    """Opaque communicator id; with torch.distributed the store carries it, so this is only a
    value type for code that passes one around."""


def NcclBackend(pg=None) -> TorchGroup:
    """The NCCL process group (``torch.distributed`` must be initialised with backend nccl)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized() and "nccl" in str(dist.get_backend(pg))):
        raise BackendUnavailable("NcclBackend: torch.distributed is not initialised with the nccl backend")
    return TorchGroup(pg)


def GlooBackend(pg=None) -> TorchGroup:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        raise BackendUnavailable("GlooBackend: torch.distributed is not initialised")
    return TorchGroup(pg)


def MpiBackend(*a, **kw):
    raise BackendUnavailable("MpiBackend: this build has no MPI transport; launch under mpirun with the tcp backend "
                             "(RendezvousConfig.from_env reads OMPI_COMM_WORLD_* / PMI_*)")


def UccBackend(*a, **kw):
    raise BackendUnavailable("UccBackend: this build has no UCC transport")


def _device_collective(name):
    def run(tensor: torch.Tensor, group: TorchGroup, *a, **kw) -> torch.Tensor:
        if not tensor.is_cuda:
            raise _b.UnsupportedOp("%s: device tensors only (host tensors go through the group's own methods)" % name)
        return getattr(group, name)(tensor, *a, **kw)
    run.__name__ = "nccl_" + name
    return run


nccl_allreduce = _device_collective("all_reduce")
nccl_broadcast = _device_collective("broadcast")
nccl_all_gather = _device_collective("all_gather")
nccl_reduce_scatter = _device_collective("reduce_scatter")


# --------------------------------------------------------------------------- distributed checkpoint types
@dataclass
class TensorShardSpec:
    full_shape: list
    shard_dim: int
    shard_sizes: list

    def to_json(self) -> dict:
        return {"full_shape": list(self.full_shape), "shard_dim": self.shard_dim, "shard_sizes": list(self.shard_sizes)}


@dataclass
class ShardMetadata:
    num_ranks: int
    tensor_specs: dict = field(default_factory=dict)

    def to_json(self) -> dict:
        return {"num_ranks": self.num_ranks, "tensor_specs": {k: v.to_json() for k, v in self.tensor_specs.items()}}

    @classmethod
    def from_json(cls, d: dict) -> "ShardMetadata":
        return cls(int(d["num_ranks"]), {k: TensorShardSpec(list(v["full_shape"]), int(v["shard_dim"]), list(v["shard_sizes"]))
                                         for k, v in d["tensor_specs"].items()})


@dataclass
class DistributedCheckpoint:
    checkpoint_dir: str
    shard_metadata: ShardMetadata

    @classmethod
    def open(cls, directory: str) -> "DistributedCheckpoint":
        import json

        path = os.path.join(directory, "metadata.json")
        if not os.path.exists(path):
            raise DistCheckpointError("no metadata.json under %s" % directory)
        with open(path) as f:
            return cls(directory, ShardMetadata.from_json(json.load(f)))

    def load(self, rank: int, world_size: int, device="cpu") -> dict:
        return reshard(self.checkpoint_dir, self.shard_metadata.num_ranks, world_size, rank, device)


def flat_shard_metadata(state_dict: dict, world_size: int) -> ShardMetadata:
    """Metadata for flat (FSDP-style) shards: every local tensor is one of ``world_size`` equal
    1-D chunks of its full tensor."""
    return ShardMetadata(world_size, {k: TensorShardSpec([v.numel() * world_size], 0, [v.numel()] * world_size)
                                      for k, v in state_dict.items()})


def reshard(directory: str, old_world_size: int, new_world_size: int, new_rank: int, device="cpu") -> dict:
    """This rank's shards of a checkpoint written by ``old_world_size`` ranks (whole shard files
    are read, concatenated and re-cut; remainders go to the leading ranks)."""
    if new_world_size < 1 or not 0 <= new_rank < new_world_size:
        raise DistCheckpointError("reshard: rank %d of %d" % (new_rank, new_world_size))
    state, _ = _load_distributed(directory, new_rank, new_world_size, device, uneven=True)
    return state


AsyncCheckpointer = AsyncDistributedCheckpointer
CheckpointFuture = AsyncDistributedCheckpointer       # save_async returns the checkpointer itself: wait() / is_done()
__all__ = [n for n in dir() if not n.startswith("_") and n not in ("annotations", "enum", "os", "dataclass", "field", "torch")]
