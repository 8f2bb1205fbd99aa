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


# the ``_dtype`` spellings take the element type explicitly in the reference (its handle-based wrappers infer
# f32 / f64 from the element size); device tensors carry their dtype, bf16 included, so they are the same calls
nccl_allreduce_dtype, nccl_broadcast_dtype = nccl_allreduce, nccl_broadcast
nccl_all_gather_dtype, nccl_reduce_scatter_dtype = nccl_all_gather, nccl_reduce_scatter


def is_available() -> bool:
    """Whether NCCL can be used here: torch was built with it and a CUDA device is present (nccl_sys.rs:513)."""
    import torch.distributed as dist

    return bool(dist.is_available() and dist.is_nccl_available() and torch.cuda.is_available())


def reduce_op_to_nccl(op):
    """This package's :class:`ReduceOp` (or its string) as the ``torch.distributed`` reduction that NCCL runs
    (``Mean`` is NCCL's ``Avg``)."""
    import torch.distributed as dist

    return {"sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.AVG, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN,
            "prod": dist.ReduceOp.PRODUCT}[_op(op)]


def get_unique_id() -> NcclUniqueId:
    """A fresh communicator id for rank 0 to hand to the others (nccl_sys.rs:282).  ``torch.distributed`` creates
    and distributes NCCL's own id through its store during ``init_process_group``; this value only names a
    rendezvous (it is what :func:`comm_init_rank` keys the store on)."""
    import os

    return NcclUniqueId(os.urandom(128))


def comm_init_rank(world_size: int, unique_id: bytes, rank: int, master_addr: str = "127.0.0.1", master_port: int = 29500,
                   backend: str | None = None) -> TorchGroup:
    """Join the communicator named by ``unique_id`` as ``rank`` of ``world_size`` (nccl_sys.rs:306): initialises
    ``torch.distributed`` (NCCL on a CUDA machine, gloo otherwise) on a TCP store whose keys are prefixed with the
    id, and returns the world group.  The device must be selected first (``torch.cuda.set_device``)."""
    import torch.distributed as dist

    if not 0 <= rank < world_size:
        raise _b.InvalidRank("rank %d outside a world of %d" % (rank, world_size))
    if not dist.is_initialized():
        store = dist.PrefixStore(bytes(unique_id)[:16].hex(), dist.TCPStore(master_addr, master_port, world_size, rank == 0))
        dist.init_process_group(backend or ("nccl" if is_available() else "gloo"), store=store, rank=rank, world_size=world_size)
    return TorchGroup(None)


class _NcclGroupCalls:
    """``group_start()`` ... ``group_end()``: point-to-point calls issued in between are launched together
    (``torch.distributed``'s batched isend / irecv); collectives are unaffected."""
    depth = 0


def group_start() -> None:
    _NcclGroupCalls.depth += 1


def group_end() -> None:
    if _NcclGroupCalls.depth == 0:
        raise DistributedError("group_end without group_start")
    _NcclGroupCalls.depth -= 1


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
