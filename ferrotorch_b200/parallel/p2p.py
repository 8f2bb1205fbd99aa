"""Point-to-point verbs, back-end availability probes and device-tensor collectives under the
reference's names (ferrotorch-distributed/src/p2p.rs:30-160, gpu_collective.rs:290-387,
nccl_backend.rs ``is_nccl_available`` and the feature-gated gloo / MPI / UCC probes)."""
from __future__ import annotations

import enum

import torch

from .backend import Group, SelfSend, UnsupportedOp
from .dist_checkpoint import PendingCollective


class PipelineSchedule(enum.Enum):
    """pipeline.rs:51-61; ``Pipeline(schedule=...)`` takes the values."""
    GPipe = "gpipe"
    OneFOneB = "1f1b"


class Placement:
    """Namespace for the three placements of a distributed tensor (dtensor.rs:56-67)."""
    from .mesh import Partial, Replicate, Shard  # noqa: F401

    @staticmethod
    def is_replicate(p) -> bool:
        return p.is_replicate()

    @staticmethod
    def is_shard(p) -> bool:
        return p.is_shard()

    @staticmethod
    def is_partial(p) -> bool:
        return p.is_partial()

    @staticmethod
    def shard_dim(p):
        return p.shard_dim()


def send(group: Group, tensor: torch.Tensor, dst: int) -> None:
    if dst == group.rank:
        raise SelfSend("rank %d cannot send to itself" % dst)
    group.send(tensor.contiguous(), dst)


def recv_into(group: Group, tensor: torch.Tensor, src: int) -> torch.Tensor:
    return recv_into_with_timeout(group, tensor, src, None)


def recv_into_with_timeout(group: Group, tensor: torch.Tensor, src: int, timeout: float | None) -> torch.Tensor:
    if src == group.rank:
        raise SelfSend("rank %d cannot receive from itself" % src)
    if not tensor.is_contiguous():
        raise ValueError("recv_into: the destination must be contiguous")
    try:
        group.recv(tensor, src, timeout) if timeout is not None else group.recv(tensor, src)
    except TypeError:                       # a group without per-call timeouts
        group.recv(tensor, src)
    return tensor


def recv(group: Group, shape, src: int, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return recv_into(group, torch.empty(tuple(shape), dtype=dtype), src)


def recv_with_timeout(group: Group, shape, src: int, timeout: float, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return recv_into_with_timeout(group, torch.empty(tuple(shape), dtype=dtype), src, timeout)


def sendrecv(group: Group, send_tensor: torch.Tensor, peer: int, recv_shape=None) -> torch.Tensor:
    """Exchange with ``peer`` without deadlock: the lower rank sends first, the higher one receives
    first (p2p.rs ``sendrecv``)."""
    out = torch.empty(tuple(recv_shape) if recv_shape is not None else send_tensor.shape, dtype=send_tensor.dtype)
    if group.rank < peer:
        send(group, send_tensor, peer)
        recv_into(group, out, peer)
    else:
        recv_into(group, out, peer)
        send(group, send_tensor, peer)
    return out


def async_reduce_scatter(group: Group, tensor: torch.Tensor, op: str = "sum") -> PendingCollective:
    return PendingCollective(group.reduce_scatter, tensor, op)


# --------------------------------------------------------------------------- availability
def is_nccl_available() -> bool:
    return bool(torch.distributed.is_available() and torch.distributed.is_nccl_available() and torch.cuda.is_available())


def is_gloo_available() -> bool:
    return bool(torch.distributed.is_available() and torch.distributed.is_gloo_available())


def is_mpi_available() -> bool:
    return bool(torch.distributed.is_available() and torch.distributed.is_mpi_available())


def is_ucc_available() -> bool:
    return bool(torch.distributed.is_available() and torch.distributed.is_ucc_available())


# --------------------------------------------------------------------------- device tensors
def gpu_allreduce(tensor: torch.Tensor, group=None, op: str = "sum") -> torch.Tensor:
    """In-place all-reduce of a CUDA tensor over NCCL on the current stream, without a host
    synchronise (the reference's version synchronises its stream, gpu_collective.rs:157-210).
    Host tensors are refused rather than bounced through the CPU."""
    if not tensor.is_cuda:
        raise UnsupportedOp("gpu_allreduce: the tensor is not on a GPU; use Group.all_reduce for host tensors")
    import torch.distributed as dist

    dist.all_reduce(tensor, op=dist.ReduceOp.SUM if op == "sum" else dist.ReduceOp.AVG, group=group)
    return tensor


def gpu_broadcast(tensor: torch.Tensor, root: int = 0, group=None) -> torch.Tensor:
    if not tensor.is_cuda:
        raise UnsupportedOp("gpu_broadcast: the tensor is not on a GPU; use Group.broadcast for host tensors")
    import torch.distributed as dist

    dist.broadcast(tensor, src=root, group=group)
    return tensor
