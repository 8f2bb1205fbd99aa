"""Parallel runtime: back-ends and collectives, data / tensor / pipeline / fully-sharded
parallelism, device meshes and distributed tensors."""
from .backend import (BackendUnavailable, DistributedError, Group, InvalidRank, InvalidWorldSize, IoError,  # noqa: F401
                      NoConnection, SelfSend, SimulatedGroup, SizeMismatch, SubGroup, TcpGroup, Timeout, TorchGroup,
                      UnsupportedOp, init_group, run_simulated)
from .fsdp import FSDP, ShardingStrategy, SyncBatchNorm2d  # noqa: F401
from .host_ddp import DDP  # noqa: F401
from .mesh import DeviceMesh, DTensor, Partial, Replicate, Shard  # noqa: F401
from .pipeline import Pipeline  # noqa: F401
