"""Parallel runtime: back-ends and collectives, data / tensor / pipeline / fully-sharded
parallelism, device meshes and distributed tensors."""
from .backend import (BackendUnavailable, DistributedError, Group, HybridGroup, InvalidRank, InvalidWorldSize, IoError,  # noqa: F401
                      NoConnection, RendezvousConfig, SelfSend, SimulatedGroup, SizeMismatch, SubGroup, TcpGroup, Timeout, TorchGroup,
                      UnsupportedOp, init_group, run_simulated)
from .elastic import FileStore, Heartbeat, RankFailure, TorchStore, survivors  # noqa: F401
from .fsdp import FSDP, ShardingStrategy, SyncBatchNorm2d  # noqa: F401
from .fsdp_flat import FsdpUnit, auto_wrap  # noqa: F401
from .host_ddp import DDP  # noqa: F401
from .mesh import DeviceMesh, DTensor, MeshTensor, Partial, Replicate, Shard  # noqa: F401
from .pipeline import Pipeline  # noqa: F401
from .vocab_sampling import sample_reference, sample_vocab_parallel, shared_uniform  # noqa: F401
from .dist_checkpoint import (AsyncDistributedCheckpointer, GroupRpcAgent, PendingCollective, RpcAgent, all_gather_async,  # noqa: F401,E402
                              all_reduce_async, load_distributed, save_distributed)
from .p2p import (PipelineSchedule, Placement, async_reduce_scatter, gpu_allreduce, gpu_broadcast,  # noqa: F401,E402
                  is_gloo_available, is_mpi_available, is_nccl_available, is_ucc_available, recv, recv_into,
                  recv_into_with_timeout, recv_with_timeout, send, sendrecv)

async_all_gather = all_gather_async
from .functional import *  # noqa: F401,F403,E402


def __getattr__(name):
    """GPU-side classes are imported on first use (they load the kernel library)."""
    lazy = {"FusedDDP": "ddp", "SymmetricBuffer": "ddp", "CommTimeout": "ddp", "TPContext": "tensor_parallel",
            "ColumnParallelLinear": "tp_layers", "RowParallelLinear": "tp_layers",
            "VocabParallelEmbedding": "tp_layers", "vocab_parallel_cross_entropy": "tp_layers",
            "PeerCollectives": "peer_collectives"}
    if name in lazy:
        import importlib

        return getattr(importlib.import_module("." + lazy[name], __name__), name)
    raise AttributeError(name)
