"""Native ops (sm_100a kernels with autograd) and their PyTorch oracles."""
from . import reference
from .functional import (cross_entropy_fwd_bwd_, embedding, gemm_nt, linear, linear_cross_entropy,
                         rmsnorm, rope_, stats, swiglu)

__all__ = ["reference", "gemm_nt", "linear", "rmsnorm", "rope_", "swiglu", "embedding",
           "cross_entropy_fwd_bwd_", "linear_cross_entropy", "stats"]
