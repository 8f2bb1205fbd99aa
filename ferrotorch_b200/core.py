"""Tensor vocabulary of the reference's core crate, mapped onto torch
(ferrotorch-core/src/{tensor,dtype,device}.rs and the tensor families listed in its lib.rs).

Nothing here re-implements a tensor: the names resolve to the torch types and constructors that
play the same role, so code written against the reference's nouns has something to import."""
from __future__ import annotations

import enum

import torch
from torch import Tensor, einsum  # noqa: F401
from torch.masked import MaskedTensor, masked_tensor  # noqa: F401
from torch.nested import nested_tensor  # noqa: F401

from .ops.quant import SemiStructuredLinear, apply_2_4_mask, pack_2_4  # noqa: F401

BoolTensor, IntTensor, LongTensor = torch.BoolTensor, torch.IntTensor, torch.LongTensor
f32, f64, bf16, f16 = torch.float32, torch.float64, torch.bfloat16, torch.float16


class MemoryFormat(enum.Enum):
    """tensor.rs:50-59."""
    Contiguous = torch.contiguous_format
    ChannelsLast = torch.channels_last
    ChannelsLast3d = torch.channels_last_3d


class Device:
    """``Device.Cpu``, ``Device.Cuda(n)``, ``Device.Meta`` (device.rs:28-47).  The Xpu and Mps
    variants of the reference have no counterpart: this package targets CUDA on sm_100a only."""
    Cpu = torch.device("cpu")
    Meta = torch.device("meta")

    @staticmethod
    def Cuda(index: int = 0) -> torch.device:
        return torch.device("cuda", index)

    # predicates on a ``torch.device`` (the reference's ``Device::is_cpu`` ... are methods of its enum)
    @staticmethod
    def is_cpu(device) -> bool:
        return torch.device(device).type == "cpu"

    @staticmethod
    def is_cuda(device) -> bool:
        return torch.device(device).type == "cuda"

    @staticmethod
    def is_meta(device) -> bool:
        return torch.device(device).type == "meta"

    @staticmethod
    def is_xpu(device) -> bool:
        return torch.device(device).type == "xpu"

    @staticmethod
    def is_mps(device) -> bool:
        return torch.device(device).type == "mps"

    @staticmethod
    def Xpu(index: int = 0):
        raise NotImplementedError("Device.Xpu: this package has no Intel back-end")

    @staticmethod
    def Mps(index: int = 0):
        raise NotImplementedError("Device.Mps: this package has no Metal back-end")


def ComplexTensor(real: Tensor, imag: Tensor) -> Tensor:
    return torch.complex(real, imag)


def SparseTensor(indices: Tensor, values: Tensor, size) -> Tensor:
    """COO sparse tensor; ``.to_sparse_csr()`` / ``.to_sparse_csc()`` give the other layouts."""
    return torch.sparse_coo_tensor(indices, values, size).coalesce()


def NestedTensor(tensors, **kw) -> Tensor:
    return torch.nested.nested_tensor(list(tensors), **kw)


def NamedTensor(data: Tensor, names) -> Tensor:
    return data.refine_names(*names)


def QuantizedTensor(data: Tensor, scale: float, zero_point: int = 0, dtype=torch.qint8) -> Tensor:
    """Per-tensor affine quantisation (quantize.rs); ``.dequantize()`` goes back."""
    return torch.quantize_per_tensor(data.float(), scale, zero_point, dtype)


def rearrange(tensor: Tensor, pattern: str, **axes) -> Tensor:
    import einops

    return einops.rearrange(tensor, pattern, **axes)


def reduce(tensor: Tensor, pattern: str, reduction: str, **axes) -> Tensor:
    import einops

    return einops.reduce(tensor, pattern, reduction, **axes)


def repeat(tensor: Tensor, pattern: str, **axes) -> Tensor:
    import einops

    return einops.repeat(tensor, pattern, **axes)


class BlockMask:
    """Block-sparse visibility for :func:`flex_attention`: ``keep[i, j]`` says whether query block i
    may see key block j at all (flex_attention.rs ``BlockMask``).  Built from an element-level
    predicate ``mask_fn(q_index, kv_index) -> bool`` evaluated once per block pair."""

    def __init__(self, keep: Tensor, block: int, q_len: int, kv_len: int):
        self.keep, self.block, self.q_len, self.kv_len = keep, block, q_len, kv_len

    @classmethod
    def from_fn(cls, mask_fn, q_len: int, kv_len: int, block: int = 64) -> "BlockMask":
        qi, ki = torch.arange(q_len)[:, None], torch.arange(kv_len)[None, :]
        dense = mask_fn(qi, ki).expand(q_len, kv_len)
        nq, nk = -(-q_len // block), -(-kv_len // block)
        pad = torch.zeros(nq * block, nk * block, dtype=torch.bool)
        pad[:q_len, :kv_len] = dense
        keep = pad.view(nq, block, nk, block).permute(0, 2, 1, 3).flatten(2).any(-1)
        return cls(keep, block, q_len, kv_len)

    # ---- the reference's constructors and queries (ferrotorch-nn/src/flex_attention.rs:69-200)
    @classmethod
    def full_mask(cls, n_q: int, n_k: int, block_size: int = 64) -> "BlockMask":
        """Every block takes part: no masking."""
        if min(n_q, n_k, block_size) < 1:
            raise ValueError("BlockMask: lengths and block size must be positive")
        return cls(torch.ones(-(-n_q // block_size), -(-n_k // block_size), dtype=torch.bool), block_size, n_q, n_k)

    @classmethod
    def causal_mask(cls, n: int, block_size: int = 64) -> "BlockMask":
        """Block ``(i, j)`` is active when some query of block i may see some key of block j under
        ``q_pos >= k_pos``, i.e. ``j <= i``."""
        return cls.from_fn(lambda q, k: q >= k, n, n, block_size)

    @classmethod
    def sliding_window_mask(cls, n: int, window_size: int, block_size: int = 64) -> "BlockMask":
        """Queries see keys within ``window_size`` positions on either side."""
        if window_size < 0:
            raise ValueError("BlockMask.sliding_window_mask: window_size must be >= 0")
        return cls.from_fn(lambda q, k: (q - k).abs() <= window_size, n, n, block_size)

    def num_q_blocks(self) -> int:
        return self.keep.shape[0]

    def num_k_blocks(self) -> int:
        return self.keep.shape[1]

    def is_active(self, q_block: int, k_block: int) -> bool:
        return bool(self.keep[q_block, k_block])

    def allows_position(self, q_pos: int, k_pos: int) -> bool:
        """Whether the pair falls in an active block (finer rules are the score function's job)."""
        if not (0 <= q_pos < self.q_len and 0 <= k_pos < self.kv_len):
            return False
        return bool(self.keep[q_pos // self.block, k_pos // self.block])

    def sparsity(self) -> float:
        return 1.0 - float(self.keep.float().mean())

    def dense(self) -> Tensor:
        m = self.keep.repeat_interleave(self.block, 0).repeat_interleave(self.block, 1)
        return m[: self.q_len, : self.kv_len]


def flex_attention(q: Tensor, k: Tensor, v: Tensor, score_mod=None, scale: float | None = None,
                   block_mask: "BlockMask | None" = None) -> Tensor:
    """Attention with a user function applied to the scores before the softmax:
    ``score_mod(score, batch, head, q_index, kv_index) -> score`` and an optional block-sparse
    mask (flex_attention.rs:56, 482).  Dense evaluation; use the flash kernels of
    :mod:`ferrotorch_b200.ops` for the standard masks."""
    B, H, S, D = q.shape
    s = (q.float() @ k.float().transpose(-1, -2)) * (scale if scale is not None else D ** -0.5)
    if block_mask is not None:
        if (block_mask.q_len, block_mask.kv_len) != (S, k.shape[2]):
            raise ValueError("flex_attention: the block mask was built for %dx%d scores" % (block_mask.q_len, block_mask.kv_len))
        s = s.masked_fill(~block_mask.dense().to(s.device), float("-inf"))
    if score_mod is not None:
        b = torch.arange(B, device=q.device).view(B, 1, 1, 1)
        h = torch.arange(H, device=q.device).view(1, H, 1, 1)
        qi = torch.arange(S, device=q.device).view(1, 1, S, 1)
        ki = torch.arange(k.shape[2], device=q.device).view(1, 1, 1, -1)
        s = score_mod(s, b, h, qi, ki)
    return (s.softmax(-1) @ v.float()).to(q.dtype)
