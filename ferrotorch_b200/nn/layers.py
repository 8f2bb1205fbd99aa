"""Transformer building blocks on the native kernels.

Module names and parameter layouts follow the reference's ``ferrotorch-nn`` so checkpoints
load unchanged: ``Linear.weight`` is ``[out, in]`` (ferrotorch-nn/src/linear.rs:101),
``RMSNorm.weight`` is ``[hidden]`` (norm.rs:1222), RoPE has the two pair conventions and the
scaling modes of transformer.rs:66-326, ``SwiGLU`` is ``down(act(gate(x)) * up(x))``
(transformer.rs:693-764) and ``KVCache`` appends along the sequence (transformer.rs:864-928).
"""
from __future__ import annotations


import torch
from torch import nn

from ..ops import functional as F
from ..ops import reference as ref


class Linear(nn.Linear):
    """``y = x W^T + b`` on the tcgen05 GEMM (bf16 CUDA inputs); any other input uses torch."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)


class FusedLinearActivation(nn.Module):
    """Linear followed by relu / gelu / silu in the GEMM epilogue -- the pattern the reference's
    JIT rewrites to ``FusedLinearActivation`` (ferrotorch-jit/src/optimize.rs:523-601).
    Inference only (no autograd formula); training code uses ``Linear`` + activation."""

    def __init__(self, in_features: int, out_features: int, activation: str = "relu", bias: bool = True):
        super().__init__()
        self.linear = Linear(in_features, out_features, bias=bias)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w, b = self.linear.weight, self.linear.bias
        if x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled():
            y = F.gemm_nt(x.reshape(-1, x.shape[-1]), w, bias=b, activation=self.activation)
            return y.view(*x.shape[:-1], w.shape[0])
        return getattr(torch.nn.functional, self.activation)(torch.nn.functional.linear(x, w, b))


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """With ``residual`` returns ``(norm(x + residual), x + residual)`` from one kernel."""
        return F.rmsnorm(x, self.weight, self.eps, residual)

    def extra_repr(self) -> str:
        return "%d, eps=%g" % (self.weight.numel(), self.eps)


class RotaryPositionEmbedding(nn.Module):
    """cos/sin tables + in-place rotation.  ``scaling``: None | {"type": "linear"|"ntk"|"yarn"|"llama3", ...}."""

    def __init__(self, head_dim: int, max_position_embeddings: int = 8192, theta: float = 10000.0,
                 interleaved: bool = False, scaling: dict | None = None):
        super().__init__()
        self.head_dim, self.max_pos, self.theta = head_dim, max_position_embeddings, theta
        self.interleaved, self.scaling = interleaved, scaling
        # fp32 tables kept outside the module's buffers so that ``module.to(bfloat16)`` cannot
        # round them; one copy per device, created on first use
        self._tables_cpu = ref.rope_tables(head_dim, max_position_embeddings, theta, scaling)
        self._tables_dev: dict = {}

    def _tables(self, device):
        key = str(device)
        t = self._tables_dev.get(key)
        if t is None:
            t = tuple(x.to(device) for x in self._tables_cpu)
            self._tables_dev[key] = t
        return t

    def forward(self, x: torch.Tensor, *, positions: torch.Tensor | None = None, seq_len: int = 0,
                pos_offset: int = 0, n_rot_heads: int | None = None) -> torch.Tensor:
        cos, sin = self._tables(x.device)
        return F.rope_(x, cos, sin, positions=positions, n_rot_heads=n_rot_heads, seq_len=seq_len,
                       pos_offset=pos_offset, interleaved=self.interleaved)

    # ---- the reference's constructors and accessors (ferrotorch-nn/src/transformer.rs:209-420)
    @classmethod
    def with_convention(cls, dim: int, max_seq_len: int, base: float = 10000.0, convention="half") -> "RotaryPositionEmbedding":
        """``convention``: ``"half"`` (LLaMA / GPT-NeoX: element i pairs with i + dim/2) or
        ``"interleaved"`` (elements 2i, 2i + 1)."""
        return cls.with_scaling(dim, max_seq_len, base, convention, None)

    @classmethod
    def with_scaling(cls, dim: int, max_seq_len: int, base: float = 10000.0, convention="half", scaling: dict | None = None
                     ) -> "RotaryPositionEmbedding":
        conv = str(getattr(convention, "value", convention))
        if conv not in ("half", "interleaved"):
            raise ValueError("RoPE convention must be 'half' or 'interleaved', got %r" % (convention,))
        if dim <= 0 or dim % 2 or max_seq_len <= 0:
            raise ValueError("RoPE needs an even positive dim and a positive max_seq_len, got %d and %d" % (dim, max_seq_len))
        return cls(dim, max_seq_len, base, interleaved=conv == "interleaved", scaling=scaling)

    @property
    def dim(self) -> int:
        return self.head_dim

    @property
    def max_seq_len(self) -> int:
        return self.max_pos

    @property
    def base(self) -> float:
        return self.theta

    @property
    def convention(self) -> str:
        return "interleaved" if self.interleaved else "half"

    def apply(self, x: torch.Tensor, seq_offset: int = 0) -> torch.Tensor:
        """Rotated copy of ``x [..., seq, dim]`` with positions ``seq_offset ..`` (transformer.rs ``apply``);
        :meth:`forward` is the in-place form on ``[B, S, heads, dim]`` that the models use."""
        S, D = x.shape[-2], x.shape[-1]
        if D != self.head_dim:
            raise ValueError("RoPE.apply: last dimension %d, expected %d" % (D, self.head_dim))
        if seq_offset + S > self.max_pos:
            raise ValueError("RoPE.apply: positions %d .. %d exceed max_seq_len %d" % (seq_offset, seq_offset + S, self.max_pos))
        y = x.reshape(-1, S, 1, D).clone()
        return self.forward(y, seq_len=S, pos_offset=seq_offset).reshape(x.shape)


class SwiGLU(nn.Module):
    """Gated MLP with one fused ``[gate | up]`` projection (2F x H) so that the activation kernel
    reads one GEMM output."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False,
                 activation_param: float | None = None):
        super().__init__()
        self.gate_up_proj = Linear(hidden_size, 2 * intermediate_size, bias=bias)
        self.down_proj = Linear(intermediate_size, hidden_size, bias=bias)
        self.activation, self.activation_param = activation, activation_param

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(F.swiglu(self.gate_up_proj(x), self.activation, self.activation_param))


class KVCache:
    """Contiguous per-layer cache ``[B, max_len, Hkv, D]`` with an append cursor
    (ferrotorch-nn/src/transformer.rs:864-928; ferrotorch-llama/src/kv_cache.rs:37-136)."""

    def __init__(self, batch: int, max_len: int, n_kv_heads: int, head_dim: int, device=None,
                 dtype=torch.bfloat16):
        self.k = torch.zeros(batch, max_len, n_kv_heads, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.len = 0

    def append(self, k: torch.Tensor, v: torch.Tensor):
        n = k.shape[1]
        if self.len + n > self.k.shape[1]:
            raise ValueError("KVCache overflow: %d + %d > %d" % (self.len, n, self.k.shape[1]))
        self.k[:, self.len:self.len + n].copy_(k)
        self.v[:, self.len:self.len + n].copy_(v)
        self.len += n
        return self.k[:, :self.len], self.v[:, :self.len]

    def reset(self):
        self.len = 0

    # ---- the reference's method set (ferrotorch-nn/src/transformer.rs:864-1010): tensors are
    # ``[B, num_kv_heads, seq, head_dim]`` there, ``[B, seq, num_kv_heads, head_dim]`` in this class
    @classmethod
    def with_dims(cls, max_seq_len: int, batch: int, num_kv_heads: int, head_dim: int, device=None, dtype=torch.bfloat16) -> "KVCache":
        """``with_dims(max_seq_len, 1, 8, 128)`` for Llama-3-8B."""
        return cls(batch, max_seq_len, num_kv_heads, head_dim, device, dtype)

    def update(self, key: torch.Tensor, value: torch.Tensor):
        """Append ``key`` / ``value`` given as ``[B, num_kv_heads, new_seq, head_dim]``; returns the full
        keys and values in the same layout."""
        want = (self.k.shape[0], self.k.shape[2], self.k.shape[3])
        if key.dim() != 4 or key.shape != value.shape or (key.shape[0], key.shape[1], key.shape[3]) != want:
            raise ValueError("KVCache.update: got %s, cache holds [B=%d, kv_heads=%d, _, head_dim=%d]" % ((tuple(key.shape),) + want))
        k, v = self.append(key.transpose(1, 2), value.transpose(1, 2))
        return k.transpose(1, 2), v.transpose(1, 2)

    def seq_len(self) -> int:
        return self.len

    def is_empty(self) -> bool:
        return self.len == 0

    def max_seq_len(self) -> int:
        return self.k.shape[1]

    def num_kv_heads(self) -> int:
        return self.k.shape[2]

    def head_dim(self) -> int:
        return self.k.shape[3]

    def batch_size(self) -> int:
        return self.k.shape[0]


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, Hkv, S, D] -> [B, Hkv * n_rep, S, D]`` (ferrotorch-nn/src/attention.rs:682)."""
    return ref.repeat_kv(x, n_rep)


def scaled_dot_product_attention(q, k, v, causal: bool = True, scale: float | None = None):
    """Attention on ``[B, S, H, D]`` tensors (differentiable; GQA when ``k`` has fewer heads)."""
    from ..ops.attention import flash_attention

    return flash_attention(q, k, v, causal=causal, scale=scale)


class GQAAttention(nn.Module):
    """Grouped-query self-attention with a fused QKV projection and in-place RoPE on the packed
    buffer (ferrotorch-llama/src/attention.rs:213-280 runs q/k/v as three GEMMs, three layout
    transposes, two RoPE launches and two repeat_kv copies; here: one GEMM, one RoPE launch,
    flash attention reading the packed buffer, one output GEMM)."""

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int | None = None,
                 rope: RotaryPositionEmbedding | None = None, bias: bool = False):
        super().__init__()
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = head_dim or hidden_size // n_heads
        self.qkv_proj = Linear(hidden_size, (n_heads + 2 * n_kv_heads) * self.head_dim, bias=bias)
        self.o_proj = Linear(n_heads * self.head_dim, hidden_size, bias=bias)
        self.rope = rope

    def forward(self, x: torch.Tensor, *, cache: KVCache | None = None, positions: torch.Tensor | None = None,
                causal: bool = True) -> torch.Tensor:
        from ..ops.attention import flash_attention, qkv_attention

        B, S, _ = x.shape
        Hq, Hkv, D = self.n_heads, self.n_kv_heads, self.head_dim
        if cache is None and positions is None:
            cos, sin = self.rope._tables(x.device) if self.rope is not None else (None, None)
            o = qkv_attention(x, self.qkv_proj.weight, self.qkv_proj.bias, cos, sin, n_heads=Hq,
                              n_kv_heads=Hkv, head_dim=D, causal=causal,
                              interleaved=self.rope.interleaved if self.rope is not None else False)
            return self.o_proj(o)
        qkv = self.qkv_proj(x).view(B, S, Hq + 2 * Hkv, D)
        if self.rope is not None:
            off = cache.len if cache is not None else 0
            qkv = self.rope(qkv, positions=positions, seq_len=S, pos_offset=off, n_rot_heads=Hq + Hkv)
        q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
        if cache is not None:
            k, v = cache.append(k, v)
        o = flash_attention(q, k, v, causal=causal)
        return self.o_proj(o.reshape(B, S, Hq * D))

    def forward_with_cache(self, x: torch.Tensor, layer_cache=None, seq_offset: int | None = None):
        """``(output, new layer cache)`` for ``x [B, S, hidden]`` on a value cache
        (ferrotorch-llama/src/attention.rs:121-200 ``forward_with_cache``): keys (after RoPE) and values of the
        new positions are appended to a copy of ``layer_cache`` (a ``LayerKvCache`` or ``None``), which is
        returned; the argument is left untouched."""
        from ..models.llama_compat import _GrowingLayerCache

        if x.shape[0] != 1:
            raise ValueError("forward_with_cache serves one sequence; got a batch of %d" % x.shape[0])
        grow = _GrowingLayerCache(layer_cache)
        if seq_offset is not None and seq_offset != grow.len:
            raise ValueError("forward_with_cache: seq_offset %d but the cache holds %d positions" % (seq_offset, grow.len))
        return self.forward(x, cache=grow), grow.as_layer()

    def num_heads(self) -> int:
        return self.n_heads

    def num_kv_heads(self) -> int:
        return self.n_kv_heads


def clip_grad_norm_(parameters, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    """Global-norm clipping; returns the pre-clip norm (ferrotorch-nn/src/utils.rs:148-240)."""
    return torch.nn.utils.clip_grad_norm_(parameters, max_norm, norm_type)


def clip_grad_value_(parameters, clip_value: float) -> None:
    torch.nn.utils.clip_grad_value_(parameters, clip_value)
