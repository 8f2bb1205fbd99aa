"""Plain-PyTorch restatements of every native op (the oracle for the CUDA kernels and the
CPU execution path).

Each function states the reference's semantics and cites where the reference defines
them.  They compute in fp32 and cast the result back to the input dtype, which is what
the kernels do (bf16 storage, fp32 math).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5, residual: torch.Tensor | None = None):
    """``x * rsqrt(mean(x^2) + eps) * w`` with fp32 statistics
    (ferrotorch-gpu/src/kernels.rs:10578, bf16.rs:1340-1346).  With ``residual`` the input
    is ``x + residual`` (rounded to the storage dtype first) and the sum is returned too."""
    if residual is not None:
        x = (x.float() + residual.float()).to(x.dtype)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = (xf * rstd * weight.float()).to(x.dtype)
    return (y, x) if residual is not None else y


def rope_tables(head_dim: int, max_pos: int, theta: float = 10000.0, scaling: dict | None = None,
                device=None):
    """cos/sin tables ``[max_pos, head_dim/2]`` in fp32.

    ``scaling`` follows the reference's ``RoPEScaling`` (ferrotorch-nn/src/transformer.rs:227-326):
    ``{"type": "linear", "factor": f}``, ``{"type": "ntk", "factor": f, "original_max": n}``,
    ``{"type": "yarn", "factor": f, "original_max": n, "beta_fast": 32, "beta_slow": 1}`` or the
    Llama-3.1 ``{"type": "llama3", ...}`` frequency smoothing used by HF checkpoints."""
    half = head_dim // 2
    idx = torch.arange(half, dtype=torch.float64)
    base = float(theta)
    kind = (scaling or {}).get("type")
    if kind == "ntk":
        f = float(scaling["factor"])
        base = base * f ** (head_dim / (head_dim - 2))
    inv_freq = 1.0 / (base ** (2.0 * idx / head_dim))
    pos = torch.arange(max_pos, dtype=torch.float64)
    mscale = 1.0
    if kind == "linear":
        pos = pos / float(scaling["factor"])
    elif kind == "yarn":
        # The reference's schedule (transformer.rs:357-392): correction range found on the full
        # dimension and halved onto the inv_freq index space, no attention temperature.  The
        # Hugging Face variant differs in both points: ``"hf_range": True`` keeps the range
        # un-halved, ``"mscale": True`` multiplies cos / sin by 0.1 ln(factor) + 1.
        f = float(scaling["factor"])
        orig = float(scaling.get("original_max", max_pos))
        bf, bs = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))

        def corr_dim(n_rot):
            return (head_dim * math.log(orig / (n_rot * 2 * math.pi))) / (2 * math.log(theta))

        low = max(float(math.floor(corr_dim(bf))), 0.0)
        high = min(float(math.ceil(corr_dim(bs))), float(head_dim - 1))
        if scaling.get("hf_range", False):
            high = min(high, float(half - 1))
        else:
            low, high = low / 2.0, high / 2.0
        denom = 0.001 if high == low else high - low
        ramp = ((idx - low) / denom).clamp(0, 1)
        mask = 1.0 - ramp  # 1 -> keep extrapolated (high freq), 0 -> interpolate
        inv_freq = inv_freq / f * (1 - mask) + inv_freq * mask
        mscale = 0.1 * math.log(f) + 1.0 if (scaling.get("mscale", False) and f > 1) else 1.0
    elif kind == "llama3":
        f = float(scaling.get("factor", 8.0))
        lo_f, hi_f = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        orig = float(scaling.get("original_max", 8192))
        wavelen = 2 * math.pi / inv_freq
        smooth = ((orig / wavelen) - lo_f) / (hi_f - lo_f)
        scaled = torch.where(wavelen > orig / lo_f, inv_freq / f, inv_freq)
        mid = (wavelen <= orig / lo_f) & (wavelen >= orig / hi_f)
        inv_freq = torch.where(mid, (1 - smooth) * inv_freq / f + smooth * inv_freq, scaled)
    ang = torch.outer(pos, inv_freq)
    cos = (ang.cos() * mscale).float()
    sin = (ang.sin() * mscale).float()
    if device is not None:
        cos, sin = cos.to(device), sin.to(device)
    return cos, sin


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor,
         interleaved: bool = False, backward: bool = False) -> torch.Tensor:
    """Rotate ``x[..., T, H, D]`` (token-major) by per-token positions.

    half convention: pairs ``(d, d + D/2)`` (ferrotorch-gpu/src/bf16.rs:1850-1855);
    interleaved: pairs ``(2d, 2d+1)`` (ferrotorch-nn/src/transformer.rs:66-72).  The backward
    is the rotation by the negative angle (transformer.rs:132-156)."""
    D = x.shape[-1]
    c = cos[positions].unsqueeze(-2).float()  # [T, 1, D/2]
    s = sin[positions].unsqueeze(-2).float()
    if backward:
        s = -s
    xf = x.float()
    if not interleaved:
        x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    else:
        x1, x2 = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
    return out.to(x.dtype)


_ACTS = {0: F.silu, 1: F.relu, 2: lambda g: F.gelu(g, approximate="tanh")}


def swiglu(gu: torch.Tensor, act: int = 0) -> torch.Tensor:
    """``act(gate) * up`` for ``gu = [gate | up]`` on the last dim (ferrotorch-llama/src/gpu.rs:696-703;
    relu / gelu variants: ferrotorch-nn/src/transformer.rs:693-764)."""
    g, u = gu.float().chunk(2, dim=-1)
    return (_ACTS[act](g) * u).to(gu.dtype)


def fatrelu_glu(gu: torch.Tensor, threshold: float = 0.01) -> torch.Tensor:
    """``fatrelu(gate, t) * up`` with ``fatrelu(x, t) = x if x >= t else 0``
    (ferrotorch-llama/src/mlp.rs:60-71); differentiable."""
    g, u = gu.chunk(2, dim=-1)
    return torch.where(g >= threshold, g, torch.zeros_like(g)) * u


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, Hkv, S, D] -> [B, Hkv*n_rep, S, D]``; output head h reads input head h // n_rep
    (ferrotorch-gpu/src/bf16.rs:2405-2410)."""
    if n_rep == 1:
        return x
    B, H, S, D = x.shape
    return x[:, :, None].expand(B, H, n_rep, S, D).reshape(B, H * n_rep, S, D)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: float | None = None, q_offset: int | None = None):
    """GQA attention on ``[B, S, H, D]`` tensors, returns ``(out [B,Sq,Hq,D], lse [B,Hq,Sq])``.

    Scores scaled by ``1/sqrt(D)``, causal mask hides ``j > i + q_offset`` where the default
    offset aligns the last query with the last key (for Sq == Sk this is the reference's
    top-left mask, ferrotorch-nn/src/flash_attention.rs:647-746), max-subtracted softmax."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = repeat_kv(k.float().permute(0, 2, 1, 3), Hq // Hkv)
    vf = repeat_kv(v.float().permute(0, 2, 1, 3), Hq // Hkv)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        off = (Sk - Sq) if q_offset is None else q_offset
        i = torch.arange(Sq, device=q.device)[:, None] + off
        j = torch.arange(Sk, device=q.device)[None, :]
        s = s.masked_fill(j > i, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100):
    """Per-row ``logsumexp(z) - z[target]`` in fp32 (0 for ignored rows)
    (ferrotorch-nn/src/loss.rs:195-305)."""
    return F.cross_entropy(logits.float(), target, reduction="none", ignore_index=ignore_index)


def adamw_step(p, g, m, v, *, lr, beta1, beta2, eps, weight_decay, step, adam_l2=False):
    """One AdamW update on fp32 tensors, in place (ferrotorch-optim/src/adamw.rs:296-334:
    ``p*(1-lr*wd) - lr*m_hat/(sqrt(v_hat)+eps)``); ``adam_l2`` gives classic Adam with the decay
    folded into the gradient (ferrotorch-gpu/src/kernels.rs:15945-15952)."""
    g = g.float()
    if adam_l2:
        g = g + weight_decay * p
    else:
        p.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    p.sub_(lr * (m / bc1) / ((v / bc2).sqrt() + eps))


def sgd_step(p, g, buf, *, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False,
             first_step=False):
    """One SGD update on fp32 tensors, in place (ferrotorch-optim/src/sgd.rs:224-330)."""
    g = g.float() + weight_decay * p
    if momentum != 0.0:
        if first_step:
            buf.copy_(g)
        else:
            buf.mul_(momentum).add_(g, alpha=1 - dampening)
        g = g + momentum * buf if nesterov else buf
    p.sub_(lr * g)


def dequant_q4_0(blocks: torch.Tensor, nibble_order: str = "ggml") -> torch.Tensor:
    """GGUF Q4_0: blocks of 18 bytes = fp16 scale + 16 bytes of nibbles, value ``(q - 8) * d``.
    ``nibble_order="ggml"`` is the file format's element order (low nibble of byte j = element j,
    high nibble = element j + 16); ``"interleaved"`` is the order the reference's decoder emits
    (elements 2j and 2j + 1, ferrotorch-serialize/src/gguf.rs:543-577).
    ``blocks``: uint8 ``[n_blocks, 18]``."""
    d = blocks[:, :2].contiguous().view(torch.float16).float()  # [n,1]
    qs = blocks[:, 2:]
    lo = (qs & 0x0F).to(torch.int16) - 8
    hi = (qs >> 4).to(torch.int16) - 8
    if nibble_order == "interleaved":
        return (torch.stack([lo, hi], dim=2).reshape(-1, 32).float() * d).reshape(-1)
    return (torch.cat([lo, hi], dim=1).float() * d).reshape(-1)
