"""Stable-Diffusion-1.5-shaped latent diffusion stack: CLIP text encoder, conditional UNet, VAE
encoder / decoder, DDIM scheduler and the text-to-image pipeline.

Mirrors the reference's ``ferrotorch-diffusion`` crate (clip_text_encoder.rs, unet.rs, vae.rs,
vae_encoder.rs, scheduler.rs, pipeline.rs; presets ``sd_v1_5`` in config.rs:68, unet_config.rs:82,
clip_text_encoder.rs:143, scheduler.rs:108).  Parameter names are the ones Hugging Face
``transformers`` / ``diffusers`` checkpoints use (``text_model.encoder.layers.0.self_attn.q_proj``,
``down_blocks.0.attentions.0.transformer_blocks.0.attn2.to_k``, ``decoder.up_blocks.1.resnets.2.conv1``
...), so a SafeTensors file of such a checkpoint loads with ``load_state_dict``.  Attention runs
through ``scaled_dot_product_attention``; on a GPU use ``.to(memory_format=torch.channels_last)``
and bf16 like the other vision models.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import nn

# Set by ``models/diffusion_gpu.py`` while one of its device twins runs: attention then goes through
# its dispatcher (flash-attention kernel where a head size fits) instead of the library call.
_attention_override = None


def _sdpa(q, k, v, is_causal: bool = False):
    if _attention_override is not None:
        return _attention_override(q, k, v, is_causal)
    return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal)


def _from_json(cls, src, rename: dict | None = None):
    raw = src
    if isinstance(src, str):
        try:
            raw = json.loads(src)
        except ValueError:
            with open(src) as f:
                raw = json.load(f)
    rename = rename or {}
    kw = {}
    for k, v in raw.items():
        k = rename.get(k, k)
        if k in cls.__dataclass_fields__:
            kw[k] = tuple(v) if isinstance(v, list) else v
    cfg = cls(**kw)
    cfg.validate()
    return cfg


# --------------------------------------------------------------------------- DDIM
@dataclass
class DDIMConfig:
    num_train_timesteps: int = 1000
    beta_start: float = 0.00085
    beta_end: float = 0.012
    beta_schedule: str = "scaled_linear"        # or "linear"
    clip_sample: bool = False
    set_alpha_to_one: bool = False
    prediction_type: str = "epsilon"
    timestep_spacing: str = "leading"           # or "trailing"
    steps_offset: int = 1

    @classmethod
    def sd_v1_5(cls) -> "DDIMConfig":
        return cls()


class DDIMScheduler:
    """Deterministic DDIM (eta = 0) with the conventions of the SD-1.5 scheduler config
    (scheduler.rs:120-330): scaled-linear betas, leading timestep spacing with an offset, the final
    step's "previous alpha" is ``alphas_cumprod[0]`` unless ``set_alpha_to_one``."""

    def __init__(self, config: DDIMConfig | None = None):
        c = self.config = config or DDIMConfig()
        if c.prediction_type != "epsilon":
            raise ValueError("DDIMScheduler: only epsilon prediction is supported")
        if c.num_train_timesteps < 1 or not 0 < c.beta_start <= c.beta_end < 1:
            raise ValueError("DDIMScheduler: bad beta range or step count")
        if c.beta_schedule == "scaled_linear":
            betas = torch.linspace(c.beta_start ** 0.5, c.beta_end ** 0.5, c.num_train_timesteps, dtype=torch.float64) ** 2
        elif c.beta_schedule == "linear":
            betas = torch.linspace(c.beta_start, c.beta_end, c.num_train_timesteps, dtype=torch.float64)
        else:
            raise ValueError("DDIMScheduler: unknown beta schedule %r" % c.beta_schedule)
        self.alphas_cumprod = torch.cumprod(1.0 - betas, 0)
        self.final_alpha_cumprod = torch.tensor(1.0, dtype=torch.float64) if c.set_alpha_to_one else self.alphas_cumprod[0]
        self.timesteps: list[int] = []
        self.num_inference_steps = 0

    def init_noise_sigma(self) -> float:
        return 1.0

    def set_timesteps(self, num_inference_steps: int) -> list[int]:
        T = self.config.num_train_timesteps
        if not 1 <= num_inference_steps <= T:
            raise ValueError("set_timesteps: need 1 <= steps <= %d, got %d" % (T, num_inference_steps))
        self.num_inference_steps = num_inference_steps
        if self.config.timestep_spacing == "leading":
            ratio = T // num_inference_steps
            ts = [min(T - 1, i * ratio + self.config.steps_offset) for i in range(num_inference_steps)][::-1]
        elif self.config.timestep_spacing == "trailing":
            ts = [max(0, round(T - i * T / num_inference_steps) - 1) for i in range(num_inference_steps)]
        else:
            raise ValueError("unknown timestep spacing %r" % self.config.timestep_spacing)
        self.timesteps = ts
        return ts

    def scale_model_input(self, sample: torch.Tensor, timestep: int) -> torch.Tensor:
        return sample                                      # DDIM needs no input scaling

    def add_noise(self, x0: torch.Tensor, noise: torch.Tensor, t) -> torch.Tensor:
        a = self.alphas_cumprod[t].to(x0.device).reshape(-1, *[1] * (x0.dim() - 1)).to(x0.dtype)
        return a.sqrt() * x0 + (1 - a).sqrt() * noise

    def step(self, model_output: torch.Tensor, timestep: int, sample: torch.Tensor) -> torch.Tensor:
        """x_{t_prev} from the predicted noise at ``timestep``."""
        if not self.num_inference_steps:
            raise RuntimeError("call set_timesteps first")
        prev = timestep - self.config.num_train_timesteps // self.num_inference_steps
        a_t = self.alphas_cumprod[timestep]
        a_prev = self.alphas_cumprod[prev] if prev >= 0 else self.final_alpha_cumprod
        x, eps = sample.double(), model_output.double()
        x0 = (x - (1 - a_t).sqrt() * eps) / a_t.sqrt()
        if self.config.clip_sample:
            x0 = x0.clamp(-1, 1)
        return (a_prev.sqrt() * x0 + (1 - a_prev).sqrt() * eps).to(sample.dtype)


# --------------------------------------------------------------------------- CLIP text encoder
@dataclass
class ClipTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 77
    layer_norm_eps: float = 1e-5
    hidden_act: str = "quick_gelu"

    @classmethod
    def sd_v1_5(cls) -> "ClipTextConfig":
        return cls()

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        if min(self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers,
               self.num_attention_heads, self.max_position_embeddings) <= 0:
            raise ValueError("ClipTextConfig: sizes must be positive")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("ClipTextConfig: hidden_size must be divisible by num_attention_heads")
        if self.hidden_act not in ("quick_gelu", "gelu"):
            raise ValueError("ClipTextConfig: unsupported hidden_act %r" % self.hidden_act)

    @classmethod
    def from_json_str(cls, s) -> "ClipTextConfig":
        return _from_json(cls, s)

    from_file = from_json_str


class _ClipAttention(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.h = c.num_attention_heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(c.hidden_size, c.hidden_size) for _ in range(4))

    def forward(self, x):
        B, S, E = x.shape
        q, k, v = (p(x).view(B, S, self.h, E // self.h).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        o = _sdpa(q, k, v, is_causal=True)       # CLIP's text tower is causal
        return self.out_proj(o.transpose(1, 2).reshape(B, S, E))


class _ClipMlp(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(c.hidden_size, c.intermediate_size), nn.Linear(c.intermediate_size, c.hidden_size)
        self.quick = c.hidden_act == "quick_gelu"

    def forward(self, x):
        h = self.fc1(x)
        return self.fc2(h * torch.sigmoid(1.702 * h) if self.quick else F.gelu(h))


class _ClipLayer(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.layer_norm1 = nn.LayerNorm(c.hidden_size, c.layer_norm_eps)
        self.self_attn = _ClipAttention(c)
        self.layer_norm2 = nn.LayerNorm(c.hidden_size, c.layer_norm_eps)
        self.mlp = _ClipMlp(c)

    def forward(self, x):
        x = x + self.self_attn(self.layer_norm1(x))
        return x + self.mlp(self.layer_norm2(x))


class _ClipEmbeddings(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embedding = nn.Embedding(c.max_position_embeddings, c.hidden_size)

    def forward(self, ids):
        return self.token_embedding(ids) + self.position_embedding.weight[: ids.shape[1]]


class _ClipEncoder(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.layers = nn.ModuleList(_ClipLayer(c) for _ in range(c.num_hidden_layers))

    def forward(self, x):
        for layer in self.layers:
            x = layer(x)
        return x


class _ClipTextModel(nn.Module):
    def __init__(self, c: ClipTextConfig):
        super().__init__()
        self.embeddings, self.encoder = _ClipEmbeddings(c), _ClipEncoder(c)
        self.final_layer_norm = nn.LayerNorm(c.hidden_size, c.layer_norm_eps)


class ClipTextEncoder(nn.Module):
    """``input_ids [B, S<=77]`` -> last hidden state ``[B, S, hidden]`` after the final layer norm
    (what the UNet cross-attends to; clip_text_encoder.rs:1031-1100)."""

    def __init__(self, config: ClipTextConfig | None = None):
        super().__init__()
        self.config = config or ClipTextConfig()
        self.config.validate()
        self.text_model = _ClipTextModel(self.config)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        if input_ids.shape[1] > self.config.max_position_embeddings:
            raise ValueError("ClipTextEncoder: %d tokens exceed max_position_embeddings %d"
                             % (input_ids.shape[1], self.config.max_position_embeddings))
        if bool((input_ids < 0).any()) or bool((input_ids >= self.config.vocab_size).any()):
            raise ValueError("ClipTextEncoder: token id outside the vocabulary")
        tm = self.text_model
        return tm.final_layer_norm(tm.encoder(tm.embeddings(input_ids)))

    forward_from_ids = forward

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        """Accepts keys with or without the ``text_model.`` prefix; ``position_ids`` buffers of
        older checkpoints are ignored."""
        sd = {(k if k.startswith("text_model.") else "text_model." + k): v for k, v in sd.items()
              if not k.endswith("position_ids")}
        return self.load_state_dict(sd, strict=strict)


# --------------------------------------------------------------------------- shared blocks
class ResnetBlock2D(nn.Module):
    """GroupNorm-SiLU-conv twice with an optional timestep projection added in between and a 1x1
    shortcut when the width changes (resnet_block_time.rs, blocks.rs)."""

    def __init__(self, cin: int, cout: int, temb: int | None, groups: int = 32, eps: float = 1e-5):
        super().__init__()
        self.norm1 = nn.GroupNorm(groups, cin, eps)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1)
        self.time_emb_proj = nn.Linear(temb, cout) if temb else None
        self.norm2 = nn.GroupNorm(groups, cout, eps)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x, temb=None):
        h = self.conv1(F.silu(self.norm1(x)))
        if self.time_emb_proj is not None and temb is not None:
            h = h + self.time_emb_proj(F.silu(temb))[:, :, None, None]
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.conv_shortcut is None else self.conv_shortcut(x)) + h


class _Attention(nn.Module):
    """Multi-head attention with diffusers' parameter names (``to_q / to_k / to_v / to_out.0``)."""

    def __init__(self, dim: int, ctx_dim: int | None, heads: int, bias: bool = False):
        super().__init__()
        self.heads = heads
        self.to_q = nn.Linear(dim, dim, bias=bias)
        self.to_k = nn.Linear(ctx_dim or dim, dim, bias=bias)
        self.to_v = nn.Linear(ctx_dim or dim, dim, bias=bias)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim)])

    def forward(self, x, ctx=None):
        ctx = x if ctx is None else ctx
        B, S, E = x.shape
        split = lambda t: t.view(B, -1, self.heads, E // self.heads).transpose(1, 2)  # noqa: E731
        o = _sdpa(split(self.to_q(x)), split(self.to_k(ctx)), split(self.to_v(ctx)))
        return self.to_out[0](o.transpose(1, 2).reshape(B, S, E))


class _GEGLU(nn.Module):
    def __init__(self, dim: int, inner: int):
        super().__init__()
        self.proj = nn.Linear(dim, 2 * inner)

    def forward(self, x):
        a, g = self.proj(x).chunk(2, dim=-1)
        return a * F.gelu(g)


class _FeedForward(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.net = nn.ModuleList([_GEGLU(dim, 4 * dim), nn.Dropout(0.0), nn.Linear(4 * dim, dim)])

    def forward(self, x):
        for m in self.net:
            x = m(x)
        return x


class BasicTransformerBlock(nn.Module):
    """Self-attention, cross-attention on the text states, GEGLU feed-forward, each pre-normed."""

    def __init__(self, dim: int, ctx_dim: int, heads: int):
        super().__init__()
        self.norm1, self.attn1 = nn.LayerNorm(dim), _Attention(dim, None, heads)
        self.norm2, self.attn2 = nn.LayerNorm(dim), _Attention(dim, ctx_dim, heads)
        self.norm3, self.ff = nn.LayerNorm(dim), _FeedForward(dim)

    def forward(self, x, ctx):
        x = x + self.attn1(self.norm1(x))
        x = x + self.attn2(self.norm2(x), ctx)
        return x + self.ff(self.norm3(x))


class Transformer2DModel(nn.Module):
    def __init__(self, ch: int, ctx_dim: int, heads: int, groups: int = 32, depth: int = 1):
        super().__init__()
        self.norm = nn.GroupNorm(groups, ch, 1e-6)
        self.proj_in = nn.Conv2d(ch, ch, 1)
        self.transformer_blocks = nn.ModuleList(BasicTransformerBlock(ch, ctx_dim, heads) for _ in range(depth))
        self.proj_out = nn.Conv2d(ch, ch, 1)

    def forward(self, x, ctx):
        B, C, H, W = x.shape
        h = self.proj_in(self.norm(x)).flatten(2).transpose(1, 2)
        for blk in self.transformer_blocks:
            h = blk(h, ctx)
        return x + self.proj_out(h.transpose(1, 2).reshape(B, C, H, W))


class _Down(nn.Module):
    def __init__(self, ch: int, pad: int = 1):
        super().__init__()
        self.conv = nn.Conv2d(ch, ch, 3, stride=2, padding=pad)
        self.asym = pad == 0

    def forward(self, x):
        return self.conv(F.pad(x, (0, 1, 0, 1)) if self.asym else x)


class _Up(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = nn.Conv2d(ch, ch, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


def timestep_embedding(t: torch.Tensor, dim: int, flip_sin_to_cos: bool = True, shift: float = 0.0) -> torch.Tensor:
    """Sinusoidal embedding ``[B, dim]`` with frequencies ``10000^(-i / (dim/2 - shift))``; SD puts
    the cosine half first (time_embedding.rs)."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / (half - shift))
    ang = t.float()[:, None] * freqs[None]
    emb = torch.cat([ang.cos(), ang.sin()] if flip_sin_to_cos else [ang.sin(), ang.cos()], dim=-1)
    return F.pad(emb, (0, 1)) if dim % 2 else emb


# --------------------------------------------------------------------------- conditional UNet
@dataclass
class UNet2DConditionConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_out_channels: tuple = (320, 640, 1280, 1280)
    down_block_types: tuple = ("CrossAttnDownBlock2D", "CrossAttnDownBlock2D", "CrossAttnDownBlock2D", "DownBlock2D")
    up_block_types: tuple = ("UpBlock2D", "CrossAttnUpBlock2D", "CrossAttnUpBlock2D", "CrossAttnUpBlock2D")
    layers_per_block: int = 2
    cross_attention_dim: int = 768
    attention_head_dim: int = 8                 # SD 1.x checkpoints use this field as the number of heads
    norm_num_groups: int = 32
    norm_eps: float = 1e-5
    flip_sin_to_cos: bool = True
    freq_shift: float = 0.0

    @classmethod
    def sd_v1_5(cls) -> "UNet2DConditionConfig":
        return cls()

    def validate(self) -> None:
        n = len(self.block_out_channels)
        if n == 0 or len(self.down_block_types) != n or len(self.up_block_types) != n:
            raise ValueError("UNet2DConditionConfig: block lists must have the same, non-zero length")
        if any(c <= 0 or c % self.norm_num_groups for c in self.block_out_channels):
            raise ValueError("UNet2DConditionConfig: every block width must be a positive multiple of norm_num_groups")
        if any(c % self.attention_head_dim for c in self.block_out_channels):
            raise ValueError("UNet2DConditionConfig: block widths must divide by the number of heads")
        if min(self.in_channels, self.out_channels, self.layers_per_block, self.cross_attention_dim) <= 0:
            raise ValueError("UNet2DConditionConfig: sizes must be positive")
        for t in self.down_block_types:
            if t not in ("CrossAttnDownBlock2D", "DownBlock2D"):
                raise ValueError("unsupported down block %r" % t)
        for t in self.up_block_types:
            if t not in ("CrossAttnUpBlock2D", "UpBlock2D"):
                raise ValueError("unsupported up block %r" % t)

    @classmethod
    def from_json_str(cls, s) -> "UNet2DConditionConfig":
        return _from_json(cls, s)

    from_file = from_json_str


class _TimestepEmbedding(nn.Module):
    def __init__(self, cin: int, dim: int):
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(cin, dim), nn.Linear(dim, dim)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


class _UNetBlock(nn.Module):
    """Down / up block: resnets, optional transformers after each, optional resampler.  For an
    up block ``skips[j]`` is the width of the skip connection that resnet j concatenates."""

    def __init__(self, c: UNet2DConditionConfig, widths: list[tuple[int, int]], temb: int, attn: bool,
                 down: bool = False, up: bool = False):
        super().__init__()
        out = widths[-1][1]
        self.resnets = nn.ModuleList(ResnetBlock2D(a, b, temb, c.norm_num_groups, c.norm_eps) for a, b in widths)
        if attn:
            self.attentions = nn.ModuleList(Transformer2DModel(out, c.cross_attention_dim, c.attention_head_dim,
                                                               c.norm_num_groups) for _ in widths)
        else:
            self.attentions = None
        if down:
            self.downsamplers = nn.ModuleList([_Down(out)])
        if up:
            self.upsamplers = nn.ModuleList([_Up(out)])

    def run(self, j: int, x, temb, ctx):
        x = self.resnets[j](x, temb)
        return self.attentions[j](x, ctx) if self.attentions is not None else x

    def forward_t(self, x, temb, ctx=None, skips=None):
        """A whole block under the reference's calling convention (ferrotorch-diffusion/src/unet.rs:160, 340,
        504, 704).  Down block (``skips is None``): returns ``(output, skips)`` with one skip per resnet and
        the down-sampled tensor as the last one.  Up block: ``skips`` holds one tensor per resnet, the
        **last** one is consumed first (the order in which the down path produced them, reversed)."""
        if skips is None:
            out_skips = []
            for j in range(len(self.resnets)):
                x = self.run(j, x, temb, ctx)
                out_skips.append(x)
            if hasattr(self, "downsamplers"):
                x = self.downsamplers[0](x)
                out_skips.append(x)
            return x, out_skips
        skips = list(skips)
        if len(skips) != len(self.resnets):
            raise ValueError("up block with %d resnets got %d skip tensors" % (len(self.resnets), len(skips)))
        for j in range(len(self.resnets)):
            x = self.run(j, torch.cat([x, skips.pop()], dim=1), temb, ctx)
        if hasattr(self, "upsamplers"):
            x = self.upsamplers[0](x)
        return x


class _UNetMid(nn.Module):
    def __init__(self, c: UNet2DConditionConfig, ch: int, temb: int):
        super().__init__()
        self.resnets = nn.ModuleList(ResnetBlock2D(ch, ch, temb, c.norm_num_groups, c.norm_eps) for _ in range(2))
        self.attentions = nn.ModuleList([Transformer2DModel(ch, c.cross_attention_dim, c.attention_head_dim,
                                                            c.norm_num_groups)])

    def forward(self, x, temb, ctx):
        return self.resnets[1](self.attentions[0](self.resnets[0](x, temb), ctx), temb)

    forward_t = forward


class UNet2DConditionModel(nn.Module):
    """``(latents [B, 4, h, w], timestep, text states [B, S, 768]) -> predicted noise [B, 4, h, w]``
    (unet.rs:1119-1400)."""

    def __init__(self, config: UNet2DConditionConfig | None = None):
        super().__init__()
        c = self.config = config or UNet2DConditionConfig()
        c.validate()
        chans, L = list(c.block_out_channels), c.layers_per_block
        temb = 4 * chans[0]
        self.conv_in = nn.Conv2d(c.in_channels, chans[0], 3, padding=1)
        self.time_embedding = _TimestepEmbedding(chans[0], temb)
        self.down_blocks = nn.ModuleList()
        prev = chans[0]
        for i, (ch, kind) in enumerate(zip(chans, c.down_block_types)):
            widths = [(prev if j == 0 else ch, ch) for j in range(L)]
            self.down_blocks.append(_UNetBlock(c, widths, temb, kind.startswith("CrossAttn"), down=i < len(chans) - 1))
            prev = ch
        self.mid_block = _UNetMid(c, chans[-1], temb)
        self.up_blocks = nn.ModuleList()
        rev = chans[::-1]
        prev = rev[0]
        for i, (ch, kind) in enumerate(zip(rev, c.up_block_types)):
            below = rev[min(i + 1, len(rev) - 1)]
            widths = [((prev if j == 0 else ch) + (below if j == L else ch), ch) for j in range(L + 1)]
            self.up_blocks.append(_UNetBlock(c, widths, temb, kind.startswith("CrossAttn"), up=i < len(rev) - 1))
            prev = ch
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, chans[0], c.norm_eps)
        self.conv_out = nn.Conv2d(chans[0], c.out_channels, 3, padding=1)

    def forward(self, sample: torch.Tensor, timestep, encoder_hidden_states: torch.Tensor) -> torch.Tensor:
        c = self.config
        if sample.shape[1] != c.in_channels:
            raise ValueError("UNet: expected %d latent channels, got %d" % (c.in_channels, sample.shape[1]))
        div = 2 ** (len(c.block_out_channels) - 1)
        if sample.shape[2] % div or sample.shape[3] % div:
            raise ValueError("UNet: latent height and width must be multiples of %d" % div)
        t = torch.as_tensor(timestep, device=sample.device)
        t = t.expand(sample.shape[0]) if t.dim() == 0 else t
        temb = timestep_embedding(t, c.block_out_channels[0], c.flip_sin_to_cos, c.freq_shift).to(sample.dtype)
        temb = self.time_embedding(temb)
        ctx = encoder_hidden_states
        x = self.conv_in(sample)
        skips = [x]
        for blk in self.down_blocks:
            for j in range(len(blk.resnets)):
                x = blk.run(j, x, temb, ctx)
                skips.append(x)
            if hasattr(blk, "downsamplers"):
                x = blk.downsamplers[0](x)
                skips.append(x)
        x = self.mid_block(x, temb, ctx)
        for blk in self.up_blocks:
            for j in range(len(blk.resnets)):
                x = blk.run(j, torch.cat([x, skips.pop()], dim=1), temb, ctx)
            if hasattr(blk, "upsamplers"):
                x = blk.upsamplers[0](x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))

    forward_t = forward

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        """The module's parameter names are the ``diffusers`` names, so this is ``load_state_dict``; kept
        under the name every other model of the stack uses."""
        return self.load_state_dict(sd, strict=strict)


# --------------------------------------------------------------------------- VAE
@dataclass
class VaeConfig:
    in_channels: int = 3
    out_channels: int = 3
    latent_channels: int = 4
    block_out_channels: tuple = (128, 256, 512, 512)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    scaling_factor: float = 0.18215

    @classmethod
    def sd_v1_5(cls) -> "VaeConfig":
        return cls()

    def validate(self) -> None:
        if not self.block_out_channels or any(c <= 0 or c % self.norm_num_groups for c in self.block_out_channels):
            raise ValueError("VaeConfig: every block width must be a positive multiple of norm_num_groups")
        if min(self.in_channels, self.out_channels, self.latent_channels, self.layers_per_block) <= 0 or self.scaling_factor <= 0:
            raise ValueError("VaeConfig: sizes and the scaling factor must be positive")

    def resnets_per_up_block(self) -> int:
        return self.layers_per_block + 1

    def num_up_blocks(self) -> int:
        return len(self.block_out_channels)

    @classmethod
    def from_json_str(cls, s) -> "VaeConfig":
        return _from_json(cls, s)

    from_file = from_json_str


VaeDecoderConfig = VaeEncoderConfig = VaeConfig


class _VaeAttention(nn.Module):
    """Single-head self-attention over the pixels of the middle block."""

    def __init__(self, ch: int, groups: int):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, 1e-6)
        self.to_q, self.to_k, self.to_v = nn.Linear(ch, ch), nn.Linear(ch, ch), nn.Linear(ch, ch)
        self.to_out = nn.ModuleList([nn.Linear(ch, ch)])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).flatten(2).transpose(1, 2)
        o = _sdpa(self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None])[:, 0]
        return x + self.to_out[0](o).transpose(1, 2).reshape(B, C, H, W)


class _VaeMid(nn.Module):
    def __init__(self, ch: int, groups: int):
        super().__init__()
        self.resnets = nn.ModuleList(ResnetBlock2D(ch, ch, None, groups, 1e-6) for _ in range(2))
        self.attentions = nn.ModuleList([_VaeAttention(ch, groups)])

    def forward(self, x):
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class _VaeStage(nn.Module):
    def __init__(self, widths, groups: int, down: bool = False, up: bool = False):
        super().__init__()
        self.resnets = nn.ModuleList(ResnetBlock2D(a, b, None, groups, 1e-6) for a, b in widths)
        if down:
            self.downsamplers = nn.ModuleList([_Down(widths[-1][1], pad=0)])
        if up:
            self.upsamplers = nn.ModuleList([_Up(widths[-1][1])])

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if hasattr(self, "downsamplers"):
            x = self.downsamplers[0](x)
        if hasattr(self, "upsamplers"):
            x = self.upsamplers[0](x)
        return x


class Encoder(nn.Module):
    """Image ``[B, 3, H, W]`` -> moments ``[B, 2 * latent, H/8, W/8]`` (vae_encoder.rs:64-300)."""

    def __init__(self, c: VaeConfig):
        super().__init__()
        ch, n = list(c.block_out_channels), len(c.block_out_channels)
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.down_blocks = nn.ModuleList()
        prev = ch[0]
        for i, w in enumerate(ch):
            self.down_blocks.append(_VaeStage([(prev if j == 0 else w, w) for j in range(c.layers_per_block)],
                                              c.norm_num_groups, down=i < n - 1))
            prev = w
        self.mid_block = _VaeMid(ch[-1], c.norm_num_groups)
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, ch[-1], 1e-6)
        self.conv_out = nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class Decoder(nn.Module):
    """Latent ``[B, latent, h, w]`` -> image ``[B, 3, 8h, 8w]`` (vae.rs:41-260)."""

    def __init__(self, c: VaeConfig):
        super().__init__()
        rev, n = list(c.block_out_channels)[::-1], len(c.block_out_channels)
        self.conv_in = nn.Conv2d(c.latent_channels, rev[0], 3, padding=1)
        self.mid_block = _VaeMid(rev[0], c.norm_num_groups)
        self.up_blocks = nn.ModuleList()
        prev = rev[0]
        for i, w in enumerate(rev):
            self.up_blocks.append(_VaeStage([(prev if j == 0 else w, w) for j in range(c.layers_per_block + 1)],
                                            c.norm_num_groups, up=i < n - 1))
            prev = w
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, rev[-1], 1e-6)
        self.conv_out = nn.Conv2d(rev[-1], c.out_channels, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class DiagonalGaussianDistribution:
    """Posterior of the encoder: mean and log-variance halves of the moments, log-variance clamped
    to [-30, 20] (vae_encoder.rs:467-560)."""

    def __init__(self, mean: torch.Tensor, logvar: torch.Tensor):
        self.mean, self.logvar = mean, logvar.clamp(-30.0, 20.0)
        self.std = torch.exp(0.5 * self.logvar)

    @classmethod
    def from_parameters(cls, params: torch.Tensor, latent_channels: int) -> "DiagonalGaussianDistribution":
        if params.dim() != 4 or params.shape[1] != 2 * latent_channels:
            raise ValueError("expected moments [B, %d, h, w], got %s" % (2 * latent_channels, tuple(params.shape)))
        return cls(*params.chunk(2, dim=1))

    def mode(self) -> torch.Tensor:
        return self.mean

    def sample_with_seed(self, seed: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(seed)
        noise = torch.randn(self.mean.shape, generator=g, dtype=torch.float32)
        return self.mean + self.std * noise.to(self.mean.device, self.mean.dtype)

    def kl(self) -> torch.Tensor:
        return 0.5 * (self.mean ** 2 + self.logvar.exp() - 1.0 - self.logvar).flatten(1).sum(1)


_OLD_VAE_ATTN = {"query": "to_q", "key": "to_k", "value": "to_v", "proj_attn": "to_out.0"}


class AutoencoderKL(nn.Module):
    """``encode`` / ``decode`` with the latent scaling factor of the pipeline (0.18215 for SD 1.5).
    ``VaeEncoder`` / ``VaeDecoder`` of the reference are the two halves of this module."""

    def __init__(self, config: VaeConfig | None = None):
        super().__init__()
        c = self.config = config or VaeConfig()
        c.validate()
        self.encoder, self.decoder = Encoder(c), Decoder(c)
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1)
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1)

    def encode(self, image: torch.Tensor) -> DiagonalGaussianDistribution:
        f = 2 ** (len(self.config.block_out_channels) - 1)
        if image.dim() != 4 or image.shape[1] != self.config.in_channels or image.shape[2] % f or image.shape[3] % f:
            raise ValueError("encode: expected [B, %d, H, W] with H and W multiples of %d" % (self.config.in_channels, f))
        return DiagonalGaussianDistribution.from_parameters(self.quant_conv(self.encoder(image)), self.config.latent_channels)

    def encode_with_scaling(self, image: torch.Tensor, seed: int) -> torch.Tensor:
        return self.encode(image).sample_with_seed(seed) * self.config.scaling_factor

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        return self.decoder(self.post_quant_conv(z))

    def decode_with_scaling(self, latent: torch.Tensor) -> torch.Tensor:
        return self.decode(latent / self.config.scaling_factor)

    def load_hf_state_dict(self, sd: dict, strict: bool = True):
        """Also accepts the attention names of older checkpoints (``query / key / value /
        proj_attn``, stored as 1x1 convolutions)."""
        out = {}
        for k, v in sd.items():
            parts = k.split(".")
            if "attentions" in parts:
                for old, new in _OLD_VAE_ATTN.items():
                    if parts[-2] == old:
                        k = ".".join(parts[:-2] + [new, parts[-1]])
                        if v.dim() == 4:
                            v = v[:, :, 0, 0]
            out[k] = v
        return self.load_state_dict(out, strict=strict)


# --------------------------------------------------------------------------- pipeline
@dataclass
class PipelineStepDump:
    """What one denoising step saw and produced (pipeline.rs:48-66), for parity debugging."""
    step: int
    timestep: int
    noise_pred_uncond: torch.Tensor
    noise_pred_cond: torch.Tensor
    guided_noise: torch.Tensor
    latent_after_step: torch.Tensor


class StableDiffusionPipeline:
    """Text states -> latents -> image with classifier-free guidance:
    ``eps = eps_uncond + g * (eps_cond - eps_uncond)``; both branches run as one batch of the UNet
    (pipeline.rs:69-330)."""

    def __init__(self, text_encoder: ClipTextEncoder, unet: UNet2DConditionModel, vae: AutoencoderKL,
                 scheduler: DDIMScheduler | None = None):
        self.text_encoder, self.unet, self.vae = text_encoder, unet, vae
        self.scheduler = scheduler or DDIMScheduler()

    @torch.no_grad()
    def encode_prompt(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.text_encoder(input_ids)

    @torch.no_grad()
    def generate(self, cond_embeds: torch.Tensor, uncond_embeds: torch.Tensor, init_latent: torch.Tensor,
                 num_inference_steps: int = 50, guidance_scale: float = 7.5, dump: bool = False):
        """Returns ``(image [B, 3, 8h, 8w], dumps)``; the image is the decoder's raw output in
        roughly [-1, 1] (:func:`to_uint8` maps it to pixels)."""
        if init_latent.dim() != 4:
            raise ValueError("generate: expected init_latent [B, C, h, w], got %s" % (tuple(init_latent.shape),))
        if cond_embeds.shape != uncond_embeds.shape:
            raise ValueError("generate: cond_embeds shape %s != uncond_embeds %s"
                             % (tuple(cond_embeds.shape), tuple(uncond_embeds.shape)))
        if cond_embeds.shape[0] != init_latent.shape[0]:
            raise ValueError("generate: %d prompts for %d latents" % (cond_embeds.shape[0], init_latent.shape[0]))
        sch = self.scheduler
        latent = init_latent * sch.init_noise_sigma()
        ctx = torch.cat([uncond_embeds, cond_embeds], dim=0)
        dumps = []
        for i, t in enumerate(sch.set_timesteps(num_inference_steps)):
            inp = sch.scale_model_input(torch.cat([latent, latent], dim=0), t)
            eps_u, eps_c = self.unet(inp, t, ctx).chunk(2, dim=0)
            eps = eps_u + guidance_scale * (eps_c - eps_u)
            latent = sch.step(eps, t, latent)
            if dump:
                dumps.append(PipelineStepDump(i, t, eps_u.clone(), eps_c.clone(), eps.clone(), latent.clone()))
        return self.vae.decode_with_scaling(latent), dumps

    @torch.no_grad()
    def __call__(self, prompt_ids: torch.Tensor, negative_ids: torch.Tensor | None = None, height: int = 512,
                 width: int = 512, num_inference_steps: int = 50, guidance_scale: float = 7.5, seed: int = 0):
        """Token ids in, image out.  Without ``negative_ids`` the unconditional branch sees the
        prompt with every token after the first replaced by the last id of the row (the padding
        convention of CLIP tokenisers: begin-of-text, then end-of-text padding)."""
        if prompt_ids.dim() == 1:
            prompt_ids = prompt_ids[None]
        if height % 8 or width % 8:
            raise ValueError("height and width must be multiples of 8")
        if negative_ids is None:
            negative_ids = prompt_ids.clone()
            negative_ids[:, 1:] = prompt_ids[:, -1:]
        p = next(self.unet.parameters())
        g = torch.Generator().manual_seed(seed)
        c = self.unet.config.in_channels
        noise = torch.randn((prompt_ids.shape[0], c, height // 8, width // 8), generator=g).to(p.device, p.dtype)
        image, _ = self.generate(self.encode_prompt(prompt_ids), self.encode_prompt(negative_ids), noise,
                                 num_inference_steps, guidance_scale)
        return image


def to_uint8(image: torch.Tensor) -> torch.Tensor:
    """Decoder output ``[B, 3, H, W]`` in [-1, 1] -> ``[B, H, W, 3]`` bytes."""
    return ((image.float() / 2 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).permute(0, 2, 3, 1).contiguous()


def load_stable_diffusion(path: str, dtype: torch.dtype = torch.float32, device="cpu") -> StableDiffusionPipeline:
    """Assemble the pipeline from a diffusers-style model directory::

        text_encoder/config.json + model.safetensors
        unet/config.json         + diffusion_pytorch_model.safetensors
        vae/config.json          + diffusion_pytorch_model.safetensors
        scheduler/scheduler_config.json          (optional)

    (ferrotorch-diffusion/src/safetensors_loader.rs reads the same three weight files.)"""
    import os

    from ..serialize.state import load_safetensors

    def part(sub, names):
        for n in names:
            p = os.path.join(path, sub, n)
            if os.path.exists(p):
                return p
        raise FileNotFoundError("no %s under %s" % (" / ".join(names), os.path.join(path, sub)))

    def cfg(cls, sub, rename=None):
        p = os.path.join(path, sub, "config.json")
        return _from_json(cls, p, rename) if os.path.exists(p) else cls()

    clip = ClipTextEncoder(cfg(ClipTextConfig, "text_encoder"))
    clip.load_hf_state_dict(load_safetensors(part("text_encoder", ["model.safetensors"])))
    unet = UNet2DConditionModel(cfg(UNet2DConditionConfig, "unet"))
    unet.load_state_dict(load_safetensors(part("unet", ["diffusion_pytorch_model.safetensors", "model.safetensors"])))
    vae = AutoencoderKL(cfg(VaeConfig, "vae"))
    vae.load_hf_state_dict(load_safetensors(part("vae", ["diffusion_pytorch_model.safetensors", "model.safetensors"])))
    sched_cfg = DDIMConfig()
    sp = os.path.join(path, "scheduler", "scheduler_config.json")
    if os.path.exists(sp):
        with open(sp) as f:
            raw = json.load(f)
        sched_cfg = DDIMConfig(**{k: raw[k] for k in DDIMConfig.__dataclass_fields__ if k in raw})
    for m in (clip, unet, vae):
        m.to(device=device, dtype=dtype).eval()
    return StableDiffusionPipeline(clip, unet, vae, DDIMScheduler(sched_cfg))


def save_stable_diffusion(pipe: StableDiffusionPipeline, path: str) -> None:
    """Write the directory layout :func:`load_stable_diffusion` reads."""
    import os
    from dataclasses import asdict

    from ..serialize.state import save_safetensors

    for sub, module, fname in (("text_encoder", pipe.text_encoder, "model.safetensors"),
                               ("unet", pipe.unet, "diffusion_pytorch_model.safetensors"),
                               ("vae", pipe.vae, "diffusion_pytorch_model.safetensors")):
        os.makedirs(os.path.join(path, sub), exist_ok=True)
        with open(os.path.join(path, sub, "config.json"), "w") as f:
            json.dump({k: (list(v) if isinstance(v, tuple) else v) for k, v in asdict(module.config).items()}, f, indent=2)
        save_safetensors(module.state_dict(), os.path.join(path, sub, fname))
    os.makedirs(os.path.join(path, "scheduler"), exist_ok=True)
    with open(os.path.join(path, "scheduler", "scheduler_config.json"), "w") as f:
        json.dump(asdict(pipe.scheduler.config), f, indent=2)


# --------------------------------------------------------------------------- the reference's block and loader names
import enum as _enum  # noqa: E402

from .pretrained import DropReport  # noqa: E402,F401  (what a partial load reports: loaded / dropped / missing keys)

Attention, FeedForward, AttnBlock2D = _Attention, _FeedForward, _VaeAttention
ClipSelfAttention, ClipMlp, ClipEncoderLayer, ClipTextEmbeddings, ClipEncoder = (_ClipAttention, _ClipMlp, _ClipLayer,
                                                                                  _ClipEmbeddings, _ClipEncoder)
TimestepEmbedding, ResnetBlock2DTime = _TimestepEmbedding, ResnetBlock2D
Downsample2D, Upsample2D = _Down, _Up
# one block class covers the plain and the cross-attention variants (``attn`` switches the transformer on)
DownBlock2D = CrossAttnDownBlock2D = UpBlock2D = CrossAttnUpBlock2D = AnyDownBlock = AnyUpBlock = _UNetBlock
UNetMidBlock2DCrossAttn = UNetMidBlock2D = _UNetMid
DownEncoderBlock2D = UpDecoderBlock2D = _VaeStage
VaeEncoder, VaeDecoder = Encoder, Decoder
# multi-argument forwards under the reference's names (its one-argument ``Module::forward`` needed a second
# entry point for time embeddings / cross-attention context; ``forward`` takes them all here)
ResnetBlock2D.forward_t = ResnetBlock2D.forward
for _c in (_Attention, BasicTransformerBlock, Transformer2DModel):
    _c.forward_xattn = _c.forward
ClipTextEncoder.forward_from_id_tensor = ClipTextEncoder.forward
ClipTextEncoder.forward_from_ids = lambda self, ids: self.forward(torch.as_tensor(list(ids), dtype=torch.long)[None].to(
    next(self.parameters()).device))
_ClipEmbeddings.forward_from_ids = lambda self, ids: self.forward(torch.as_tensor(list(ids), dtype=torch.long)[None].to(
    next(self.parameters()).device))
UNet2DConditionConfig.num_blocks = lambda self: len(self.block_out_channels)
UNet2DConditionConfig.time_embed_dim = lambda self: 4 * self.block_out_channels[0]


class Timesteps(nn.Module):
    """Sinusoidal timestep features (the function :func:`timestep_embedding` as a module)."""

    def __init__(self, dim: int, flip_sin_to_cos: bool = True, shift: float = 0.0):
        super().__init__()
        self.dim, self.flip, self.shift = dim, flip_sin_to_cos, shift

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        return timestep_embedding(t, self.dim, self.flip, self.shift)

    forward_t = forward


class BetaSchedule(str, _enum.Enum):
    Linear = "linear"
    ScaledLinear = "scaled_linear"
    SquaredCosCapV2 = "squaredcos_cap_v2"

    def __str__(self) -> str:
        return self.value


class PredictionType(str, _enum.Enum):
    Epsilon = "epsilon"
    VPrediction = "v_prediction"
    Sample = "sample"

    def __str__(self) -> str:
        return self.value


class TimestepSpacing(str, _enum.Enum):
    Leading = "leading"
    Trailing = "trailing"
    Linspace = "linspace"

    def __str__(self) -> str:
        return self.value


def _load_part(cls_model, cls_cfg, path: str, weight_names, hf: bool, dtype, device, pick=None):
    import os

    from ..serialize.state import load_safetensors

    cfg_path = os.path.join(path, "config.json")
    model = cls_model(_from_json(cls_cfg, cfg_path) if os.path.exists(cfg_path) else cls_cfg())
    for n in weight_names:
        p = os.path.join(path, n)
        if os.path.exists(p):
            sd = load_safetensors(p)
            model.load_hf_state_dict(sd) if hf else model.load_state_dict(sd)
            break
    else:
        raise FileNotFoundError("no %s under %s" % (" / ".join(weight_names), path))
    model.to(device=device, dtype=dtype).eval()
    return pick(model) if pick else model


_W = ("diffusion_pytorch_model.safetensors", "model.safetensors")


def load_clip_text_encoder(path: str, dtype=torch.float32, device="cpu") -> ClipTextEncoder:
    """``path``: a directory with ``config.json`` and ``model.safetensors`` (a pipeline's ``text_encoder/``)."""
    return _load_part(ClipTextEncoder, ClipTextConfig, path, ("model.safetensors",), True, dtype, device)


def load_unet(path: str, dtype=torch.float32, device="cpu") -> UNet2DConditionModel:
    return _load_part(UNet2DConditionModel, UNet2DConditionConfig, path, _W, False, dtype, device)


def load_vae_decoder(path: str, dtype=torch.float32, device="cpu") -> Decoder:
    return _load_part(AutoencoderKL, VaeConfig, path, _W, True, dtype, device, pick=lambda m: m.decoder)


def load_vae_encoder(path: str, dtype=torch.float32, device="cpu") -> Encoder:
    return _load_part(AutoencoderKL, VaeConfig, path, _W, True, dtype, device, pick=lambda m: m.encoder)
