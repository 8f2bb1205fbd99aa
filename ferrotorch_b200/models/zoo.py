"""Small model families of the reference's zoo, built on torch.nn and this package's layers:
BERT encoder + sentence embeddings (ferrotorch-bert/src/model.rs), Whisper encoder + log-mel
front end (ferrotorch-whisper/src/encoder.rs, audio.rs), GCN (ferrotorch-graph/src/gcn.rs), the
SB3-style PPO ``MlpPolicy`` (ferrotorch-rl/src/mlp_policy.rs) and the diffusion pieces -- DDIM
scheduler + a small conditional UNet (ferrotorch-diffusion/src/{pipeline,unet}.rs)."""
from __future__ import annotations

import math

import torch
from torch import nn


# --------------------------------------------------------------------------- BERT
class BertModel(nn.Module):
    def __init__(self, vocab_size=30522, hidden=768, layers=12, heads=12, intermediate=3072, max_pos=512,
                 type_vocab=2, eps=1e-12, dropout=0.0):
        super().__init__()
        self.word = nn.Embedding(vocab_size, hidden)
        self.pos = nn.Embedding(max_pos, hidden)
        self.token_type = nn.Embedding(type_vocab, hidden)
        self.norm = nn.LayerNorm(hidden, eps=eps)
        layer = nn.TransformerEncoderLayer(hidden, heads, intermediate, dropout, activation="gelu", batch_first=True,
                                           layer_norm_eps=eps)
        self.encoder = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
        self.pooler = nn.Linear(hidden, hidden)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        B, S = input_ids.shape
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = self.word(input_ids) + self.pos(torch.arange(S, device=input_ids.device))[None] + self.token_type(tt)
        pad = (attention_mask == 0) if attention_mask is not None else None
        h = self.encoder(self.norm(x), src_key_padding_mask=pad)
        return h, torch.tanh(self.pooler(h[:, 0]))


class SentenceTransformer(nn.Module):
    """Mean-pooled, L2-normalised sentence embeddings over a BERT encoder."""

    def __init__(self, bert: BertModel):
        super().__init__()
        self.bert = bert

    def forward(self, input_ids, attention_mask=None):
        h, _ = self.bert(input_ids, attention_mask)
        m = (attention_mask if attention_mask is not None else torch.ones_like(input_ids)).unsqueeze(-1).to(h.dtype)
        return nn.functional.normalize((h * m).sum(1) / m.sum(1).clamp_min(1e-9), dim=-1)


# --------------------------------------------------------------------------- Whisper encoder
def log_mel_spectrogram(audio: torch.Tensor, n_mels: int = 80, n_fft: int = 400, hop: int = 160,
                        sample_rate: int = 16000) -> torch.Tensor:
    """``audio [..., T]`` -> ``[..., n_mels, frames]`` log-mel features with Whisper's clamping / scaling."""
    win = torch.hann_window(n_fft, device=audio.device)
    spec = torch.stft(audio, n_fft, hop, window=win, return_complex=True)[..., :-1].abs() ** 2
    f = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1, device=audio.device)
    mel = lambda hz: 2595.0 * torch.log10(1.0 + hz / 700.0)  # noqa: E731
    pts = 700.0 * (10 ** (torch.linspace(float(mel(torch.tensor(0.0))), float(mel(torch.tensor(sample_rate / 2.0))),
                                         n_mels + 2, device=audio.device) / 2595.0) - 1.0)
    lo, ce, hi = pts[:-2, None], pts[1:-1, None], pts[2:, None]
    fb = torch.clamp(torch.minimum((f[None] - lo) / (ce - lo), (hi - f[None]) / (hi - ce)), min=0.0)
    logmel = torch.log10((fb @ spec).clamp_min(1e-10))
    logmel = torch.maximum(logmel, logmel.amax(dim=(-2, -1), keepdim=True) - 8.0)
    return (logmel + 4.0) / 4.0


class WhisperEncoder(nn.Module):
    def __init__(self, n_mels=80, d_model=384, heads=6, layers=4, n_ctx=1500):
        super().__init__()
        self.conv1 = nn.Conv1d(n_mels, d_model, 3, padding=1)
        self.conv2 = nn.Conv1d(d_model, d_model, 3, stride=2, padding=1)
        half = d_model // 2
        inv = torch.exp(-math.log(10000.0) / (half - 1) * torch.arange(half))
        ang = torch.arange(n_ctx)[:, None] * inv[None]
        self.register_buffer("pos", torch.cat([ang.sin(), ang.cos()], 1), persistent=False)
        layer = nn.TransformerEncoderLayer(d_model, heads, 4 * d_model, 0.0, activation="gelu", batch_first=True,
                                           norm_first=True)
        self.blocks = nn.TransformerEncoder(layer, layers, enable_nested_tensor=False)
        self.ln_post = nn.LayerNorm(d_model)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        x = nn.functional.gelu(self.conv2(nn.functional.gelu(self.conv1(mel)))).transpose(1, 2)
        return self.ln_post(self.blocks(x + self.pos[: x.shape[1]].to(x.dtype)))


# --------------------------------------------------------------------------- GCN
class GcnConv(nn.Module):
    """``D^-1/2 (A + I) D^-1/2 X W`` on a dense or sparse adjacency."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.lin = nn.Linear(in_features, out_features, bias=bias)

    @staticmethod
    def normalize(adj: torch.Tensor) -> torch.Tensor:
        a = adj.to_dense() if adj.is_sparse else adj
        a = a + torch.eye(a.shape[0], device=a.device, dtype=a.dtype)
        d = a.sum(1).pow(-0.5)
        return d[:, None] * a * d[None]

    def forward(self, x: torch.Tensor, adj_norm: torch.Tensor) -> torch.Tensor:
        return adj_norm @ self.lin(x)


class Gcn(nn.Module):
    def __init__(self, in_features, hidden, classes, dropout=0.5):
        super().__init__()
        self.c1, self.c2, self.drop = GcnConv(in_features, hidden), GcnConv(hidden, classes), nn.Dropout(dropout)

    def forward(self, x, adj_norm):
        return self.c2(self.drop(torch.relu(self.c1(x, adj_norm))), adj_norm)


# --------------------------------------------------------------------------- PPO policy
class MlpPolicy(nn.Module):
    """Separate actor / critic MLPs with tanh, state-independent log-std for Box actions or a
    categorical head for Discrete ones."""

    def __init__(self, obs_dim: int, act_dim: int, discrete: bool = False, hidden=(64, 64)):
        super().__init__()

        def mlp(out):
            dims, layers = (obs_dim,) + tuple(hidden), []
            for a, b in zip(dims[:-1], dims[1:]):
                layers += [nn.Linear(a, b), nn.Tanh()]
            return nn.Sequential(*layers, nn.Linear(dims[-1], out))

        self.actor, self.critic, self.discrete = mlp(act_dim), mlp(1), discrete
        self.log_std = None if discrete else nn.Parameter(torch.zeros(act_dim))

    def distribution(self, obs):
        out = self.actor(obs)
        if self.discrete:
            return torch.distributions.Categorical(logits=out)
        return torch.distributions.Independent(torch.distributions.Normal(out, self.log_std.exp()), 1)

    def forward(self, obs, deterministic: bool = False):
        dist = self.distribution(obs)
        if deterministic:
            act = dist.probs.argmax(-1) if self.discrete else dist.mean
        else:
            act = dist.sample()
        return act, self.critic(obs).squeeze(-1), dist.log_prob(act)

    def evaluate_actions(self, obs, actions):
        dist = self.distribution(obs)
        return self.critic(obs).squeeze(-1), dist.log_prob(actions), dist.entropy()


def ppo_loss(policy: MlpPolicy, obs, actions, old_log_prob, advantages, returns, clip=0.2, vf_coef=0.5, ent_coef=0.0):
    values, log_prob, entropy = policy.evaluate_actions(obs, actions)
    ratio = (log_prob - old_log_prob).exp()
    pg = -torch.min(ratio * advantages, ratio.clamp(1 - clip, 1 + clip) * advantages).mean()
    return pg + vf_coef * nn.functional.mse_loss(values, returns) - ent_coef * entropy.mean()


# --------------------------------------------------------------------------- diffusion
class DDIMScheduler:
    def __init__(self, num_train_timesteps=1000, beta_start=0.00085, beta_end=0.012):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_timesteps) ** 2
        self.alphas_cumprod = torch.cumprod(1.0 - betas, 0)
        self.num_train_timesteps = num_train_timesteps

    def set_timesteps(self, n: int):
        step = self.num_train_timesteps // n
        self.timesteps = (torch.arange(n) * step).flip(0)
        self._step = step

    def add_noise(self, x0, noise, t):
        a = self.alphas_cumprod[t].view(-1, *[1] * (x0.dim() - 1)).to(x0)
        return a.sqrt() * x0 + (1 - a).sqrt() * noise

    def step(self, eps, t: int, x):
        a_t = self.alphas_cumprod[t]
        prev = t - self._step
        a_prev = self.alphas_cumprod[prev] if prev >= 0 else torch.tensor(1.0)
        x0 = (x - (1 - a_t).sqrt() * eps) / a_t.sqrt()
        return a_prev.sqrt() * x0 + (1 - a_prev).sqrt() * eps


class TinyUNet(nn.Module):
    """A two-level conditional UNet (timestep embedding + optional cross-attention context)."""

    def __init__(self, channels=4, base=32, ctx_dim: int | None = None):
        super().__init__()
        self.t_mlp = nn.Sequential(nn.Linear(base, base * 4), nn.SiLU(), nn.Linear(base * 4, base * 2))
        self.inc = nn.Conv2d(channels, base, 3, padding=1)
        self.down = nn.Conv2d(base, base * 2, 3, stride=2, padding=1)
        self.mid = nn.Sequential(nn.GroupNorm(8, base * 2), nn.SiLU(), nn.Conv2d(base * 2, base * 2, 3, padding=1))
        self.attn = nn.MultiheadAttention(base * 2, 4, kdim=ctx_dim, vdim=ctx_dim, batch_first=True) if ctx_dim else None
        self.up = nn.ConvTranspose2d(base * 2, base, 4, stride=2, padding=1)
        self.out = nn.Sequential(nn.GroupNorm(8, base * 2), nn.SiLU(), nn.Conv2d(base * 2, channels, 3, padding=1))
        self.base = base

    def forward(self, x, t, context=None):
        half = self.base // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=x.device) / half)
        emb = torch.cat([(t[:, None].float() * freqs).sin(), (t[:, None].float() * freqs).cos()], 1)
        temb = self.t_mlp(emb)[:, :, None, None]
        h0 = self.inc(x)
        h = self.mid(self.down(h0) + temb)
        if self.attn is not None and context is not None:
            B, C, H, W = h.shape
            seq = h.flatten(2).transpose(1, 2)
            h = (seq + self.attn(seq, context, context)[0]).transpose(1, 2).view(B, C, H, W)
        return self.out(torch.cat([self.up(h), h0], 1))


@torch.no_grad()
def ddim_sample(unet: TinyUNet, scheduler: DDIMScheduler, shape, steps=10, context=None, generator=None):
    x = torch.randn(shape, generator=generator)
    scheduler.set_timesteps(steps)
    for t in scheduler.timesteps.tolist():
        x = scheduler.step(unet(x, torch.full((shape[0],), t), context), t, x)
    return x
