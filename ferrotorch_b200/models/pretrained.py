"""Checkpoint-compatible small models: BERT encoder + sentence embeddings, Whisper audio encoder,
a two-layer GCN and the Stable-Baselines3 PPO ``MlpPolicy``.

Each class keeps the parameter names of the checkpoints the reference's loaders read
(ferrotorch-bert/src/{model,safetensors_loader}.rs: Hugging Face BERT, e.g.
``sentence-transformers/all-MiniLM-L6-v2``; ferrotorch-whisper/src/{encoder,safetensors_loader}.rs:
``openai/whisper-tiny``'s ``model.encoder.*``; ferrotorch-graph/src/{gcn,safetensors_loader}.rs:
PyTorch-Geometric ``GCNConv``; ferrotorch-rl/src/{mlp_policy,safetensors_loader}.rs: SB3 PPO), so
a SafeTensors / ``.pt`` state dict of those loads with ``load_hf_state_dict``; keys that do not
belong to the module (decoder weights, optimizer slots, ``position_ids`` buffers) are reported in a
:class:`DropReport` instead of failing.  ``models.zoo`` holds lighter, free-form variants.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch import nn


@dataclass
class DropReport:
    """Keys of a checkpoint that were not used, and parameters it did not provide."""
    dropped: list = field(default_factory=list)
    missing: list = field(default_factory=list)


def _load(module: nn.Module, sd: dict, strip: tuple = (), strict: bool = True) -> DropReport:
    own = module.state_dict()
    use, rep = {}, DropReport()
    for k, v in sd.items():
        for p in strip:
            if k.startswith(p):
                k = k[len(p):]
                break
        if k in own:
            if tuple(v.shape) != tuple(own[k].shape):
                raise ValueError("%s: checkpoint shape %s, module shape %s" % (k, tuple(v.shape), tuple(own[k].shape)))
            use[k] = v
        else:
            rep.dropped.append(k)
    rep.missing = [k for k in own if k not in use]
    if strict and rep.missing:
        raise KeyError("checkpoint lacks %d parameters, e.g. %s" % (len(rep.missing), rep.missing[:3]))
    module.load_state_dict(use, strict=False)
    return rep


def _json(src) -> dict:
    if isinstance(src, dict):
        return src
    try:
        return json.loads(src)
    except ValueError:
        with open(src) as f:
            return json.load(f)


# --------------------------------------------------------------------------- BERT
@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 384
    num_hidden_layers: int = 6
    num_attention_heads: int = 12
    intermediate_size: int = 1536
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"

    @classmethod
    def all_minilm_l6_v2(cls) -> "BertConfig":
        return cls()

    @classmethod
    def bert_base(cls) -> "BertConfig":
        return cls(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072)

    @classmethod
    def from_hf(cls, src) -> "BertConfig":
        raw = _json(src)
        need = ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size")
        missing = [k for k in need if k not in raw]
        if missing:
            raise ValueError("BertConfig: config lacks %s" % ", ".join(missing))
        cfg = cls(**{k: raw[k] for k in cls.__dataclass_fields__ if raw.get(k) is not None})
        cfg.validate()
        return cfg

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        if min(self.vocab_size, self.hidden_size, self.num_hidden_layers, self.num_attention_heads,
               self.intermediate_size, self.max_position_embeddings, self.type_vocab_size) <= 0:
            raise ValueError("BertConfig: sizes must be positive")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("BertConfig: hidden_size (%d) must be divisible by num_attention_heads (%d)"
                             % (self.hidden_size, self.num_attention_heads))
        if self.hidden_act not in ("gelu", "relu", "gelu_new"):
            raise ValueError("BertConfig: unsupported hidden_act %r" % self.hidden_act)


def _act(name: str):
    return {"gelu": F.gelu, "relu": F.relu, "gelu_new": lambda x: F.gelu(x, approximate="tanh")}[name]


class BertEmbeddings(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embeddings = nn.Embedding(c.max_position_embeddings, c.hidden_size)
        self.token_type_embeddings = nn.Embedding(c.type_vocab_size, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, c.layer_norm_eps)

    def forward(self, ids, token_type_ids=None):
        S = ids.shape[1]
        tt = torch.zeros_like(ids) if token_type_ids is None else token_type_ids
        x = self.word_embeddings(ids) + self.position_embeddings.weight[:S] + self.token_type_embeddings(tt)
        return self.LayerNorm(x)


class BertSelfAttention(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.h = c.num_attention_heads
        self.query, self.key, self.value = (nn.Linear(c.hidden_size, c.hidden_size) for _ in range(3))

    def forward(self, x, mask):
        B, S, E = x.shape
        q, k, v = (p(x).view(B, S, self.h, E // self.h).transpose(1, 2) for p in (self.query, self.key, self.value))
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask).transpose(1, 2).reshape(B, S, E)


class BertSelfOutput(nn.Module):
    def __init__(self, c: BertConfig, cin: int | None = None):
        super().__init__()
        self.dense = nn.Linear(cin or c.hidden_size, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, c.layer_norm_eps)

    def forward(self, h, residual):
        return self.LayerNorm(self.dense(h) + residual)


class BertAttention(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.self, self.output = BertSelfAttention(c), BertSelfOutput(c)

    def forward(self, x, mask):
        return self.output(self.self(x, mask), x)


class BertIntermediate(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.dense, self.act = nn.Linear(c.hidden_size, c.intermediate_size), _act(c.hidden_act)

    def forward(self, x):
        return self.act(self.dense(x))


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.attention, self.intermediate = BertAttention(c), BertIntermediate(c)
        self.output = BertSelfOutput(c, c.intermediate_size)

    def forward(self, x, mask):
        x = self.attention(x, mask)
        return self.output(self.intermediate(x), x)


class BertEncoder(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.layer = nn.ModuleList(BertLayer(c) for _ in range(c.num_hidden_layers))

    def forward(self, x, mask):
        for blk in self.layer:
            x = blk(x, mask)
        return x


class BertPooler(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.dense = nn.Linear(c.hidden_size, c.hidden_size)

    def forward(self, h):
        return torch.tanh(self.dense(h[:, 0]))


class BertModel(nn.Module):
    """Post-norm encoder; ``forward`` returns ``(last_hidden_state [B, S, H], pooled [B, H])``."""

    def __init__(self, config: BertConfig | None = None):
        super().__init__()
        self.config = config or BertConfig()
        self.config.validate()
        self.embeddings, self.encoder, self.pooler = BertEmbeddings(self.config), BertEncoder(self.config), BertPooler(self.config)

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        if input_ids.shape[1] > self.config.max_position_embeddings:
            raise ValueError("BertModel: %d tokens exceed max_position_embeddings %d"
                             % (input_ids.shape[1], self.config.max_position_embeddings))
        mask = None
        if attention_mask is not None:
            mask = attention_mask[:, None, None, :].bool()         # keys that are padding are not attended to
        h = self.encoder(self.embeddings(input_ids, token_type_ids), mask)
        return h, self.pooler(h)

    forward_from_ids = forward

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> DropReport:
        return _load(self, sd, strip=("bert.", "0.auto_model."), strict=strict)


class SentenceTransformer(nn.Module):
    """Mean pooling over the attended tokens (+ L2 normalisation): the sentence-transformers recipe
    of all-MiniLM-L6-v2 (model.rs:384-470)."""

    def __init__(self, config: BertConfig | None = None, normalize: bool = True):
        super().__init__()
        self.bert, self.normalize = BertModel(config), normalize

    def encode(self, input_ids, attention_mask=None):
        h, _ = self.bert(input_ids, attention_mask)
        m = (torch.ones_like(input_ids) if attention_mask is None else attention_mask).unsqueeze(-1).to(h.dtype)
        e = (h * m).sum(1) / m.sum(1).clamp_min(1e-9)
        return F.normalize(e, dim=-1) if self.normalize else e

    forward = encode

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> DropReport:
        return self.bert.load_hf_state_dict(sd, strict)


# --------------------------------------------------------------------------- Whisper encoder
@dataclass
class WhisperConfig:
    num_mel_bins: int = 80
    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    max_source_positions: int = 1500

    @classmethod
    def whisper_tiny(cls) -> "WhisperConfig":
        return cls()

    @classmethod
    def from_hf(cls, src) -> "WhisperConfig":
        raw = _json(src)
        cfg = cls(**{k: raw[k] for k in cls.__dataclass_fields__ if raw.get(k) is not None})
        cfg.validate()
        return cfg

    def encoder_head_dim(self) -> int:
        return self.d_model // self.encoder_attention_heads

    def validate(self) -> None:
        if min(self.num_mel_bins, self.d_model, self.encoder_layers, self.encoder_attention_heads,
               self.encoder_ffn_dim, self.max_source_positions) <= 0:
            raise ValueError("WhisperConfig: sizes must be positive")
        if self.d_model % self.encoder_attention_heads:
            raise ValueError("WhisperConfig: d_model must be divisible by encoder_attention_heads")


class _WhisperAttention(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.h = c.encoder_attention_heads
        self.k_proj = nn.Linear(c.d_model, c.d_model, bias=False)      # Whisper's key projection has no bias
        self.v_proj, self.q_proj, self.out_proj = (nn.Linear(c.d_model, c.d_model) for _ in range(3))

    def forward(self, x):
        B, S, E = x.shape
        q, k, v = (p(x).view(B, S, self.h, E // self.h).transpose(1, 2) for p in (self.q_proj, self.k_proj, self.v_proj))
        return self.out_proj(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, S, E))


class WhisperEncoderLayer(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.self_attn, self.self_attn_layer_norm = _WhisperAttention(c), nn.LayerNorm(c.d_model)
        self.fc1, self.fc2 = nn.Linear(c.d_model, c.encoder_ffn_dim), nn.Linear(c.encoder_ffn_dim, c.d_model)
        self.final_layer_norm = nn.LayerNorm(c.d_model)

    def forward(self, x):
        x = x + self.self_attn(self.self_attn_layer_norm(x))
        return x + self.fc2(F.gelu(self.fc1(self.final_layer_norm(x))))


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Whisper's fixed position table: ``[sin | cos]`` halves with log-spaced timescales."""
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    ang = torch.arange(length, dtype=torch.float32)[:, None] * inv[None]
    return torch.cat([ang.sin(), ang.cos()], dim=1)


class WhisperEncoder(nn.Module):
    """``mel [B, n_mels, T]`` -> ``[B, T/2, d_model]``: two GELU convolutions (the second with stride
    2), added position table, pre-norm transformer layers, final layer norm
    (ferrotorch-whisper/src/encoder.rs:155-260)."""

    def __init__(self, config: WhisperConfig | None = None):
        super().__init__()
        c = self.config = config or WhisperConfig()
        c.validate()
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, 3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, 3, stride=2, padding=1)
        self.embed_positions = nn.Embedding(c.max_source_positions, c.d_model)
        with torch.no_grad():
            if self.embed_positions.weight.device.type != "meta":
                self.embed_positions.weight.copy_(sinusoids(c.max_source_positions, c.d_model))
        self.embed_positions.weight.requires_grad_(False)
        self.layers = nn.ModuleList(WhisperEncoderLayer(c) for _ in range(c.encoder_layers))
        self.layer_norm = nn.LayerNorm(c.d_model)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        if mel.dim() != 3 or mel.shape[1] != self.config.num_mel_bins:
            raise ValueError("WhisperEncoder: expected mel [B, %d, T], got %s" % (self.config.num_mel_bins, tuple(mel.shape)))
        x = F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)
        if x.shape[1] > self.config.max_source_positions:
            raise ValueError("WhisperEncoder: %d frames exceed max_source_positions %d"
                             % (x.shape[1], self.config.max_source_positions))
        x = x + self.embed_positions.weight[: x.shape[1]].to(x.dtype)
        for layer in self.layers:
            x = layer(x)
        return self.layer_norm(x)

    forward_from_mel = forward

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> DropReport:
        """Takes a whole Whisper checkpoint: decoder weights land in ``DropReport.dropped``."""
        return _load(self, sd, strip=("model.encoder.", "encoder."), strict=strict)


# --------------------------------------------------------------------------- Whisper front end
SAMPLE_RATE, N_FFT, HOP_LENGTH, CHUNK_SECONDS = 16000, 400, 160, 30


def mel_filterbank(n_mels: int = 80, n_fft: int = N_FFT, sample_rate: int = SAMPLE_RATE) -> torch.Tensor:
    """Slaney-style mel filters ``[n_mels, n_fft/2 + 1]`` (linear below 1 kHz, logarithmic above,
    each triangle normalised by its bandwidth): the table Whisper ships."""
    def hz_to_mel(f):
        f = torch.as_tensor(f, dtype=torch.float64)
        lin = f / (200.0 / 3)
        log = 15.0 + torch.log(f.clamp_min(1e-10) / 1000.0) / (math.log(6.4) / 27.0)
        return torch.where(f >= 1000.0, log, lin)

    def mel_to_hz(m):
        lin = m * (200.0 / 3)
        log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
        return torch.where(m >= 15.0, log, lin)

    fft_freqs = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1, dtype=torch.float64)
    pts = mel_to_hz(torch.linspace(float(hz_to_mel(0.0)), float(hz_to_mel(sample_rate / 2)), n_mels + 2, dtype=torch.float64))
    lower = (fft_freqs[None] - pts[:-2, None]) / (pts[1:-1] - pts[:-2])[:, None]
    upper = (pts[2:, None] - fft_freqs[None]) / (pts[2:] - pts[1:-1])[:, None]
    fb = torch.minimum(lower, upper).clamp_min(0.0)
    return (fb * (2.0 / (pts[2:] - pts[:-2]))[:, None]).float()


def log_mel_spectrogram(audio: torch.Tensor, n_mels: int = 80, pad_to_chunk: bool = True) -> torch.Tensor:
    """16 kHz mono ``audio [..., T]`` -> ``[..., n_mels, frames]`` as Whisper computes it: pad or cut
    to 30 s (3000 frames), Hann-windowed STFT (400 / 160, reflect padding, last frame dropped),
    power -> Slaney mel -> log10 clamped at 1e-10, floor at max - 8, then ``(x + 4) / 4``
    (ferrotorch-whisper/src/audio.rs:189)."""
    audio = audio.float()
    if pad_to_chunk:
        n = SAMPLE_RATE * CHUNK_SECONDS
        audio = audio[..., :n] if audio.shape[-1] >= n else F.pad(audio, (0, n - audio.shape[-1]))
    if audio.shape[-1] < N_FFT // 2 + 1:
        raise ValueError("log_mel_spectrogram: need at least %d samples" % (N_FFT // 2 + 1))
    win = torch.hann_window(N_FFT, device=audio.device)
    spec = torch.stft(audio, N_FFT, HOP_LENGTH, window=win, return_complex=True)[..., :-1].abs() ** 2
    logmel = torch.log10((mel_filterbank(n_mels).to(audio.device) @ spec).clamp_min(1e-10))
    logmel = torch.maximum(logmel, logmel.amax(dim=(-2, -1), keepdim=True) - 8.0)
    return (logmel + 4.0) / 4.0


# --------------------------------------------------------------------------- GCN (PyTorch-Geometric layout)
@dataclass
class Graph:
    """Node features ``x [N, F]``, ``edge_index [2, E]`` (row 0 sources, row 1 destinations), labels
    ``y [N]`` (ferrotorch-graph/src/data.rs:26-110)."""
    x: torch.Tensor
    edge_index: torch.Tensor
    y: torch.Tensor | None = None

    def __post_init__(self):
        self.edge_index = torch.as_tensor(self.edge_index, dtype=torch.int64).reshape(2, -1)
        if self.x.dim() != 2:
            raise ValueError("Graph: x must be [N, F]")
        if self.edge_index.numel() and (int(self.edge_index.min()) < 0 or int(self.edge_index.max()) >= self.x.shape[0]):
            raise ValueError("Graph: an edge names a node outside 0..%d" % (self.x.shape[0] - 1))
        if self.y is not None and self.y.shape[0] != self.x.shape[0]:
            raise ValueError("Graph: one label per node expected")

    def num_nodes(self) -> int:
        return self.x.shape[0]

    def num_features(self) -> int:
        return self.x.shape[1]

    def num_edges(self) -> int:
        return self.edge_index.shape[1]

    def edge_src(self, e: int) -> int:
        return int(self.edge_index[0, e])

    def edge_dst(self, e: int) -> int:
        return int(self.edge_index[1, e])


class _GcnLin(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, cin))
        nn.init.xavier_uniform_(self.weight)


class GcnConv(nn.Module):
    """``out[v] = b + sum over edges (u, v), self-loops added, of (deg[u] deg[v])^-1/2 (x W^T)[u]``
    with ``deg`` counted at the destination: PyG's ``GCNConv`` defaults.  Parameters:
    ``lin.weight [out, in]`` and ``bias [out]`` (gcn.rs:78-290)."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.lin = _GcnLin(in_features, out_features)
        self.bias = nn.Parameter(torch.zeros(out_features))

    def forward(self, x: torch.Tensor, edge_index: torch.Tensor) -> torch.Tensor:
        N = x.shape[0]
        ei = torch.as_tensor(edge_index, dtype=torch.int64, device=x.device).reshape(2, -1)
        if ei.numel() and (int(ei.min()) < 0 or int(ei.max()) >= N):
            raise ValueError("GcnConv: an edge names a node outside 0..%d" % (N - 1))
        loops = torch.arange(N, device=x.device)
        src, dst = torch.cat([ei[0], loops]), torch.cat([ei[1], loops])
        deg = torch.zeros(N, dtype=x.dtype, device=x.device).index_add_(0, dst, torch.ones_like(dst, dtype=x.dtype))
        dis = deg.pow(-0.5)
        dis = torch.where(torch.isinf(dis), torch.zeros_like(dis), dis)
        h = x @ self.lin.weight.t()
        out = torch.zeros_like(h).index_add_(0, dst, h[src] * (dis[src] * dis[dst])[:, None])
        return out + self.bias


class GcnNet(nn.Module):
    """``conv2(dropout(relu(conv1(x))))``: raw class logits (gcn.rs:297-360)."""

    def __init__(self, in_features: int, hidden: int, num_classes: int, dropout: float = 0.5):
        super().__init__()
        self.conv1, self.conv2, self.dropout = GcnConv(in_features, hidden), GcnConv(hidden, num_classes), dropout

    def in_features(self) -> int:
        return self.conv1.lin.weight.shape[1]

    def hidden(self) -> int:
        return self.conv1.lin.weight.shape[0]

    def num_classes(self) -> int:
        return self.conv2.lin.weight.shape[0]

    def forward(self, x, edge_index):
        h = F.dropout(F.relu(self.conv1(x, edge_index)), self.dropout, self.training)
        return self.conv2(h, edge_index)

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> DropReport:
        return _load(self, sd, strict=strict)


# --------------------------------------------------------------------------- SB3 PPO policy
@dataclass
class MlpPolicyConfig:
    obs_dim: int = 4
    hidden: int = 64
    n_actions: int = 2

    @classmethod
    def cartpole_v1(cls) -> "MlpPolicyConfig":
        return cls()


class MlpExtractor(nn.Module):
    """Stable-Baselines3's two separate tanh trunks: ``policy_net`` and ``value_net``, each
    Linear-Tanh-Linear-Tanh (the Tanh modules take the odd indices, hence keys ``0`` and ``2``)."""

    def __init__(self, obs_dim: int, hidden: int):
        super().__init__()
        mk = lambda: nn.Sequential(nn.Linear(obs_dim, hidden), nn.Tanh(), nn.Linear(hidden, hidden), nn.Tanh())  # noqa: E731
        self.policy_net, self.value_net = mk(), mk()

    def forward_actor(self, features):
        return self.policy_net(features)

    def forward_critic(self, features):
        return self.value_net(features)

    def obs_dim(self) -> int:
        return self.policy_net[0].in_features

    def hidden(self) -> int:
        return self.policy_net[0].out_features


@dataclass
class PolicyOutput:
    action_logits: torch.Tensor
    value: torch.Tensor


class MlpPolicy(nn.Module):
    """Discrete-action actor-critic of SB3 PPO (mlp_policy.rs:452-540): observation -> action logits
    and state value.  A checkpoint's ``log_std`` (continuous policies) is reported as dropped."""

    def __init__(self, config: MlpPolicyConfig | None = None):
        super().__init__()
        c = self.cfg = config or MlpPolicyConfig()
        if min(c.obs_dim, c.hidden, c.n_actions) <= 0:
            raise ValueError("MlpPolicyConfig: sizes must be positive")
        self.mlp_extractor = MlpExtractor(c.obs_dim, c.hidden)
        self.action_net, self.value_net = nn.Linear(c.hidden, c.n_actions), nn.Linear(c.hidden, 1)

    def config(self) -> MlpPolicyConfig:
        return self.cfg

    def forward(self, obs: torch.Tensor) -> PolicyOutput:
        if obs.dim() == 1:
            obs = obs[None]
        if obs.shape[-1] != self.cfg.obs_dim:
            raise ValueError("MlpPolicy: expected observations of %d values, got %d" % (self.cfg.obs_dim, obs.shape[-1]))
        return PolicyOutput(self.action_net(self.mlp_extractor.forward_actor(obs)),
                            self.value_net(self.mlp_extractor.forward_critic(obs)).squeeze(-1))

    def act(self, obs: torch.Tensor, deterministic: bool = True, generator: torch.Generator | None = None) -> torch.Tensor:
        logits = self.forward(obs).action_logits
        if deterministic:
            return logits.argmax(-1)
        return torch.multinomial(logits.softmax(-1), 1, generator=generator).squeeze(-1)

    def load_hf_state_dict(self, sd: dict, strict: bool = True) -> DropReport:
        return _load(self, sd, strip=("policy.",), strict=strict)


# --------------------------------------------------------------------------- loaders (safetensors_loader.rs of each crate)
def _read_weights(path: str) -> dict:
    """A SafeTensors file, a ``.pt`` / ``.bin`` state dict, or a model directory."""
    import os

    from ..serialize.state import load_pytorch_state_dict, load_safetensors, load_safetensors_auto

    if os.path.isdir(path):
        if any(os.path.exists(os.path.join(path, f)) for f in ("model.safetensors", "model.safetensors.index.json")):
            return load_safetensors_auto(path)
        for f in ("pytorch_model.bin", "policy.pth", "model.pt"):
            if os.path.exists(os.path.join(path, f)):
                return load_pytorch_state_dict(os.path.join(path, f))
        raise FileNotFoundError("no weights (model.safetensors, pytorch_model.bin ...) under %s" % path)
    if path.endswith(".safetensors"):
        return load_safetensors(path)
    return load_pytorch_state_dict(path)


def _config_path(path: str) -> str | None:
    import os

    p = os.path.join(path, "config.json") if os.path.isdir(path) else os.path.join(os.path.dirname(path), "config.json")
    return p if os.path.exists(p) else None


def load_bert_model(path: str, config: BertConfig | None = None) -> tuple[BertModel, DropReport]:
    """``(model, report)`` from a Hugging Face BERT directory or weight file; the configuration
    comes from the neighbouring ``config.json`` unless given."""
    cfg_file = _config_path(path)
    cfg = config or (BertConfig.from_hf(cfg_file) if cfg_file else BertConfig())
    model = BertModel(cfg).eval()
    return model, model.load_hf_state_dict(_read_weights(path))


def load_sentence_transformer(path: str, config: BertConfig | None = None, normalize: bool = True):
    cfg_file = _config_path(path)
    cfg = config or (BertConfig.from_hf(cfg_file) if cfg_file else BertConfig())
    model = SentenceTransformer(cfg, normalize).eval()
    return model, model.load_hf_state_dict(_read_weights(path))


def load_whisper_encoder(path: str, config: WhisperConfig | None = None):
    cfg_file = _config_path(path)
    cfg = config or (WhisperConfig.from_hf(cfg_file) if cfg_file else WhisperConfig())
    model = WhisperEncoder(cfg).eval()
    return model, model.load_hf_state_dict(_read_weights(path))


def load_gcn_net(path: str, in_features: int | None = None, hidden: int | None = None, num_classes: int | None = None):
    """The layer sizes are read off the weights (``conv1.lin.weight [hidden, in]``,
    ``conv2.lin.weight [classes, hidden]``) unless given."""
    sd = _read_weights(path)
    h, i = sd["conv1.lin.weight"].shape
    c = sd["conv2.lin.weight"].shape[0]
    model = GcnNet(in_features or i, hidden or h, num_classes or c).eval()
    return model, model.load_hf_state_dict(sd)


def load_ppo_policy(path: str, config: MlpPolicyConfig | None = None):
    """An SB3 ``policy.pth`` / SafeTensors export; sizes come from the weights unless given."""
    sd = _read_weights(path)
    sd = {(k[7:] if k.startswith("policy.") else k): v for k, v in sd.items()}
    if config is None:
        hid, obs = sd["mlp_extractor.policy_net.0.weight"].shape
        config = MlpPolicyConfig(obs, hid, sd["action_net.weight"].shape[0])
    model = MlpPolicy(config).eval()
    return model, model.load_hf_state_dict(sd)


# --------------------------------------------------------------------------- the reference's remaining names
HfBertConfig, HfWhisperConfig = BertConfig, WhisperConfig     # the config classes read Hugging Face's config.json as is


def _from_file(cls, path: str):
    """``path``: a ``config.json`` file or the model directory that holds one."""
    import os

    return cls.from_hf(os.path.join(path, "config.json") if os.path.isdir(path) else path)


def _from_json_str(cls, text: str):
    import json

    return cls.from_hf(json.loads(text))


for _cfg in (BertConfig, WhisperConfig):
    _cfg.from_file = classmethod(_from_file)
    _cfg.from_json_str = classmethod(_from_json_str)
BertSelfOutput.forward_residual = BertSelfOutput.forward
BertEmbeddings.forward_from_ids = lambda self, ids, token_type_ids=None: self.forward(
    torch.as_tensor(list(ids), dtype=torch.long, device=self.word_embeddings.weight.device)[None],
    None if token_type_ids is None else torch.as_tensor(list(token_type_ids), dtype=torch.long, device=self.word_embeddings.weight.device)[None])
WhisperEncoderSelfAttention = _WhisperAttention
N_MELS, N_FRAMES = 80, CHUNK_SECONDS * SAMPLE_RATE // HOP_LENGTH      # 80 mel bins, 3000 frames per 30 s chunk


@dataclass
class BertOutput:
    last_hidden_state: torch.Tensor
    pooler_output: torch.Tensor

    @classmethod
    def of(cls, model: BertModel, input_ids, attention_mask=None, token_type_ids=None) -> "BertOutput":
        return cls(*model(input_ids, attention_mask, token_type_ids))


class WhisperConvStem(nn.Module):
    """The two GELU convolutions in front of the encoder (the second halves the frame rate), as a
    module over an encoder's own weights."""

    def __init__(self, encoder: WhisperEncoder):
        super().__init__()
        self.conv1, self.conv2 = encoder.conv1, encoder.conv2

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        return F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)


class ActionNet(nn.Linear):
    """Policy head: latent -> action logits (``MlpPolicy.action_net``)."""


class ValueHead(nn.Linear):
    """Critic head: latent -> state value (``MlpPolicy.value_net``)."""

    def __init__(self, in_features: int, out_features: int = 1, **kw):
        super().__init__(in_features, out_features, **kw)
