"""Llama-family decoder on the native kernels.

Architecture and checkpoint contract follow the reference's ``ferrotorch-llama``:
config presets (config.rs:50-64 ``llama3_8b``, config.rs:98-112 ``llama3_3_70b_instruct``),
pre-norm decoder layer (layer.rs:63), GQA attention with half-rotation RoPE
(attention.rs:213-280), SwiGLU MLP (mlp.rs), HF-native state-dict keys
(gpu.rs:1007-1060; tied embeddings copy ``embed_tokens`` into ``lm_head``, model.rs:382-386).

Internally the q/k/v and gate/up projections are fused into one weight each (one GEMM, one
RoPE launch on the packed buffer, one SwiGLU kernel); :meth:`LlamaForCausalLM.load_hf_state_dict`
and :meth:`hf_state_dict` convert from / to the HF key layout, so SafeTensors, ``.pt`` and
GGUF checkpoints load unchanged.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass

import torch
from torch import nn

from ..nn.layers import GQAAttention, KVCache, Linear, RMSNorm, RotaryPositionEmbedding, SwiGLU
from ..ops import functional as F


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int | None = None
    max_position_embeddings: int = 8192
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    rope_scaling: dict | None = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"            # "silu", "relu" (ReluLLaMA), "gelu", "fatrelu" (ProSparse)
    hidden_act_param: float | None = None   # FatReLU threshold (0.01 when absent, config.rs:137-140)
    attention_bias: bool = False
    mlp_bias: bool = False
    initializer_range: float = 0.02

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    # ---- presets (ferrotorch-llama/src/config.rs:50-112)
    @classmethod
    def llama3_8b(cls) -> "LlamaConfig":
        return cls()

    @classmethod
    def llama3_70b(cls) -> "LlamaConfig":
        return cls(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                   num_key_value_heads=8, max_position_embeddings=131072)

    llama3_3_70b_instruct = llama3_70b

    @classmethod
    def llama2_7b(cls) -> "LlamaConfig":
        return cls(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                   num_attention_heads=32, num_key_value_heads=32, max_position_embeddings=4096, rope_theta=10000.0)

    @classmethod
    def prosparse_7b(cls) -> "LlamaConfig":
        """Llama-2-7B shape with ``fatrelu(gate, 0.01) * up`` in the MLP (config.rs:85-90)."""
        c = cls.llama2_7b()
        c.hidden_act, c.hidden_act_param = "fatrelu", 0.01
        return c

    @classmethod
    def tiny(cls) -> "LlamaConfig":
        """The CPU plumbing config: 4 layers, d 256, 4 q / 2 kv heads of 64, FFN 688, vocab 4096."""
        return cls(vocab_size=4096, hidden_size=256, intermediate_size=688, num_hidden_layers=4,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=2048,
                   rope_theta=10000.0)

    @classmethod
    def from_hf(cls, cfg: dict | str) -> "LlamaConfig":
        """Build from an HF ``config.json`` dict or path (ferrotorch-llama/src/config.rs:126)."""
        if isinstance(cfg, str):
            with open(cfg) as f:
                cfg = json.load(f)
        cfg = dict(cfg)
        rp = cfg.get("rope_parameters")
        if isinstance(rp, dict):
            # newer config.json files keep the rotary settings in one "rope_parameters" object
            if "rope_theta" in rp:
                cfg.setdefault("rope_theta", rp["rope_theta"])
            if rp.get("rope_type", rp.get("type", "default")) != "default" and not cfg.get("rope_scaling"):
                cfg["rope_scaling"] = rp
        # what a config.json may leave out takes the Hugging Face defaults, not the Llama-3 preset's
        # (ferrotorch-hub/src/hf_config.rs: rms_norm_eps 1e-6, rope_theta 10000)
        cfg.setdefault("rope_theta", 10000.0)
        cfg.setdefault("rms_norm_eps", 1e-6)
        known = {k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg and cfg[k] is not None}
        if "num_key_value_heads" not in known and "num_attention_heads" in known:
            known["num_key_value_heads"] = known["num_attention_heads"]      # plain multi-head attention
        act = known.get("hidden_act", "silu")
        act = "silu" if act == "swish" else act
        if act not in ("silu", "relu", "gelu", "fatrelu"):
            raise ValueError("LlamaConfig: unsupported hidden_act %r" % (act,))
        known["hidden_act"] = act
        if act == "fatrelu":
            known["hidden_act_param"] = float(known.get("hidden_act_param", 0.01))
        rs = known.get("rope_scaling")
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            known["rope_scaling"] = {"type": kind, "factor": rs.get("factor", 1.0),
                                     "original_max": rs.get("original_max_position_embeddings", 8192),
                                     "low_freq_factor": rs.get("low_freq_factor", 1.0),
                                     "high_freq_factor": rs.get("high_freq_factor", 4.0)}
        out = cls(**known)
        out.validate()
        return out

    def to_dict(self) -> dict:
        return asdict(self)

    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def validate(self) -> None:
        """The reference's checks (config.rs:160-215): positive sizes, heads divide the hidden
        size (when no explicit head_dim is given they must), KV heads divide the query heads."""
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "max_position_embeddings", "head_dim"):
            if int(getattr(self, k)) <= 0:
                raise ValueError("LlamaConfig: %s must be positive" % k)
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("LlamaConfig: num_attention_heads (%d) must be divisible by num_key_value_heads (%d)"
                             % (self.num_attention_heads, self.num_key_value_heads))
        if self.head_dim % 2:
            raise ValueError("LlamaConfig: head_dim (%d) must be even for rotary embeddings" % self.head_dim)
        if not (self.rms_norm_eps > 0 and self.rope_theta > 0):
            raise ValueError("LlamaConfig: rms_norm_eps and rope_theta must be positive")

    def num_parameters(self) -> int:
        h, f, v, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        qkv = (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_dim * h
        o = self.num_attention_heads * self.head_dim * h
        per_layer = qkv + o + 3 * h * f + 2 * h
        return L * per_layer + v * h * (1 if self.tie_word_embeddings else 2) + h


class LlamaDecoderLayer(nn.Module):
    def __init__(self, cfg: LlamaConfig, rope: RotaryPositionEmbedding):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.self_attn = GQAAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                                      cfg.head_dim, rope, bias=cfg.attention_bias)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.mlp = SwiGLU(cfg.hidden_size, cfg.intermediate_size, cfg.hidden_act, bias=cfg.mlp_bias,
                          activation_param=cfg.hidden_act_param)

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None = None, *, cache: KVCache | None = None,
                positions: torch.Tensor | None = None):
        """Takes the residual stream ``x`` and the previous block's pending branch output
        ``delta`` (added inside the norm kernel); returns ``(x, delta)`` for the next layer."""
        if delta is None:
            h = self.input_layernorm(x)
        else:
            h, x = self.input_layernorm(x, delta)
        a = self.self_attn(h, cache=cache, positions=positions)
        h, x = self.post_attention_layernorm(x, a)
        return x, self.mlp(h)

    def forward_with_cache(self, x: torch.Tensor, layer_cache=None):
        """One decoder layer on a value cache (layer.rs ``forward_with_cache``): ``(hidden states, new layer
        cache)`` with the residual additions applied."""
        from .llama_compat import _GrowingLayerCache

        grow = _GrowingLayerCache(layer_cache)
        h, delta = self.forward(x, cache=grow)
        return h + delta, grow.as_layer()


class LlamaModel(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.rope = RotaryPositionEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta,
                                            scaling=cfg.rope_scaling)
        self.layers = nn.ModuleList(LlamaDecoderLayer(cfg, self.rope) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps)
        self.checkpoint_layers = False

    def forward(self, input_ids: torch.Tensor, *, caches: list[KVCache] | None = None,
                positions: torch.Tensor | None = None) -> torch.Tensor:
        x = F.embedding(input_ids, self.embed_tokens.weight)
        delta = None
        for i, layer in enumerate(self.layers):
            cache = caches[i] if caches is not None else None
            if self.checkpoint_layers and self.training and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint

                if delta is None:
                    x, delta = checkpoint(lambda a, l=layer: l(a), x, use_reentrant=False)
                else:
                    x, delta = checkpoint(lambda a, b, l=layer: l(a, b), x, delta, use_reentrant=False)
            else:
                x, delta = layer(x, delta, cache=cache, positions=positions)
        h, _ = self.norm(x, delta)
        return h


class LlamaForCausalLM(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.config = cfg
        self.model = LlamaModel(cfg)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight
        self.reset_parameters()

    def reset_parameters(self) -> None:
        std = self.config.initializer_range
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2:
                    p.normal_(0.0, std)
                elif name.endswith("bias"):
                    p.zero_()
                else:
                    p.fill_(1.0)

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, *,
                caches: list[KVCache] | None = None, positions: torch.Tensor | None = None,
                last_token_only: bool = False, loss_denominator: int | None = None):
        """Returns logits ``[B, S, V]`` (or ``[B, 1, V]``), or the mean next-token loss when
        ``labels`` (already shifted, same shape as ``input_ids``) is given -- the loss path never
        materialises the logits (chunked lm_head + fused cross-entropy)."""
        h = self.model(input_ids, caches=caches, positions=positions)
        if labels is not None:
            return F.linear_cross_entropy(h, self.lm_head.weight, labels, num_valid=loss_denominator)
        if last_token_only:
            h = h[:, -1:]
        return self.lm_head(h)

    # ------------------------------------------------------------------ the reference's id-level entry points
    def forward_from_ids(self, ids) -> torch.Tensor:
        """Logits ``[1, S, V]`` for one sequence of token ids (ferrotorch-llama/src/model.rs:223)."""
        dev = self.model.embed_tokens.weight.device
        return self(torch.as_tensor(list(ids), dtype=torch.long, device=dev)[None])

    @torch.no_grad()
    def forward_one_with_cache(self, token: int, cache):
        """One decode step on a value cache (model.rs:284): ``(logits [V] float64, longer cache)``.
        ``cache`` is a :class:`~ferrotorch_b200.models.llama_compat.LlamaKvCache` (empty for the
        first token); it is not modified.  Decoding a sequence token by token this way gives the
        logits of :meth:`forward_from_ids` at every position.  The pre-allocated in-place caches of
        :meth:`make_caches` are what ``generate`` uses; this form is for code written against the
        reference's functional cache."""
        from .llama_compat import LlamaKvCache, _GrowingLayerCache

        n_layers = len(self.model.layers)
        if cache.layers and len(cache.layers) != n_layers:
            raise ValueError("forward_one_with_cache: cache has %d layers but model has %d" % (len(cache.layers), n_layers))
        dev = self.model.embed_tokens.weight.device
        grow = [_GrowingLayerCache(cache.layers[i] if cache.layers else None) for i in range(n_layers)]
        logits = self(torch.tensor([[int(token)]], dtype=torch.long, device=dev), caches=grow, last_token_only=True)
        new = LlamaKvCache(tuple(g.as_layer() for g in grow), len(cache) + 1)
        return logits[0, -1].double(), new

    def load_hqq_state_dict(self, hqq_state: dict, strict: bool = True) -> None:
        """Load a checkpoint whose linears are HQQ 4-bit (``W_q`` / ``scale`` / ``zero`` / ``shape``
        per layer): expanded to dense weights, then :meth:`load_hf_state_dict` (model.rs:414)."""
        from ..serialize.quant_loaders import hqq_state_dict_to_dense

        self.load_hf_state_dict(hqq_state_dict_to_dense(hqq_state), strict)

    def make_caches(self, batch: int, max_len: int, device=None, dtype=torch.bfloat16) -> list[KVCache]:
        c = self.config
        return [KVCache(batch, max_len, c.num_key_value_heads, c.head_dim, device, dtype)
                for _ in range(c.num_hidden_layers)]

    # ------------------------------------------------------------------ model directories and files
    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, device="cpu") -> "LlamaForCausalLM":
        """Build the model a Hugging Face directory describes (``config.json`` plus
        ``model.safetensors``, a sharded ``model.safetensors.index.json`` or ``pytorch_model.bin``)
        and load its weights; a tied checkpoint without ``lm_head.weight`` shares the embedding
        (ferrotorch-llama/src/model.rs:382-386)."""
        import os

        from ..serialize.state import load_pytorch_state_dict, load_safetensors_auto

        cfg = LlamaConfig.from_hf(os.path.join(path, "config.json"))
        model = cls(cfg).to(device=device, dtype=dtype)
        if any(os.path.exists(os.path.join(path, f)) for f in ("model.safetensors", "model.safetensors.index.json")):
            sd = load_safetensors_auto(path, dtype=dtype)
        elif os.path.exists(os.path.join(path, "pytorch_model.bin")):
            sd = load_pytorch_state_dict(os.path.join(path, "pytorch_model.bin"))
        else:
            raise FileNotFoundError("no model.safetensors[.index.json] or pytorch_model.bin under %s" % path)
        if "lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        model.load_hf_state_dict(sd)
        if cfg.tie_word_embeddings:
            model.lm_head.weight = model.model.embed_tokens.weight
        return model

    def save_pretrained(self, path: str, max_shard_bytes: int | None = None) -> None:
        """Write ``config.json`` and the weights under their Hugging Face names (one
        ``model.safetensors``, or shards plus an index when ``max_shard_bytes`` is given)."""
        import json as _json
        import os

        from ..serialize.state import save_safetensors, save_safetensors_sharded

        os.makedirs(path, exist_ok=True)
        cfg = {k: v for k, v in self.config.to_dict().items() if v is not None}
        cfg.update(architectures=["LlamaForCausalLM"], model_type="llama")
        with open(os.path.join(path, "config.json"), "w") as f:
            _json.dump(cfg, f, indent=2)
        sd = self.hf_state_dict()
        if self.config.tie_word_embeddings:
            sd.pop("lm_head.weight", None)
        if max_shard_bytes:
            save_safetensors_sharded(sd, path, max_shard_bytes=max_shard_bytes)
        else:
            save_safetensors(sd, os.path.join(path, "model.safetensors"))

    @classmethod
    def from_gguf(cls, path: str, dtype: torch.dtype = torch.bfloat16, device="cpu", nibble_order: str = "ggml") -> "LlamaForCausalLM":
        """Build from a GGUF file: the ``llama.*`` metadata gives the configuration, the tensors are
        dequantised on the host and renamed to the Hugging Face keys
        (ferrotorch-serialize/src/gguf.rs:909, ferrotorch-llama/src/gguf_remap.rs:23-52)."""
        from ..serialize.gguf import GgufFile, gguf_key_to_hf

        with GgufFile(path) as f:
            md = f.metadata
            arch = md.get("general.architecture", "llama")
            g = lambda k, default=None: md.get("%s.%s" % (arch, k), default)      # noqa: E731
            emb = f.tensors.get("token_embd.weight")
            heads = int(g("attention.head_count"))
            cfg = LlamaConfig(vocab_size=int(g("vocab_size", emb[1][0] if emb else 0)), hidden_size=int(g("embedding_length")),
                              intermediate_size=int(g("feed_forward_length")), num_hidden_layers=int(g("block_count")),
                              num_attention_heads=heads, num_key_value_heads=int(g("attention.head_count_kv", heads)),
                              max_position_embeddings=int(g("context_length", 8192)),
                              rms_norm_eps=float(g("attention.layer_norm_rms_epsilon", 1e-5)),
                              rope_theta=float(g("rope.freq_base", 10000.0)), tie_word_embeddings="output.weight" not in f.tensors)
            cfg.validate()
            sd = {(gguf_key_to_hf(n) or n): f.dequantize(n, dtype, nibble_order) for n in f.tensors}
        if "lm_head.weight" not in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        model = cls(cfg).to(device=device, dtype=dtype)
        model.load_hf_state_dict({k: v for k, v in sd.items() if k.startswith(("model.", "lm_head."))})
        if cfg.tie_word_embeddings:
            model.lm_head.weight = model.model.embed_tokens.weight
        return model

    # ------------------------------------------------------------------ HF key layout
    def hf_state_dict(self) -> dict[str, torch.Tensor]:
        """State dict with HF-native keys (separate q/k/v and gate/up projections)."""
        c = self.config
        nq, nkv, d = c.num_attention_heads * c.head_dim, c.num_key_value_heads * c.head_dim, c.head_dim
        out: dict[str, torch.Tensor] = {}
        for k, v in self.state_dict().items():
            if ".self_attn.qkv_proj." in k:
                base, kind = k.split(".self_attn.qkv_proj.")
                q, kk, vv = v.split([nq, nkv, nkv], dim=0)
                out["%s.self_attn.q_proj.%s" % (base, kind)] = q
                out["%s.self_attn.k_proj.%s" % (base, kind)] = kk
                out["%s.self_attn.v_proj.%s" % (base, kind)] = vv
            elif ".mlp.gate_up_proj." in k:
                base, kind = k.split(".mlp.gate_up_proj.")
                g, u = v.chunk(2, dim=0)
                out["%s.mlp.gate_proj.%s" % (base, kind)] = g
                out["%s.mlp.up_proj.%s" % (base, kind)] = u
            else:
                out[k] = v
        if c.tie_word_embeddings:
            out.pop("lm_head.weight", None)
        return out

    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], strict: bool = True) -> None:
        """Load HF-native keys (also accepts this module's own fused keys)."""
        fused: dict[str, torch.Tensor] = {}
        groups: dict[str, dict[str, torch.Tensor]] = {}
        for k, v in sd.items():
            for tag, parts in (("self_attn", ("q_proj", "k_proj", "v_proj")), ("mlp", ("gate_proj", "up_proj"))):
                hit = next((p for p in parts if ".%s.%s." % (tag, p) in k), None)
                if hit is not None:
                    base, kind = k.split(".%s.%s." % (tag, hit))
                    name = "%s.%s.%s.%s" % (base, tag, "qkv_proj" if tag == "self_attn" else "gate_up_proj", kind)
                    groups.setdefault(name, {})[hit] = v
                    break
            else:
                fused[k] = v
        for name, parts in groups.items():
            order = ("q_proj", "k_proj", "v_proj") if "qkv_proj" in name else ("gate_proj", "up_proj")
            missing = [p for p in order if p not in parts]
            if missing:
                raise KeyError("incomplete projection group for %s: missing %s" % (name, missing))
            fused[name] = torch.cat([parts[p] for p in order], dim=0)
        if "lm_head.weight" not in fused and "model.embed_tokens.weight" in fused:
            fused["lm_head.weight"] = fused["model.embed_tokens.weight"]
        self.load_state_dict(fused, strict=strict)
