"""Single-sequence inference objects with the reference's method set: logits out, one sequence in.

``LlamaGpuInferencer`` (ferrotorch-llama/src/gpu.rs:153-548) holds the bf16 weights on a device and
answers ``forward_from_ids`` (last-position logits), ``forward_logits_from_ids_all`` (every
position) and the *profiled* forward that the reference's weight-sparsity tooling consumes: per
layer, per token, the largest attention-output magnitude of every head (taken before ``o_proj``)
and the largest gated-activation magnitude of every block of MLP neurons (what multiplies the rows
of ``down_proj``), optionally the hidden state that enters a chosen layer, and optionally the
"local plain-act" variant in which a neuron's activation is weighted by its closed-form gradient of
``|y|^2`` (``y`` = the layer's output) instead of being taken raw (gpu.rs:361-512, 666-775).

``GraphedDecoder`` (gpu.rs:854-1000) captures the single-token forward into a CUDA graph with a
stable input and output buffer; ``decode_step(token)`` replays it and returns logits that are
bit-identical to ``forward_from_ids([token])``.

Both sit on :class:`~ferrotorch_b200.models.llama.LlamaForCausalLM`, whose layers run this
package's kernels on a GPU and torch ops on the host, so everything here also works (without a
graph) on the CPU.  Batched, paged, tensor-parallel serving is
:class:`~ferrotorch_b200.models.engine.LlamaEngine`; this module is the reference's simpler contract.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .llama import LlamaConfig, LlamaForCausalLM


@dataclass
class ProfiledForwardResult:
    """Magnitudes in token-major order, as the reference lays them out."""
    seq_len: int
    attn_magnitudes: torch.Tensor            # [seq, n_layers, n_heads] fp32
    mlp_magnitudes: torch.Tensor             # [seq, n_layers, n_mlp_blocks] fp32
    bootstrap_hidden: torch.Tensor | None    # [seq, hidden] in the model's dtype: the input of layer ``bootstrap_k``
    bootstrap_k: int | None
    hidden_size: int

    def attn_at(self, token: int, layer: int, head: int) -> float:
        return float(self.attn_magnitudes[token, layer, head])

    def mlp_at(self, token: int, layer: int, block: int) -> float:
        return float(self.mlp_magnitudes[token, layer, block])


class LlamaGpuInferencer:
    def __init__(self, model: LlamaForCausalLM, device=None, dtype: torch.dtype | None = None):
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        if dtype is None:
            dtype = torch.bfloat16 if self.device.type == "cuda" else next(model.parameters()).dtype
        self.model = model.to(device=self.device, dtype=dtype).eval()
        self.config: LlamaConfig = model.config

    @classmethod
    def new(cls, config: LlamaConfig, state_dict: dict | None = None, device=None, dtype: torch.dtype | None = None
            ) -> "LlamaGpuInferencer":
        """From a configuration and (optionally) a Hugging Face-style state dict."""
        model = LlamaForCausalLM(config)
        if state_dict is not None:
            model.load_hf_state_dict(state_dict)
        return cls(model, device, dtype)

    @classmethod
    def from_gguf_gpu_dequant(cls, path: str, device=None, dtype: torch.dtype | None = None, config: LlamaConfig | None = None
                              ) -> "LlamaGpuInferencer":
        """From a GGUF file whose quantised tensors cross to the device as raw blocks and are expanded there
        (ferrotorch-llama/src/gpu_gguf.rs:336); on the host the file's own decoder does the expansion.  The
        configuration comes from the file's metadata unless one is given."""
        from ..serialize.gguf import GgufFile, load_gguf_state_dict, load_gguf_state_dict_gpu

        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        device = torch.device(device)
        if config is None:
            with GgufFile(path) as f:
                md = f.metadata
            arch = md.get("general.architecture", "llama")

            def key(name, default=None):
                return md.get("%s.%s" % (arch, name), default)

            heads = int(key("attention.head_count"))
            config = LlamaConfig(vocab_size=int(md.get("%s.vocab_size" % arch, len(md.get("tokenizer.ggml.tokens", [])) or 32000)),
                                 hidden_size=int(key("embedding_length")), intermediate_size=int(key("feed_forward_length")),
                                 num_hidden_layers=int(key("block_count")), num_attention_heads=heads,
                                 num_key_value_heads=int(key("attention.head_count_kv", heads)),
                                 max_position_embeddings=int(key("context_length", 2048)),
                                 rms_norm_eps=float(key("attention.layer_norm_rms_epsilon", 1e-5)),
                                 rope_theta=float(key("rope.freq_base", 10000.0)))
        want = dtype or (torch.bfloat16 if device.type == "cuda" else torch.float32)
        sd = load_gguf_state_dict_gpu(path, device, want) if device.type == "cuda" else load_gguf_state_dict(path, want)
        if "lm_head.weight" not in sd and "model.embed_tokens.weight" in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        model = LlamaForCausalLM(config)
        model.load_hf_state_dict(sd)
        return cls(model, device, want)

    def generate_masked(self, prompt_ids, processor, max_new_tokens: int) -> list:
        """Greedy decoding under a grammar (a ``JsonSchemaProcessor`` or ``None``): every step's logits are
        masked to the tokens the grammar admits, on the device the logits live on; generation stops when the
        grammar is complete (gpu_gguf.rs:510-560).  Returns the generated ids."""
        from .llama_compat import masked_decode_loop

        return masked_decode_loop(lambda ids: self.forward_from_ids(ids), processor, prompt_ids, max_new_tokens,
                                  self.device.index if self.device.type == "cuda" else None)

    def _ids(self, ids) -> torch.Tensor:
        ids = list(ids)
        if not ids:
            raise ValueError("forward_from_ids: empty id list")
        if max(ids) >= self.config.vocab_size or min(ids) < 0:
            raise ValueError("forward_from_ids: token id outside [0, %d)" % self.config.vocab_size)
        return torch.tensor([ids], dtype=torch.long, device=self.device)

    @torch.no_grad()
    def forward_from_ids(self, ids) -> torch.Tensor:
        """Logits after the last position, ``[vocab]`` fp32 on the host."""
        return self.model(self._ids(ids), last_token_only=True)[0, -1].float().cpu()

    @torch.no_grad()
    def forward_logits_from_ids_all(self, ids) -> torch.Tensor:
        """Logits after every position, ``[seq, vocab]`` fp32 on the host."""
        return self.model(self._ids(ids))[0].float().cpu()

    def forward_from_ids_profiled(self, ids, mlp_block_size: int, n_mlp_blocks: int) -> ProfiledForwardResult:
        return self.forward_from_ids_profiled_with_bootstrap(ids, mlp_block_size, n_mlp_blocks, None, False)

    @torch.no_grad()
    def forward_from_ids_profiled_with_bootstrap(self, ids, mlp_block_size: int, n_mlp_blocks: int, bootstrap_k: int | None = None,
                                                 plainact_local: bool = False) -> ProfiledForwardResult:
        """The lm_head is skipped: profiling needs no logits.  ``bootstrap_k`` in
        ``1 ..= num_hidden_layers`` asks for the hidden state after layer ``k - 1``."""
        cfg = self.config
        if mlp_block_size <= 0 or n_mlp_blocks <= 0 or mlp_block_size * n_mlp_blocks != cfg.intermediate_size:
            raise ValueError("profiled forward: mlp_block_size * n_mlp_blocks must equal intermediate_size %d, got %d * %d"
                             % (cfg.intermediate_size, mlp_block_size, n_mlp_blocks))
        if bootstrap_k is not None and not 1 <= bootstrap_k <= cfg.num_hidden_layers:
            raise ValueError("profiled forward: bootstrap_k must be in 1 ..= %d, got %d" % (cfg.num_hidden_layers, bootstrap_k))
        t = self._ids(ids)
        S, Hq, D = t.shape[1], cfg.num_attention_heads, cfg.head_dim
        attn, mlp, gated_of, boot = [], [], {}, [None]
        handles = []
        for li, layer in enumerate(self.model.model.layers):
            def attn_tap(_m, args):
                attn.append(args[0].reshape(S, Hq, D).abs().amax(-1).float())

            def mlp_tap(_m, args, li=li):
                g = args[0].reshape(S, n_mlp_blocks, mlp_block_size)
                if plainact_local:
                    gated_of[li] = g
                else:
                    mlp.append(g.abs().amax(-1).float())

            def layer_tap(m, _args, out, li=li):
                x, delta = out
                y = x + delta                                      # the residual stream after this layer
                if plainact_local:
                    z = (y.reshape(S, -1) @ m.mlp.down_proj.weight).reshape(S, n_mlp_blocks, mlp_block_size)
                    mlp.append((gated_of.pop(li) * z).abs().amax(-1).float())
                if bootstrap_k is not None and li + 1 == bootstrap_k:
                    boot[0] = y.reshape(S, -1).clone()

            handles += [layer.self_attn.o_proj.register_forward_pre_hook(attn_tap),
                        layer.mlp.down_proj.register_forward_pre_hook(mlp_tap), layer.register_forward_hook(layer_tap)]
        try:
            self.model.model(t)
        finally:
            for h in handles:
                h.remove()
        return ProfiledForwardResult(S, torch.stack(attn, 1).cpu(), torch.stack(mlp, 1).cpu(),
                                     boot[0].cpu() if boot[0] is not None else None, bootstrap_k, cfg.hidden_size)


class GraphedDecoder:
    """``capture`` runs the single-token forward once eagerly (so that every lazily built table
    exists), then records it into a CUDA graph that reads the token from a fixed buffer and leaves
    the logits in another; torch serves the capture's allocations from a pool private to the graph,
    so replays and eager forwards can be interleaved.  Without a CUDA device there is nothing to
    capture: ``decode_step`` calls the same forward eagerly and still counts its calls."""

    def __init__(self, model: LlamaGpuInferencer, graph, ids_static: torch.Tensor, logits_static: torch.Tensor | None):
        self.model, self.graph, self.ids_static, self.logits_static = model, graph, ids_static, logits_static
        self.vocab = model.config.vocab_size
        self._replays = 0

    @classmethod
    @torch.no_grad()
    def capture(cls, model: LlamaGpuInferencer, warmup_token: int) -> "GraphedDecoder":
        if model.config.vocab_size == 0:
            raise ValueError("GraphedDecoder.capture: model vocab_size is 0")
        ids = torch.tensor([[int(warmup_token)]], dtype=torch.long, device=model.device)
        if model.device.type != "cuda":
            model.model(ids, last_token_only=True)
            return cls(model, None, ids, None)
        side = torch.cuda.Stream(model.device)
        side.wait_stream(torch.cuda.current_stream(model.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                model.model(ids, last_token_only=True)
        torch.cuda.current_stream(model.device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = model.model(ids, last_token_only=True)[0, -1]
        return cls(model, graph, ids, logits)

    @torch.no_grad()
    def decode_step(self, token: int) -> torch.Tensor:
        """``[vocab]`` fp32 on the host, bit-identical to ``model.forward_from_ids([token])``."""
        if not 0 <= int(token) < self.vocab:
            raise ValueError("decode_step: token id outside [0, %d)" % self.vocab)
        self.ids_static.fill_(int(token))
        self._replays += 1
        if self.graph is None:
            return self.model.model(self.ids_static, last_token_only=True)[0, -1].float().cpu()
        self.graph.replay()
        return self.logits_static.float().cpu()

    def num_replays(self) -> int:
        return self._replays

    def __repr__(self) -> str:
        return "GraphedDecoder(vocab=%d, num_replays=%d, graph=%s)" % (self.vocab, self._replays, self.graph is not None)
