"""Batched Llama inference engine: prefill + paged-KV greedy decode, single GPU or tensor parallel.

The reference's GPU inferencer is batch-1 and cache-less -- every new token re-runs the whole
prefix through 9 GEMMs + 16 elementwise launches per layer
(ferrotorch-llama/src/gpu.rs:300-334, 549-788) -- and ``GraphedDecoder`` captures that seq=1
forward in a CUDA graph (gpu.rs:896-994).  This engine keeps a paged KV cache on the device
(block 16), prefills with flash attention, decodes one token per sequence per step with the
paged decode kernel, and shards the model Megatron-style across a tensor-parallel group:

    residual stream rows sharded by rank (sequence parallel)
    RMSNorm(own rows) -> gather buffer -> [all-gather -> QKV GEMM] -> RoPE -> KV append
      -> attention (local heads) -> [o_proj GEMM -> reduce-scatter + residual]
      -> RMSNorm -> [all-gather -> gate/up GEMM] -> SwiGLU -> [down GEMM -> reduce-scatter + residual]

Bracketed steps are single fused kernels (``csrc/tp_gemm.cu``).  With one rank the same kernels
run with an empty collective part.

``weight_format="q4_0"`` keeps the linear weights as GGUF Q4_0 planes (0.5625 bytes per element,
ferrotorch-serialize/src/gguf.rs:543-545; the reference dequantises whole tensors to bf16 at load
time, ferrotorch-llama/src/gpu_gguf.rs:336).  The column-parallel layers then run as this
library's gather kernel followed by the dequant-GEMM (``csrc/quant_gemm.cu``) on the gathered
rows, the row-parallel ones as the dequant-GEMM followed by an NCCL reduce-scatter and the
residual add: two launches per layer instead of one fused kernel.
"""
from __future__ import annotations


import zlib

import torch
import torch.distributed as dist

from .. import _native
from ..nn.paged import PagedAttentionManager, PagedKVCache
from ..ops import functional as F
from ..ops import reference as ref
from ..ops.quant import q4_0_linear, quantize_q4_0_planes
from ..parallel.tensor_parallel import TPContext
from .llama import LlamaConfig


def _shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


class LlamaEngine:
    def __init__(self, cfg: LlamaConfig, tp: TPContext | None = None, *, max_batch: int = 64,
                 max_seq_len: int = 4096, block_size: int = 16, weights: dict | None = None, seed: int = 0,
                 device=None, prefill_chunk_tokens: int = 16384, cuda_graph: bool = False,
                 weight_format: str = "bf16"):
        assert weight_format in ("bf16", "q4_0")
        if cfg.hidden_act not in F._ACT_ID:
            raise NotImplementedError("LlamaEngine: hidden_act %r has no fused kernel (use LlamaForCausalLM)" % cfg.hidden_act)
        self.weight_format = weight_format
        self.cfg = cfg
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.tp = tp if tp is not None else TPContext(None, self.device)
        W, r = self.tp.world, self.tp.rank
        self.W, self.r = W, r
        assert cfg.num_attention_heads % W == 0 and cfg.num_key_value_heads % W == 0 and cfg.intermediate_size % W == 0
        self.Hq, self.Hkv, self.D = cfg.num_attention_heads // W, cfg.num_key_value_heads // W, cfg.head_dim
        self.F = cfg.intermediate_size // W
        self.H = cfg.hidden_size
        self.Vloc = (cfg.vocab_size + W - 1) // W
        self.prefill_chunk_tokens = prefill_chunk_tokens
        self.cuda_graph = cuda_graph
        self._graph, self._graph_batch, self._eager_steps = None, 0, 0
        self.max_batch = max_batch
        self.cos, self.sin = ref.rope_tables(cfg.head_dim, max(max_seq_len, 16), cfg.rope_theta, cfg.rope_scaling,
                                             device=self.device)
        n_blocks = max_batch * ((max_seq_len + block_size - 1) // block_size)
        self.cache = PagedKVCache(cfg.num_hidden_layers, self.Hkv, self.D, n_blocks, max_batch, max_seq_len,
                                  block_size, self.device)
        self.manager = PagedAttentionManager(self.cache)
        self._load(weights, seed)

    @classmethod
    def from_pretrained(cls, path: str, tp: TPContext | None = None, **kw) -> "LlamaEngine":
        """An engine over the weights of a Hugging Face model directory (``config.json`` and
        SafeTensors, single file or sharded); every rank reads the files and keeps its shard."""
        import os

        from ..serialize.state import load_safetensors_auto

        cfg = LlamaConfig.from_hf(os.path.join(path, "config.json"))
        sd = load_safetensors_auto(path)
        if "lm_head.weight" not in sd:
            sd["lm_head.weight"] = sd["model.embed_tokens.weight"]
        return cls(cfg, tp, weights=sd, **kw)

    # ------------------------------------------------------------------ weights
    def _load(self, sd: dict | None, seed: int) -> None:
        cfg, dev, W, r = self.cfg, self.device, self.W, self.r
        std = cfg.initializer_range
        g = torch.Generator(device=dev)

        def rnd(shape, tag):
            g.manual_seed(zlib.crc32(repr((seed, tag)).encode()) & 0x7FFFFFFF)   # same on every rank and run
            return (torch.randn(shape, device=dev, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)

        def get(name, shape, tag, shard=None):
            if sd is None:
                return rnd(shape, tag)
            w = sd[name].to(dev, torch.bfloat16)
            return shard(w).contiguous() if shard is not None else w.contiguous()

        D, nq, nkv = self.D, cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
        self.embed = get("model.embed_tokens.weight", (cfg.vocab_size, self.H), ("embed",))
        self.layers = []
        for i in range(cfg.num_hidden_layers):
            pre = "model.layers.%d." % i
            if sd is None:
                qkv = rnd(((self.Hq + 2 * self.Hkv) * D, self.H), (i, "qkv", r))
                gu = rnd((2 * self.F, self.H), (i, "gu", r))
                o = rnd((self.H, self.Hq * D), (i, "o", r))
                dn = rnd((self.H, self.F), (i, "down", r))
                n1 = torch.ones(self.H, device=dev, dtype=torch.bfloat16)
                n2 = torch.ones(self.H, device=dev, dtype=torch.bfloat16)
            else:
                q = _shard_rows(sd[pre + "self_attn.q_proj.weight"], r, W)
                k = _shard_rows(sd[pre + "self_attn.k_proj.weight"], r, W)
                v = _shard_rows(sd[pre + "self_attn.v_proj.weight"], r, W)
                qkv = torch.cat([q, k, v], 0).to(dev, torch.bfloat16).contiguous()
                gu = torch.cat([_shard_rows(sd[pre + "mlp.gate_proj.weight"], r, W),
                                _shard_rows(sd[pre + "mlp.up_proj.weight"], r, W)], 0).to(dev, torch.bfloat16).contiguous()
                ow = sd[pre + "self_attn.o_proj.weight"]
                o = ow[:, r * self.Hq * D:(r + 1) * self.Hq * D].to(dev, torch.bfloat16).contiguous()
                dw = sd[pre + "mlp.down_proj.weight"]
                dn = dw[:, r * self.F:(r + 1) * self.F].to(dev, torch.bfloat16).contiguous()
                n1 = sd[pre + "input_layernorm.weight"].to(dev, torch.bfloat16)
                n2 = sd[pre + "post_attention_layernorm.weight"].to(dev, torch.bfloat16)
            if self.weight_format == "q4_0":
                qkv, gu, o, dn = (quantize_q4_0_planes(w) for w in (qkv, gu, o, dn))
            self.layers.append(dict(qkv=qkv, gu=gu, o=o, down=dn, n1=n1, n2=n2))
        self.norm = (torch.ones(self.H, device=dev, dtype=torch.bfloat16) if sd is None
                     else sd["model.norm.weight"].to(dev, torch.bfloat16))
        if sd is None:
            self.lm_head = rnd((self.Vloc, self.H), ("lm_head", r))
        else:
            full = sd.get("lm_head.weight", sd["model.embed_tokens.weight"])
            lo = r * self.Vloc
            shard = full[lo:lo + self.Vloc].to(dev, torch.bfloat16)
            if shard.shape[0] < self.Vloc:  # pad the last shard; padded rows can never win the argmax
                shard = torch.cat([shard, torch.zeros(self.Vloc - shard.shape[0], self.H, device=dev, dtype=torch.bfloat16)])
            self.lm_head = shard.contiguous()
        if self.weight_format == "q4_0":
            if self.Vloc % 8:                   # the dequant-GEMM wants N % 8 == 0: pad with zero rows
                pad = 8 - self.Vloc % 8
                self.lm_head = torch.cat([self.lm_head, torch.zeros(pad, self.H, device=dev, dtype=torch.bfloat16)])
            self.lm_head = quantize_q4_0_planes(self.lm_head)

    # ------------------------------------------------------------------ one transformer pass
    def _rows(self, M: int):
        ms = self.tp.rows_per_rank(M)
        lo = min(M, self.r * ms)
        return lo, min(M, lo + ms)

    def _norm_into(self, slot: int, x_rows: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, M: int):
        """RMSNorm of this rank's rows (optionally fused with a residual add) written straight into
        the gather buffer of ``slot``; returns the updated residual rows."""
        dst = self.tp.my_rows(slot, M, self.H)
        self.tp.wait_gather_buffer_free(slot)
        rows = x_rows.shape[0]
        if rows == 0:
            return x_rows
        lib = _native.kernels()
        if delta is None:
            rc = lib.ft_rmsnorm_fwd(x_rows.data_ptr(), None, w.data_ptr(), dst.data_ptr(), None, None, rows, self.H,
                                    self.cfg.rms_norm_eps, self.device.index, F._stream())
            out = x_rows
        else:
            out = torch.empty_like(x_rows)
            rc = lib.ft_rmsnorm_fwd(x_rows.data_ptr(), delta.data_ptr(), w.data_ptr(), dst.data_ptr(), out.data_ptr(),
                                    None, rows, self.H, self.cfg.rms_norm_eps, self.device.index, F._stream())
        _native.check(rc, "ft_rmsnorm_fwd")
        return out

    def _col(self, slot: int, M: int, w) -> torch.Tensor:
        """Column-parallel linear on the gather buffer of ``slot``: ``[M, N_loc]``."""
        if not isinstance(w, tuple):
            if self.W == 1 and M <= 128:
                # one GPU, decode-sized batch: the weight-stationary small-batch GEMM
                return F.gemm_small_m(self.tp.gather_buffer(slot, M, self.H), w)
            return self.tp.ag_gemm(slot, M, w)
        xg = self.tp.gather_buffer(slot, M, self.H) if self.W == 1 else self.tp.all_gather_rows(slot, M, self.H)
        return q4_0_linear(xg, w[0], w[1])

    def _row(self, slot: int, a: torch.Tensor, w, residual: torch.Tensor) -> torch.Tensor:
        """Row-parallel linear + reduce-scatter + residual add: this rank's rows ``[rows, H]``."""
        if not isinstance(w, tuple):
            if self.W == 1 and a.shape[0] <= 128:
                return F.gemm_small_m(a, w, residual=residual)    # residual added by its split-K finalize pass
            return self.tp.gemm_rs(slot, a, w, residual=residual)
        y = q4_0_linear(a, w[0], w[1])
        if self.W == 1:
            return y.add_(residual)
        M, ms = a.shape[0], self.tp.rows_per_rank(a.shape[0])
        if M < self.W * ms:
            y = torch.cat([y, y.new_zeros(self.W * ms - M, self.H)])
        mine = torch.empty((ms, self.H), device=self.device, dtype=y.dtype)
        dist.reduce_scatter_tensor(mine, y, group=self.tp.group)
        return mine[:residual.shape[0]].add_(residual)

    def _forward(self, tokens: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor | None,
                 B: int, S: int, decode: bool, ctx_len: torch.Tensor | None) -> torch.Tensor:
        """tokens: flat [M] ids.  Returns this rank's rows of the final hidden state [rows, H]
        (before the final norm) and leaves nothing else behind."""
        M = tokens.numel()
        lo, hi = self._rows(M)
        x = F.embedding(tokens[lo:hi], self.embed) if hi > lo else torch.empty((0, self.H), device=self.device, dtype=torch.bfloat16)
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        nh = Hq + 2 * Hkv
        for li, L in enumerate(self.layers):
            self._norm_into(0, x, None, L["n1"], M)
            qkv = self._col(0, M, L["qkv"]).view(M, nh, D)
            F._rope_launch(qkv, self.cos, self.sin, positions, Hq + Hkv, S, 0, False, False)
            k, v = qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
            self.cache.append(li, k, v, positions, seq_ids, tokens_per_seq=S)
            if decode:
                attn = self.cache.decode(li, qkv[:, :Hq], ctx_len)
            else:
                q4 = qkv.view(B, S, nh, D)
                attn, _ = F.flash_attn_fwd(q4[:, :, :Hq], q4[:, :, Hq:Hq + Hkv], q4[:, :, Hq + Hkv:], True,
                                           return_lse=False)
            # o_proj + reduce-scatter + residual add  -> new residual rows
            x = self._row(1, attn.reshape(M, Hq * D), L["o"], x)
            self._norm_into(2, x, None, L["n2"], M)
            gu = self._col(2, M, L["gu"])
            act = torch.empty((M, self.F), device=self.device, dtype=torch.bfloat16)
            rc = _native.kernels().ft_swiglu_fwd(gu.data_ptr(), act.data_ptr(), M, self.F, gu.stride(0),
                                                 F._ACT_ID[self.cfg.hidden_act],
                                                 self.device.index, F._stream())
            _native.check(rc, "ft_swiglu_fwd")
            x = self._row(3, act, L["down"], x)
        return x

    def _local_argmax(self, h_rows: torch.Tensor, M: int) -> torch.Tensor:
        """Final norm + this rank's vocabulary shard of the lm_head -> ``[M, 2]`` (best logit, global id)."""
        self._norm_into(4, h_rows, None, self.norm, M)
        logits = self._col(4, M, self.lm_head)[:, :self.Vloc].float()
        if self.cfg.vocab_size % self.W and self.r == self.W - 1:
            logits[:, self.cfg.vocab_size - self.r * self.Vloc:] = -float("inf")
        val, idx = logits.max(dim=-1)
        return torch.stack([val, (idx + self.r * self.Vloc).float()], dim=-1).contiguous()

    def _combine_argmax(self, pair: torch.Tensor) -> torch.Tensor:
        """Greedy token over all vocabulary shards (a 512-byte all-gather; kept outside any
        captured graph so that the graph holds only this library's kernels and torch ops)."""
        if self.W == 1:
            return pair[:, 1].long()
        allp = torch.empty((self.W,) + tuple(pair.shape), device=self.device, dtype=pair.dtype)
        dist.all_gather_into_tensor(allp, pair, group=self.tp.group)
        best = allp[..., 0].argmax(dim=0)
        return allp[..., 1].gather(0, best[None]).squeeze(0).long()

    def _next_tokens(self, h_rows: torch.Tensor, M: int) -> torch.Tensor:
        return self._combine_argmax(self._local_argmax(h_rows, M))

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        """``prompts [B, S]`` token ids (all sequences the same length).  Fills the KV cache and
        returns the first generated token of every sequence ``[B]``."""
        B, S = prompts.shape
        for b in list(self.manager.active):
            self.manager.remove_sequence(b)
        self.seqs = [self.manager.add_sequence(S) for _ in range(B)]
        assert self.seqs == list(range(B)), "sequence slots must be 0..B-1 after a reset"
        if getattr(self, "lengths", None) is not None and self.lengths.numel() == B:
            self.lengths.fill_(S)           # keep the tensor a captured graph refers to
        else:
            self.lengths = torch.full((B,), S, device=self.device, dtype=torch.int32)
            self._graph = None
        per = max(1, self.prefill_chunk_tokens // S)
        firsts = []
        for b0 in range(0, B, per):
            b1 = min(B, b0 + per)
            nb = b1 - b0
            toks = prompts[b0:b1].reshape(-1).to(self.device)
            pos = torch.arange(S, device=self.device, dtype=torch.int32).repeat(nb)
            sid = torch.arange(b0, b1, device=self.device, dtype=torch.int32).repeat_interleave(S)
            h = self._forward(toks, pos, sid, nb, S, False, None)
            # last-token rows of this chunk -> [nb, H] on every rank (rows live on different ranks)
            M = nb * S
            lo, hi = self._rows(M)
            last = torch.zeros((nb, self.H), device=self.device, dtype=torch.float32)
            want = torch.arange(nb, device=self.device) * S + (S - 1)
            mine = (want >= lo) & (want < hi)
            if bool(mine.any()):
                last[mine] = h[(want[mine] - lo)].float()
            if self.W > 1:
                dist.all_reduce(last, group=self.tp.group)
            lo2, hi2 = self._rows(nb)
            firsts.append(self._next_tokens(last[lo2:hi2].to(torch.bfloat16).contiguous(), nb))
        return torch.cat(firsts)

    def _decode_device(self, tokens: torch.Tensor) -> torch.Tensor:
        """The device part of a decode step (everything a CUDA graph captures)."""
        B = tokens.numel()
        pos = self.lengths.clone()          # position of the new token
        self.lengths += 1
        h = self._forward(tokens, pos, self._sid, B, 1, True, self.lengths)
        return self._local_argmax(h, B)

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """One greedy step: ``tokens [B]`` (the previous step's output) -> next tokens ``[B]``.

        With ``cuda_graph=True`` the device part is captured once (after two eager steps that size
        every buffer) and replayed: the reference's ``GraphedDecoder`` idea
        (ferrotorch-llama/src/gpu.rs:896-994) extended to the tensor-parallel step -- the fused
        collective kernels keep their epochs in device memory, so a replay stays in step with
        the other ranks."""
        B = tokens.numel()
        for s in self.seqs:
            self.manager.extend(s, 1)       # host bookkeeping: new pages when a block fills up
        self.cache.sync_table()
        if getattr(self, "_sid", None) is None or self._sid.numel() != B:
            self._sid = torch.arange(B, device=self.device, dtype=torch.int32)
        tokens = tokens.to(self.device)
        if not self.cuda_graph:
            return self._combine_argmax(self._decode_device(tokens))
        if self._graph is not None and self._graph_batch == B:
            self._tok_in.copy_(tokens)
            self._graph.replay()
            return self._combine_argmax(self._pair_out)
        self._eager_steps += 1
        if self._eager_steps <= 2:
            return self._combine_argmax(self._decode_device(tokens))
        self._tok_in = tokens.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._pair_out = self._decode_device(self._tok_in)
        self._graph, self._graph_batch = g, B
        g.replay()                           # capture only records; this executes the step
        return self._combine_argmax(self._pair_out)

    @torch.no_grad()
    def sample_step(self, tokens: torch.Tensor, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                    seed: int = 0) -> torch.Tensor:
        """One decode step that samples instead of taking the arg-max: temperature, top-k and
        nucleus sampling on the vocabulary-sharded logits (``parallel/vocab_sampling.py``: candidates
        and softmax normaliser are exchanged, never the ``[B, V]`` logits; every rank draws the same
        token from ``(seed, step)``).  Runs eagerly (the candidate exchange is a library collective,
        which stays outside captured graphs here)."""
        from ..parallel.backend import SimulatedGroup, TorchGroup
        from ..parallel.vocab_sampling import sample_vocab_parallel, shared_uniform

        B = tokens.numel()
        for s in self.seqs:
            self.manager.extend(s, 1)
        self.cache.sync_table()
        if getattr(self, "_sid", None) is None or self._sid.numel() != B:
            self._sid = torch.arange(B, device=self.device, dtype=torch.int32)
        pos = self.lengths.clone()
        self.lengths += 1
        h = self._forward(tokens.to(self.device), pos, self._sid, B, 1, True, self.lengths)
        self._norm_into(4, h, None, self.norm, B)
        logits = self._col(4, B, self.lm_head)[:, :self.Vloc]
        group = TorchGroup(self.tp.group) if self.W > 1 else SimulatedGroup.create_group(1)[0]
        valid = min(self.Vloc, max(0, self.cfg.vocab_size - self.r * self.Vloc))
        self._sample_steps = getattr(self, "_sample_steps", 0) + 1
        u = shared_uniform(B, seed, self._sample_steps, self.device)
        return sample_vocab_parallel(logits, group, self.r * self.Vloc, u, temperature, top_k, top_p, valid=valid)

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 seed: int = 0) -> torch.Tensor:
        """Greedy by default (graph-replayed decode steps); ``temperature > 0`` samples every token
        after the first with :meth:`sample_step`."""
        tok = self.prefill(prompts)
        out = [tok]
        for _ in range(max_new_tokens - 1):
            tok = self.decode_step(tok) if temperature <= 0.0 else self.sample_step(tok, temperature, top_k, top_p, seed)
            out.append(tok)
        return torch.stack(out, dim=1)
