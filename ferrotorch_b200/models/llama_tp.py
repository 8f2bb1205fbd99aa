"""Llama for tensor-parallel *training* with sequence parallelism.

Each rank holds ``1/world`` of every projection (heads for attention, FFN columns for the MLP,
vocabulary rows for the embedding and the lm_head) and ``1/world`` of the token rows of the
residual stream.  The four projections of a block run on the fused collective GEMMs in forward
and backward (``parallel/tp_layers.py``); RMSNorm, RoPE, flash attention, SwiGLU, the optimizer
and the loss are the same kernels the single-GPU model uses.

The reference trains Llama on one device only (ferrotorch-llama/src/model.rs:75-189 is its
decoder; tensor parallelism is a design note, .design/phase-7-distributed.md:269-307).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..nn.layers import RMSNorm, RotaryPositionEmbedding
from ..ops import functional as F
from ..ops.attention import packed_attention
from ..parallel.tensor_parallel import TPContext
from ..parallel.tp_layers import (ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding,
                                  all_reduce_replicated_grads, vocab_parallel_cross_entropy)
from .llama import LlamaConfig, LlamaForCausalLM

# symmetric-buffer slots: (forward, backward ...) per projection
SLOTS_QKV = (0, 5, 6)
SLOTS_O = (1, 7)
SLOTS_GU = (2, 8, 9)
SLOTS_DOWN = (3, 10)
SLOTS_LM = (4, 11, 12)


class TPLlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, rope: RotaryPositionEmbedding, device=None):
        super().__init__()
        W = tp.world
        assert cfg.num_attention_heads % W == 0 and cfg.num_key_value_heads % W == 0 and cfg.intermediate_size % W == 0
        self.hq, self.hkv, self.d = cfg.num_attention_heads // W, cfg.num_key_value_heads // W, cfg.head_dim
        self.i_loc = cfg.intermediate_size // W
        H = cfg.hidden_size
        self.rope, self.act, self.act_param = rope, cfg.hidden_act, cfg.hidden_act_param
        self.input_layernorm = RMSNorm(H, cfg.rms_norm_eps).to(device=device, dtype=torch.bfloat16)
        self.post_attention_layernorm = RMSNorm(H, cfg.rms_norm_eps).to(device=device, dtype=torch.bfloat16)
        self.qkv_proj = ColumnParallelLinear(H, (self.hq + 2 * self.hkv) * self.d, tp, SLOTS_QKV, device=device)
        self.o_proj = RowParallelLinear(self.hq * self.d, H, tp, SLOTS_O, device=device)
        self.gate_up_proj = ColumnParallelLinear(H, 2 * self.i_loc, tp, SLOTS_GU, device=device)
        self.down_proj = RowParallelLinear(self.i_loc, H, tp, SLOTS_DOWN, device=device)

    def forward(self, x_rows: torch.Tensor, B: int, S: int) -> torch.Tensor:
        M = B * S
        h = self.input_layernorm(x_rows)
        qkv = self.qkv_proj(h, M).view(B, S, self.hq + 2 * self.hkv, self.d)
        cos, sin = self.rope._tables(x_rows.device)
        a = packed_attention(qkv, cos, sin, n_heads=self.hq, n_kv_heads=self.hkv, head_dim=self.d,
                             interleaved=self.rope.interleaved)
        x_rows = self.o_proj(a.view(M, self.hq * self.d), M, x_rows)
        h = self.post_attention_layernorm(x_rows)
        act = F.swiglu(self.gate_up_proj(h, M), self.act, self.act_param)
        return self.down_proj(act, M, x_rows)


class TPLlamaForCausalLM(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp: TPContext, device=None):
        super().__init__()
        self.config, self.tp = cfg, tp
        device = device or tp.device
        W = tp.world
        assert cfg.vocab_size % W == 0, "vocabulary must divide by the tensor-parallel size"
        assert not cfg.tie_word_embeddings, "tied embeddings are not sharded here"
        self.v_loc = cfg.vocab_size // W
        self.rope = RotaryPositionEmbedding(cfg.head_dim, cfg.max_position_embeddings, cfg.rope_theta,
                                            scaling=cfg.rope_scaling)
        self.embed_tokens = VocabParallelEmbedding(self.v_loc, cfg.hidden_size, tp.group, tp.rank, W, device=device)
        self.layers = nn.ModuleList(TPLlamaBlock(cfg, tp, self.rope, device) for _ in range(cfg.num_hidden_layers))
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps).to(device=device, dtype=torch.bfloat16)
        self.lm_head = ColumnParallelLinear(cfg.hidden_size, self.v_loc, tp, SLOTS_LM, device=device)
        self.checkpoint_layers = False

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, *,
                loss_denominator: int | None = None):
        """Mean next-token loss (``labels`` already shifted), identical on every rank; without
        ``labels`` returns this rank's vocabulary columns of the logits ``[B*S, V/world]``."""
        B, S = input_ids.shape
        M = B * S
        assert M % self.tp.world == 0, "batch*seq must divide by the tensor-parallel size"
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            if self.checkpoint_layers and self.training and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint

                x = checkpoint(lambda a, l=layer: l(a, B, S), x, use_reentrant=False)
            else:
                x = layer(x, B, S)
        logits = self.lm_head(self.norm(x), M)
        if labels is None:
            return logits
        return vocab_parallel_cross_entropy(logits, labels, self.tp.group, self.tp.rank, self.tp.world,
                                            loss_denominator)

    # ------------------------------------------------------------------ replicated parameters
    def replicated_parameters(self):
        return [p for n, p in self.named_parameters() if n.endswith("layernorm.weight") or n == "norm.weight"]

    def sync_replicated_grads(self) -> None:
        all_reduce_replicated_grads(self.replicated_parameters(), self.tp.group)

    # ------------------------------------------------------------------ sharding a full model
    @torch.no_grad()
    def load_full(self, full: LlamaForCausalLM) -> "TPLlamaForCausalLM":
        """Copy this rank's shards out of an unsharded model (same config)."""
        c, r, W = self.config, self.tp.rank, self.tp.world
        D = c.head_dim
        nq, nkv = c.num_attention_heads * D, c.num_key_value_heads * D

        def rows(t, lo, n):
            return t[lo:lo + n]

        self.embed_tokens.weight.copy_(rows(full.model.embed_tokens.weight, r * self.v_loc, self.v_loc))
        self.lm_head.weight.copy_(rows(full.lm_head.weight, r * self.v_loc, self.v_loc))
        self.norm.weight.copy_(full.model.norm.weight)
        for mine, ref in zip(self.layers, full.model.layers):
            mine.input_layernorm.weight.copy_(ref.input_layernorm.weight)
            mine.post_attention_layernorm.weight.copy_(ref.post_attention_layernorm.weight)
            wq, wk, wv = ref.self_attn.qkv_proj.weight.split([nq, nkv, nkv], dim=0)
            ql, kl = nq // W, nkv // W
            mine.qkv_proj.weight.copy_(torch.cat([rows(wq, r * ql, ql), rows(wk, r * kl, kl), rows(wv, r * kl, kl)]))
            mine.o_proj.weight.copy_(ref.self_attn.o_proj.weight[:, r * ql:(r + 1) * ql])
            g, u = ref.mlp.gate_up_proj.weight.chunk(2, dim=0)
            il = mine.i_loc
            mine.gate_up_proj.weight.copy_(torch.cat([rows(g, r * il, il), rows(u, r * il, il)]))
            mine.down_proj.weight.copy_(ref.mlp.down_proj.weight[:, r * il:(r + 1) * il])
        return self

    def full_grad_slices(self, full: LlamaForCausalLM) -> list[tuple[str, torch.Tensor, torch.Tensor]]:
        """``(name, this rank's gradient, matching slice of the unsharded model's gradient)`` for
        every parameter -- what an equivalence test compares."""
        c, r, W = self.config, self.tp.rank, self.tp.world
        D = c.head_dim
        nq, nkv = c.num_attention_heads * D, c.num_key_value_heads * D
        ql, kl = nq // W, nkv // W

        def g(p):
            mg = getattr(p, "main_grad", None)
            return mg if mg is not None else p.grad

        out = [("embed", g(self.embed_tokens.weight), g(full.model.embed_tokens.weight)[r * self.v_loc:(r + 1) * self.v_loc]),
               ("lm_head", g(self.lm_head.weight), g(full.lm_head.weight)[r * self.v_loc:(r + 1) * self.v_loc]),
               ("norm", g(self.norm.weight), g(full.model.norm.weight))]
        for i, (mine, ref) in enumerate(zip(self.layers, full.model.layers)):
            gq, gk, gv = g(ref.self_attn.qkv_proj.weight).split([nq, nkv, nkv], dim=0)
            out.append(("l%d.qkv" % i, g(mine.qkv_proj.weight),
                        torch.cat([gq[r * ql:(r + 1) * ql], gk[r * kl:(r + 1) * kl], gv[r * kl:(r + 1) * kl]])))
            out.append(("l%d.o" % i, g(mine.o_proj.weight), g(ref.self_attn.o_proj.weight)[:, r * ql:(r + 1) * ql]))
            gg, gu = g(ref.mlp.gate_up_proj.weight).chunk(2, dim=0)
            il = mine.i_loc
            out.append(("l%d.gu" % i, g(mine.gate_up_proj.weight),
                        torch.cat([gg[r * il:(r + 1) * il], gu[r * il:(r + 1) * il]])))
            out.append(("l%d.down" % i, g(mine.down_proj.weight), g(ref.mlp.down_proj.weight)[:, r * il:(r + 1) * il]))
            out.append(("l%d.ln1" % i, g(mine.input_layernorm.weight), g(ref.input_layernorm.weight)))
            out.append(("l%d.ln2" % i, g(mine.post_attention_layernorm.weight), g(ref.post_attention_layernorm.weight)))
        return out


def make_tp_trainer(model: TPLlamaForCausalLM, **kw):
    """A :class:`FlatTrainer` over this rank's shards; the replicated norm weights' gradients are
    summed over the tensor-parallel group before every update."""
    from ..train.engine import FlatTrainer

    tr = FlatTrainer(model, **kw)
    tr.pre_update = model.sync_replicated_grads
    if model.tp.world > 1:
        tr.model_parallel_group = model.tp.group
    return tr


def hybrid_groups(tp_size: int, backend: str | None = None):
    """Split the default process group into a ``dp x tp`` mesh, rank ``= dp_index * tp_size +
    tp_index`` (tensor-parallel peers are neighbours, i.e. share a node's NVLink domain).  Every
    rank must call this; returns ``(tp_group, dp_group)`` of the calling rank
    (device_mesh.rs:37-203 gives the same row-major rank <-> coordinate maps)."""
    import torch.distributed as dist

    world, rank = dist.get_world_size(), dist.get_rank()
    if tp_size <= 0 or world % tp_size:
        raise ValueError("hybrid_groups: world size %d is not a multiple of tp_size %d" % (world, tp_size))
    dp_size = world // tp_size
    mine_tp = mine_dp = None
    for d in range(dp_size):
        ranks = list(range(d * tp_size, (d + 1) * tp_size))
        g = dist.new_group(ranks, backend=backend)
        if rank in ranks:
            mine_tp = g
    for t in range(tp_size):
        ranks = list(range(t, world, tp_size))
        g = dist.new_group(ranks, backend=backend)
        if rank in ranks:
            mine_dp = g
    return mine_tp, mine_dp


def add_data_parallel(trainer, dp_group):
    """Average the gradient arena of a :class:`FlatTrainer` over ``dp_group`` before every update
    (after whatever ``pre_update`` hook it already has, before the norm / clip).  With a
    tensor-parallel trainer this gives TP x DP: the TP collectives are the fused kernels, the DP
    reduction is one all-reduce of the arena on the process group's own back-end."""
    import torch.distributed as dist

    inner = trainer.pre_update

    def hook():
        if inner is not None:
            inner()
        n = dist.get_world_size(dp_group)
        if n > 1:
            g = trainer.arena.grads
            if g.is_cuda:
                dist.all_reduce(g, op=dist.ReduceOp.AVG, group=dp_group)
            else:                                   # gloo has no AVG
                dist.all_reduce(g, group=dp_group)
                g.div_(n)

    trainer.pre_update = hook
    return trainer


def make_hybrid_trainer(model: TPLlamaForCausalLM, dp_group, **kw):
    """:func:`make_tp_trainer` plus data parallelism across ``dp_group`` (see :func:`hybrid_groups`)."""
    return add_data_parallel(make_tp_trainer(model, **kw), dp_group)
