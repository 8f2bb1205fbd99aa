"""Tensor-parallel training layers with sequence parallelism (forward *and* backward on the
fused collective GEMM kernels of ``csrc/tp_gemm.cu``).

The reference names these layers only in its design notes (.design/phase-7-distributed.md:269-307).
Layout (Megatron with sequence parallelism): the residual stream is sharded by rows -- rank r
holds rows ``[r*Ms, (r+1)*Ms)`` of the ``M = batch*seq`` token rows.

=====================  ==========================================  ====================================
layer                  forward                                     backward
=====================  ==========================================  ====================================
ColumnParallelLinear   ``Y = allgather(X) Wloc^T``   AG->GEMM      ``dX = reduce_scatter(dY Wloc)`` GEMM->RS;
                                                                   X re-gathered on a side stream while
                                                                   that GEMM runs; ``dW = dY^T Xfull``
RowParallelLinear      ``Y = reduce_scatter(X Wloc^T)`` GEMM->RS   ``dX = allgather(dY) Wloc``  AG->GEMM;
                                                                   ``dW = allgather(dY)^T X`` reads the
                                                                   rows the fused kernel just gathered
=====================  ==========================================  ====================================

``VocabParallelEmbedding`` and :func:`vocab_parallel_cross_entropy` shard the vocabulary; their
collectives (a reduce-scatter / all-gather of activations, two all-reduces of per-row scalars)
are not adjacent to a GEMM and go through ``torch.distributed``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..ops import functional as F
from .tensor_parallel import TPContext


def _accumulate_wgrad(w: torch.Tensor, a_t: torch.Tensor, b_t: torch.Tensor):
    """``dW (+)= a_t @ b_t.T`` into ``w.main_grad`` when the flat-arena trainer owns the gradient,
    else returned."""
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        F.gemm_nt(a_t, b_t, out=mg, accumulate=True)
        hook = getattr(w, "grad_ready_hook", None)
        if hook is not None:
            hook(w)
        return None
    return F.gemm_nt(a_t, b_t)


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_rows, w, bias, tp: TPContext, slots, M):
        f_ag, _, _ = slots
        K = w.shape[1]
        dst = tp.my_rows(f_ag, M, K)
        tp.wait_gather_buffer_free(f_ag)
        dst.copy_(x_rows)
        y = tp.ag_gemm(f_ag, M, w, bias)
        ctx.save_for_backward(x_rows, w)
        ctx.tp, ctx.slots, ctx.M, ctx.has_bias = tp, slots, M, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_rows, w = ctx.saved_tensors
        tp, (_, b_rs, b_ag), M = ctx.tp, ctx.slots, ctx.M
        K = w.shape[1]
        dy = dy if dy.is_contiguous() else dy.contiguous()
        cur = torch.cuda.current_stream()
        need_w = ctx.needs_input_grad[1]
        xg = None
        if need_w:
            if tp.world > 1:
                # re-gather the input rows for the weight gradient while the dgrad GEMM runs
                side = tp.side_stream
                side.wait_stream(cur)
                with torch.cuda.stream(side):
                    dst = tp.my_rows(b_ag, M, K)
                    tp.wait_gather_buffer_free(b_ag)
                    dst.copy_(x_rows)
                    xg = tp.all_gather_rows(b_ag, M, K)
            else:
                xg = x_rows
        dx = None
        if ctx.needs_input_grad[0]:
            dx = tp.gemm_rs(b_rs, dy, w, w_is_kn=True)
        dw = db = None
        if need_w:
            if tp.world > 1:
                cur.wait_stream(tp.side_stream)
            dw = _accumulate_wgrad(w, dy.t(), xg.t())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, residual_rows, tp: TPContext, slots, M):
        f_rs, _ = slots
        x = x if x.is_contiguous() else x.contiguous()
        out = tp.gemm_rs(f_rs, x, w, residual=residual_rows)
        ctx.save_for_backward(x, w)
        ctx.tp, ctx.slots, ctx.M, ctx.has_res = tp, slots, M, residual_rows is not None
        return out

    @staticmethod
    def backward(ctx, dout_rows):
        x, w = ctx.saved_tensors
        tp, (_, b_ag), M = ctx.tp, ctx.slots, ctx.M
        N = w.shape[0]
        dout_rows = dout_rows if dout_rows.is_contiguous() else dout_rows.contiguous()
        dst = tp.my_rows(b_ag, M, N)
        tp.wait_gather_buffer_free(b_ag)
        dst.copy_(dout_rows)
        # dX = allgather(dY) @ W : the fused kernel also leaves all of dY in the local gather buffer
        dx = tp.ag_gemm(b_ag, M, w, w_is_kn=True)
        dw = None
        if ctx.needs_input_grad[1]:
            dyg = tp.gather_buffer(b_ag, M, N)
            dw = _accumulate_wgrad(w, dyg.t(), x.t())
        return (dx if ctx.needs_input_grad[0] else None), dw, (dout_rows if ctx.has_res else None), None, None, None


class ColumnParallelLinear(nn.Module):
    """``[Ms, in]`` row shard -> ``[M, out/world]``; weight rows (outputs) are sharded.
    ``slots = (forward all-gather, backward reduce-scatter, backward re-gather)``."""

    def __init__(self, in_features: int, out_features_local: int, tp: TPContext, slots: tuple[int, int, int],
                 bias: bool = False, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.tp, self.slots = tp, tuple(slots)
        self.weight = nn.Parameter(torch.empty(out_features_local, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features_local, device=device, dtype=dtype)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x_rows: torch.Tensor, M: int) -> torch.Tensor:
        return _ColumnParallelFn.apply(x_rows, self.weight, self.bias, self.tp, self.slots, M)


class RowParallelLinear(nn.Module):
    """``[M, in/world]`` -> ``[Ms, out]`` row shard (+ residual rows); weight columns (inputs) are
    sharded.  ``slots = (forward reduce-scatter, backward all-gather)``."""

    def __init__(self, in_features_local: int, out_features: int, tp: TPContext, slots: tuple[int, int],
                 device=None, dtype=torch.bfloat16):
        super().__init__()
        self.tp, self.slots = tp, tuple(slots)
        self.weight = nn.Parameter(torch.empty(out_features, in_features_local, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor, M: int, residual_rows: torch.Tensor | None = None) -> torch.Tensor:
        return _RowParallelFn.apply(x, self.weight, residual_rows, self.tp, self.slots, M)


# --------------------------------------------------------------------------- vocabulary parallel
def _reduce_scatter_rows(full: torch.Tensor, group, rank: int, world: int) -> torch.Tensor:
    ms = full.shape[0] // world
    if full.is_cuda:
        out = torch.empty((ms,) + tuple(full.shape[1:]), device=full.device, dtype=full.dtype)
        dist.reduce_scatter_tensor(out, full, group=group)
        return out
    dist.all_reduce(full, group=group)      # gloo has no reduce-scatter
    return full[rank * ms:(rank + 1) * ms].clone()


def _all_gather_rows(rows: torch.Tensor, group, world: int) -> torch.Tensor:
    out = torch.empty((rows.shape[0] * world,) + tuple(rows.shape[1:]), device=rows.device, dtype=rows.dtype)
    if rows.is_cuda:
        dist.all_gather_into_tensor(out, rows.contiguous(), group=group)
    else:
        dist.all_gather(list(out.chunk(world)), rows.contiguous(), group=group)
    return out


class _VocabParallelEmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w, group, rank, world):
        v_loc = w.shape[0]
        lo = rank * v_loc
        ids = ids.reshape(-1)
        mask = (ids >= lo) & (ids < lo + v_loc)
        local = (ids - lo).clamp_(0, v_loc - 1)
        part = torch.nn.functional.embedding(local, w)
        part.mul_(mask.unsqueeze(-1).to(part.dtype))
        ctx.save_for_backward(local, mask, w)
        ctx.group, ctx.world = group, world
        if world == 1:
            return part
        assert part.shape[0] % world == 0, "token rows must divide by the tensor-parallel size"
        return _reduce_scatter_rows(part, group, rank, world)

    @staticmethod
    def backward(ctx, d_rows):
        local, mask, w = ctx.saved_tensors
        d = d_rows if ctx.world == 1 else _all_gather_rows(d_rows, ctx.group, ctx.world)
        d = d * mask.unsqueeze(-1).to(d.dtype)
        mg = getattr(w, "main_grad", None)
        if mg is not None:
            mg.index_add_(0, local, d.to(mg.dtype))
            return None, None, None, None, None
        dw = torch.zeros_like(w)
        dw.index_add_(0, local, d.to(w.dtype))
        return None, dw, None, None, None


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded by vocabulary rows; returns this rank's ``[Ms, H]`` row shard."""

    def __init__(self, vocab_local: int, hidden: int, group=None, rank: int = 0, world: int = 1, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.group, self.rank, self.world = group, rank, world
        self.weight = nn.Parameter(torch.empty(vocab_local, hidden, device=device, dtype=dtype))
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return _VocabParallelEmbeddingFn.apply(ids, self.weight, self.group, self.rank, self.world)


class _VocabParallelCEFn(torch.autograd.Function):
    """Mean next-token loss over vocabulary-sharded logits; the gradient is formed in the forward
    and kept in bf16 in place of the logits."""

    @staticmethod
    def forward(ctx, logits, target, group, rank, world, denom, ignore_index):
        M, v_loc = logits.shape
        lo = rank * v_loc
        lf = logits.float()
        mx = lf.max(dim=1).values
        if world > 1:
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
        lf.sub_(mx.unsqueeze(1))
        tmask = (target >= lo) & (target < lo + v_loc)
        tl = (target - lo).clamp(0, v_loc - 1)
        packed = torch.empty((2, M), device=logits.device, dtype=torch.float32)
        packed[1] = lf.gather(1, tl.unsqueeze(1)).squeeze(1) * tmask
        lf.exp_()
        packed[0] = lf.sum(1)
        if world > 1:
            dist.all_reduce(packed, group=group)
        se, tlogit = packed[0], packed[1]
        valid = target != ignore_index
        n = float(denom) if denom is not None else float(valid.sum().clamp_min(1))
        loss = ((se.log() - tlogit) * valid).sum() / n
        lf.div_(se.unsqueeze(1))
        lf[torch.arange(M, device=logits.device), tl] -= tmask.to(lf.dtype)
        lf.mul_((valid.to(lf.dtype) / n).unsqueeze(1))
        ctx.save_for_backward(lf.to(logits.dtype))
        return loss

    @staticmethod
    def backward(ctx, dloss):
        (g,) = ctx.saved_tensors
        return g * dloss.to(g.dtype), None, None, None, None, None, None


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, target: torch.Tensor, group=None, rank: int = 0,
                                 world: int = 1, denominator: int | None = None,
                                 ignore_index: int = -100) -> torch.Tensor:
    """``logits_local``: ``[M, V/world]`` (this rank's vocabulary columns of every row);
    ``target``: ``[M]`` global ids."""
    return _VocabParallelCEFn.apply(logits_local, target.reshape(-1), group, rank, world, denominator, ignore_index)


def all_reduce_replicated_grads(params, group) -> None:
    """Sum the gradients of parameters every rank holds a full copy of (norm weights): under
    sequence parallelism each rank only saw its own rows."""
    if group is None or dist.get_world_size(group) == 1:
        return
    grads = []
    for p in params:
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            grads.append(g)
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g).to(g.dtype))
        off += g.numel()
