#!/usr/bin/env python
"""Plain-PyTorch tensor-parallel baselines for the Llama benchmarks: a Megatron-style sharded model
(column-parallel QKV / gate-up, row-parallel o_proj / down_proj with an NCCL all-reduce after
each, vocabulary-parallel lm_head and cross-entropy) built only from torch operators: cuBLAS,
``scaled_dot_product_attention``, ``torch.optim.AdamW(fused=True)``, ``torch.distributed``.
None of this library's kernels run here; it is the same-box bar for ``benchmarks/bench_train_tp.py``
(``--mode train``) and ``benchmarks/bench_inference.py`` (``--mode decode``).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_torch_tp.py --mode train
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_torch_tp.py --mode decode

Same data shapes as the benchmarks they stand beside: training on a global batch of 32 x 4096
random tokens per optimizer step (micro-batches of ``--micro-batch-seqs`` sequences, every rank
sees the whole micro-batch, as tensor parallelism requires), bf16 parameters, fp32 AdamW moments
through ``fused=True``; decoding a batch of 64 prompts of 2048 tokens for 256 greedy steps with
a static KV cache.  CUDA events, max over ranks.  ``--device cpu`` runs the same code over gloo
(used by the unit test on a miniature model).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

SHAPES = {
    "llama3-8b": dict(vocab=128256, hidden=4096, ffn=14336, layers=32, heads=32, kv_heads=8, theta=500000.0),
    "llama3-70b": dict(vocab=128256, hidden=8192, ffn=28672, layers=80, heads=64, kv_heads=8, theta=500000.0),
    "tiny": dict(vocab=512, hidden=64, ffn=128, layers=2, heads=4, kv_heads=2, theta=10000.0),
}


class _CopyToRanks(torch.autograd.Function):          # identity forward, all-reduce backward (Megatron's f)
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromRanks(torch.autograd.Function):     # all-reduce forward, identity backward (Megatron's g)
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def _rope(x, cos, sin):
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


class Block(nn.Module):
    def __init__(self, s, world, dtype, device):
        super().__init__()
        self.hq, self.hkv, self.d = s["heads"] // world, s["kv_heads"] // world, s["hidden"] // s["heads"]
        H, Fl = s["hidden"], s["ffn"] // world
        mk = lambda o, i: nn.Parameter(torch.randn(o, i, dtype=dtype, device=device) * 0.02)  # noqa: E731
        self.qkv, self.o = mk((self.hq + 2 * self.hkv) * self.d, H), mk(H, self.hq * self.d)
        self.gate_up, self.down = mk(2 * Fl, H), mk(H, Fl)
        self.n1 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.n2 = nn.Parameter(torch.ones(H, dtype=dtype, device=device))

    def forward(self, x, cos, sin, group, cache=None, pos=0):
        B, S, H = x.shape
        h = _CopyToRanks.apply(F.rms_norm(x, (H,), self.n1, 1e-5), group)
        qkv = F.linear(h, self.qkv).view(B, S, self.hq + 2 * self.hkv, self.d)
        q, k, v = qkv.split([self.hq, self.hkv, self.hkv], 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        q, k, v = (t.transpose(1, 2) for t in (q, k, v))
        if cache is not None:                         # static cache [B, hkv, S_max, d]
            ck, cv = cache
            ck[:, :, pos:pos + S], cv[:, :, pos:pos + S] = k, v
            k, v = ck[:, :, :pos + S], cv[:, :, :pos + S]
        a = F.scaled_dot_product_attention(q, k, v, is_causal=S > 1, enable_gqa=True)
        x = x + _ReduceFromRanks.apply(F.linear(a.transpose(1, 2).reshape(B, S, -1), self.o), group)
        h = _CopyToRanks.apply(F.rms_norm(x, (H,), self.n2, 1e-5), group)
        g, u = F.linear(h, self.gate_up).chunk(2, -1)
        return x + _ReduceFromRanks.apply(F.linear(F.silu(g) * u, self.down), group)


class TPLlama(nn.Module):
    def __init__(self, s, world, rank, dtype, device, max_pos):
        super().__init__()
        self.s, self.world, self.rank = s, world, rank
        H, self.vloc = s["hidden"], (s["vocab"] + world - 1) // world
        self.embed = nn.Parameter(torch.randn(s["vocab"], H, dtype=dtype, device=device) * 0.02)      # replicated
        self.blocks = nn.ModuleList(Block(s, world, dtype, device) for _ in range(s["layers"]))
        self.norm = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.randn(self.vloc, H, dtype=dtype, device=device) * 0.02)     # vocabulary shard
        d = H // s["heads"]
        inv = 1.0 / (s["theta"] ** (torch.arange(0, d, 2, device=device).float() / d))
        ang = torch.arange(max_pos, device=device).float()[:, None] * inv[None]
        self.register_buffer("cos", ang.cos().to(dtype), persistent=False)
        self.register_buffer("sin", ang.sin().to(dtype), persistent=False)

    def hidden(self, ids, group, caches=None, pos=0):
        S = ids.shape[1]
        cos, sin = self.cos[pos:pos + S][None, :, None], self.sin[pos:pos + S][None, :, None]
        x = F.embedding(ids, self.embed)
        for i, b in enumerate(self.blocks):
            x = b(x, cos, sin, group, None if caches is None else caches[i], pos)
        return F.rms_norm(x, (x.shape[-1],), self.norm, 1e-5)

    def loss(self, ids, labels, group):
        """Vocabulary-parallel cross-entropy: max, sum of exponentials and the target logit are
        combined over the ranks with three small all-reduces."""
        h = _CopyToRanks.apply(self.hidden(ids, group), group)
        z = F.linear(h, self.lm_head).float().view(-1, self.vloc)
        if self.vloc * (self.rank + 1) > self.s["vocab"]:
            z[:, self.s["vocab"] - self.vloc * self.rank:] = float("-inf")
        t = labels.reshape(-1)
        m = z.detach().max(-1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        se = _ReduceFromRanks.apply(torch.exp(z - m[:, None]).sum(-1), group)
        lo = self.vloc * self.rank
        mine = (t >= lo) & (t < lo + self.vloc)
        tz = torch.where(mine, z.gather(1, (t - lo).clamp(0, self.vloc - 1)[:, None])[:, 0], torch.zeros_like(m))
        tz = _ReduceFromRanks.apply(tz, group)
        return (torch.log(se) + m - tz).mean()

    @torch.no_grad()
    def next_token(self, h_last, group):
        z = F.linear(h_last, self.lm_head).float()
        if self.vloc * (self.rank + 1) > self.s["vocab"]:
            z[:, self.s["vocab"] - self.vloc * self.rank:] = float("-inf")
        val, idx = z.max(-1)
        pair = torch.stack([val, (idx + self.vloc * self.rank).float()], -1)
        allp = [torch.empty_like(pair) for _ in range(self.world)]
        dist.all_gather(allp, pair, group=group)
        allp = torch.stack(allp)
        return allp[..., 1].gather(0, allp[..., 0].argmax(0)[None])[0].long()


def _timed(fn, device, world):
    cuda = device.type == "cuda"
    dist.barrier()
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    else:
        import time

        t0 = time.perf_counter()
        out = fn()
        ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t), out


def run_train(a, s, model, group, device, world):
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=device.type == "cuda")
    g = torch.Generator().manual_seed(0)                                   # the same batch on every rank
    data = torch.randint(0, s["vocab"], (a.global_batch, a.seq_len + 1), generator=g).to(device)
    n_micro = a.global_batch // a.micro_batch_seqs

    def step():
        opt.zero_grad(set_to_none=True)
        total = 0.0
        for i in range(n_micro):
            mb = data[i * a.micro_batch_seqs:(i + 1) * a.micro_batch_seqs]
            loss = model.loss(mb[:, :-1], mb[:, 1:], group) / n_micro
            loss.backward()
            total += float(loss.detach())
        # replicated parameters (embedding, norms) see the same gradient on every rank already
        opt.step()
        return total

    for _ in range(a.warmup):
        step()
    ms, last = _timed(lambda: [step() for _ in range(a.steps)][-1], device, world)
    return {"metric": "llama_tp_train_tokens_per_s", "impl": "torch", "value": a.global_batch * a.seq_len * a.steps / (ms / 1e3),
            "ms_per_step": ms / a.steps, "loss": last, "micro_batch_seqs": a.micro_batch_seqs,
            "how": "Megatron-style TP (no sequence parallelism), NCCL all-reduce after every row-parallel layer, eager"}


def run_decode(a, s, model, group, device, world):
    B, P, N = a.batch, a.prompt, a.new
    ids = torch.randint(0, s["vocab"], (B, P), generator=torch.Generator().manual_seed(0)).to(device)
    d, hkv = s["hidden"] // s["heads"], s["kv_heads"] // world
    dtype = model.embed.dtype
    caches = [(torch.zeros(B, hkv, P + N, d, dtype=dtype, device=device), torch.zeros(B, hkv, P + N, d, dtype=dtype, device=device))
              for _ in range(s["layers"])]

    @torch.no_grad()
    def prefill():
        tok = None
        for b0 in range(0, B, a.prefill_seqs):                                  # bounded activation memory
            sub = [(k[b0:b0 + a.prefill_seqs], v[b0:b0 + a.prefill_seqs]) for k, v in caches]
            h = model.hidden(ids[b0:b0 + a.prefill_seqs], group, sub, 0)[:, -1]
            t = model.next_token(h, group)
            tok = t if tok is None else torch.cat([tok, t])
        return tok

    @torch.no_grad()
    def decode(tok):
        for i in range(N):
            tok = model.next_token(model.hidden(tok[:, None], group, caches, P + i)[:, -1], group)
        return tok

    tok = prefill()
    decode(tok) if a.warmup else None
    ms_p, tok = _timed(prefill, device, world)
    ms_d, _ = _timed(lambda: decode(tok), device, world)
    return {"metric": "llama_tp_decode_tokens_per_s", "impl": "torch", "batch": B, "prompt": P, "new_tokens": N,
            "prefill_ms": ms_p, "prefill_tokens_per_s": B * P / (ms_p / 1e3), "decode_ms_per_step": ms_d / N,
            "decode_tokens_per_s": B * N / (ms_d / 1e3), "how": "static KV cache, SDPA, NCCL all-reduce per row-parallel layer, eager"}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="train", choices=["train", "decode"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(SHAPES))
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--global-batch", type=int, default=32)
    ap.add_argument("--micro-batch-seqs", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--prefill-seqs", type=int, default=8)
    a = ap.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    if a.device == "cuda":
        torch.cuda.set_device(local)
        device, dtype = torch.device("cuda", local), torch.bfloat16
        dist.init_process_group("nccl", device_id=device, rank=rank, world_size=world)
    else:
        device, dtype = torch.device("cpu"), torch.float32
        dist.init_process_group("gloo", rank=rank, world_size=world)
    s = dict(SHAPES[a.model])
    if a.layers:
        s["layers"] = a.layers
    assert s["heads"] % world == 0 and s["kv_heads"] % world == 0 and s["ffn"] % world == 0, "heads / ffn must divide by the world size"
    torch.manual_seed(1234 + rank)
    model = TPLlama(s, world, rank, dtype, device, max(a.seq_len, a.prompt + a.new) + 8)
    # replicated parameters start equal on every rank
    for p in [model.embed, model.norm] + [q for b in model.blocks for q in (b.n1, b.n2)]:
        dist.broadcast(p.data, 0)
    group = dist.group.WORLD
    out = (run_train if a.mode == "train" else run_decode)(a, s, model, group, device, world)
    out.update({"model": a.model, "layers": s["layers"], "tp": world, "dtype": str(dtype), "data": "synthetic"})
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
    sys.exit(0)
