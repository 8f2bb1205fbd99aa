#!/usr/bin/env python
"""Llama training with tensor + sequence parallelism over the GPUs of one node (the TP=8 point
of the Llama-3-8B training config: seq 4096, global batch 32 sequences, AdamW lr 3e-4 wd 0.1).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/bench_train_tp.py --model llama3-8b --global-batch 32 --seq-len 4096

Every rank holds 1/TP of each projection and 1/TP of the token rows; the four projections of a
block run on the fused all-gather->GEMM / GEMM->reduce-scatter kernels in forward and backward.
Random-init weights, uniform-random token ids (synthetic), copied from pinned host memory each
step.  Timing: CUDA events around K full optimizer steps, max over ranks.  One JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "small"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--global-batch", type=int, default=32)
    ap.add_argument("--micro-batch-seqs", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--checkpoint", action="store_true", help="activation checkpointing per block")
    ap.add_argument("--max-grad-norm", type=float, default=0.0)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from ferrotorch_b200 import _native
    from ferrotorch_b200.models.llama import LlamaConfig
    from ferrotorch_b200.models.llama_tp import TPLlamaForCausalLM, make_tp_trainer
    from ferrotorch_b200.parallel.tensor_parallel import TPContext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    cfg = {"llama3-8b": LlamaConfig.llama3_8b,
           "small": lambda: LlamaConfig(vocab_size=32000, hidden_size=2048, intermediate_size=8192,
                                        num_hidden_layers=8, num_attention_heads=16, num_key_value_heads=8,
                                        head_dim=128)}[args.model]()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    cfg.max_position_embeddings = max(cfg.max_position_embeddings, args.seq_len)
    tp = TPContext(group, dev)
    torch.manual_seed(1234 + rank)
    model = TPLlamaForCausalLM(cfg, tp)
    model.checkpoint_layers = args.checkpoint
    assert args.global_batch % args.micro_batch_seqs == 0
    tr = make_tp_trainer(model, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                         max_grad_norm=args.max_grad_norm or None,
                         micro_batches=args.global_batch // args.micro_batch_seqs)
    B, S = args.global_batch, args.seq_len
    g = torch.Generator().manual_seed(0)          # the same data on every rank (one model replica)
    host = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory()

    def one_step():
        t = host.to(dev, non_blocking=True)
        return tr.step(t[:, :-1], t[:, 1:])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        loss = one_step()
    sync()
    tp.check_status()
    l0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = one_step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    tp.check_status()
    tokens = B * S * args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "llama_train_tokens_per_s", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "loss": float(loss),
            "gpu_launches": _native.launch_count() - l0,
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
            "config": {"model": args.model, "layers": cfg.num_hidden_layers, "global_batch": B, "seq_len": S,
                       "micro_batch_seqs": args.micro_batch_seqs, "checkpoint": bool(args.checkpoint),
                       "parallelism": "tp%d+sp" % world, "optimizer": "adamw lr 3e-4 wd 0.1"}}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
