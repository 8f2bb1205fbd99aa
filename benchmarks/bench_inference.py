#!/usr/bin/env python
"""Llama inference benchmark (the two inference configs of the benchmark spec): prefill + greedy decode with the
paged KV cache, tensor parallel over the GPUs of one node.

    python benchmarks/bench_inference.py --model llama3-8b --batch 64 --prompt 2048 --new 256
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/bench_inference.py --model llama3-8b --batch 64 --prompt 2048 --new 256

Random-init weights ~N(0, 0.02), uniform-random prompt ids.  Timing: CUDA events, max over
ranks; prints one JSON line with prefill and decode tokens/s (whole job).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama3-70b", "small"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--warmup-steps", type=int, default=8)
    ap.add_argument("--graph", action="store_true", help="capture the decode step in a CUDA graph")
    ap.add_argument("--weights", default="bf16", choices=["bf16", "q4_0"],
                    help="q4_0: the same random weights quantised to GGUF Q4_0 planes (dequant-GEMM path)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from ferrotorch_b200 import _native
    from ferrotorch_b200.models.engine import LlamaEngine
    from ferrotorch_b200.models.llama import LlamaConfig
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
    cfg = {"llama3-8b": LlamaConfig.llama3_8b, "llama3-70b": LlamaConfig.llama3_70b,
           "small": lambda: LlamaConfig(vocab_size=32000, hidden_size=2048, intermediate_size=8192,
                                        num_hidden_layers=8, num_attention_heads=16, num_key_value_heads=8,
                                        head_dim=128)}[args.model]()
    if args.layers:
        cfg.num_hidden_layers = args.layers
    eng = LlamaEngine(cfg, TPContext(group, dev), max_batch=args.batch, max_seq_len=args.prompt + args.new + 32, cuda_graph=args.graph,
                      weight_format=args.weights)
    prompts = torch.randint(0, cfg.vocab_size, (args.batch, args.prompt), generator=torch.Generator().manual_seed(0))

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        sync()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, out

    eng.prefill(prompts[:, : min(args.prompt, 256)])      # warm-up (allocations, symmetric buffers)
    tok = eng.prefill(prompts)
    for _ in range(args.warmup_steps):
        tok = eng.decode_step(tok)
    ms_prefill, tok = timed(lambda: eng.prefill(prompts))
    l0 = _native.launch_count()

    def run_decode():
        t = tok
        for _ in range(args.new):
            t = eng.decode_step(t)
        return t

    ms_decode, _ = timed(run_decode)
    launches = _native.launch_count() - l0
    status = _native.device_status(local)
    if rank == 0:
        print(json.dumps({
            "metric": "llama_tp_decode_tokens_per_s", "model": args.model, "layers": cfg.num_hidden_layers,
            "tp": world, "batch": args.batch, "prompt": args.prompt, "new_tokens": args.new,
            "prefill_tokens_per_s": args.batch * args.prompt / (ms_prefill / 1e3), "prefill_ms": ms_prefill,
            "decode_tokens_per_s": args.batch * args.new / (ms_decode / 1e3),
            "decode_ms_per_step": ms_decode / args.new, "cuda_graph": bool(args.graph), "gpu_launches_decode": launches, "device_status": status,
            "dtype": "bf16", "weights": args.weights, "data": "synthetic"}))
    if world > 1:
        # release the captured decode graph (it holds NCCL work in the Q4_0 path) before the
        # communicator goes away; tearing the group down under a live graph can block at exit
        dist.barrier()
        torch.cuda.synchronize()
        del eng
        import gc

        gc.collect()
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
