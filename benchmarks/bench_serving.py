#!/usr/bin/env python
"""Throughput of the continuous-batching server against serving the same requests one after another.

    python benchmarks/bench_serving.py --device cpu --requests 32

Both arms run the same model on the same synthetic requests (random prompts of 16 .. ``--max-prompt`` tokens,
8 .. ``--max-new`` new tokens, greedy) and produce the same tokens (checked).  ``sequential`` is
``models.generation.generate`` per request (the reference's serving model: one sequence, one cache);
``batched`` is ``models.serving.ContinuousBatcher``.  Prints one JSON line with generated tokens per second of
both, the mean tokens per step and the share of prompt tokens taken from the prefix table when
``--shared-prefix`` tokens are common to all prompts.  Wall clock around the whole arm (on CUDA after a
synchronise on both sides); the first request of each arm is run once before the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200.models.generation import GenerationConfig, generate  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.models.serving import ContinuousBatcher, Request  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--requests", type=int, default=32)
    ap.add_argument("--max-prompt", type=int, default=96)
    ap.add_argument("--max-new", type=int, default=48)
    ap.add_argument("--shared-prefix", type=int, default=0)
    ap.add_argument("--max-running", type=int, default=16)
    ap.add_argument("--lookahead", type=int, default=0, help="look-up speculation of the batched arm (same tokens, fewer steps)")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--vocab", type=int, default=4096)
    args = ap.parse_args(argv)
    dev = torch.device(args.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=args.vocab, hidden_size=args.hidden, intermediate_size=4 * args.hidden, num_hidden_layers=args.layers,
                      num_attention_heads=args.hidden // 64, num_key_value_heads=max(1, args.hidden // 128), head_dim=64,
                      max_position_embeddings=args.shared_prefix + args.max_prompt + args.max_new)
    model = LlamaForCausalLM(cfg).to(device=dev, dtype=dtype).eval()
    g = torch.Generator().manual_seed(1)
    shared = torch.randint(0, args.vocab, (args.shared_prefix,), generator=g).tolist()
    prompts = [shared + torch.randint(0, args.vocab, (int(torch.randint(16, args.max_prompt + 1, (1,), generator=g)),), generator=g).tolist()
               for _ in range(args.requests)]
    new = [int(torch.randint(8, args.max_new + 1, (1,), generator=g)) for _ in prompts]

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize()

    def sequential():
        return [generate(model, torch.tensor([p], device=dev), GenerationConfig.greedy(n))[0, len(p):].tolist() for p, n in zip(prompts, new)]

    def batched():
        pages = sum((len(p) + n + 15) // 16 for p, n in zip(prompts, new))
        b = ContinuousBatcher(model, num_blocks=pages, block_size=16, max_running=args.max_running, max_seq_len=cfg.max_position_embeddings,
                              prefix_caching=args.shared_prefix > 0)
        reqs = [b.submit(Request(p, n, lookahead=args.lookahead)) for p, n in zip(prompts, new)]
        b.run()
        return [r.output for r in reqs], b.stats

    generate(model, torch.tensor([prompts[0]], device=dev), GenerationConfig.greedy(2))
    sync()
    t0 = time.perf_counter()
    seq_out = sequential()
    sync()
    t_seq = time.perf_counter() - t0
    t0 = time.perf_counter()
    bat_out, stats = batched()
    sync()
    t_bat = time.perf_counter() - t0
    same = sum(a == b for a, b in zip(seq_out, bat_out))
    total = sum(new)
    print(json.dumps({"device": str(dev), "dtype": str(dtype).replace("torch.", ""), "requests": args.requests, "generated_tokens": total,
                      "prompt_tokens": sum(map(len, prompts)), "sequential_tok_s": round(total / t_seq, 1), "batched_tok_s": round(total / t_bat, 1),
                      "speedup": round(t_seq / t_bat, 2), "steps": stats.steps, "mean_tokens_per_step": round(stats.mean_batch_tokens(), 1),
                      "prefix_hit_tokens": stats.prefix_hit_tokens, "preemptions": stats.preemptions,
                      "speculated": "%d of %d accepted" % (stats.spec_accepted, stats.spec_proposed),
                      "requests_with_identical_tokens": "%d / %d" % (same, args.requests)}))
    return same


if __name__ == "__main__":
    main()
