#!/usr/bin/env python
"""Continuous batching: sixteen requests of different lengths served through a paged KV cache that is too
small to hold them all at once.  Every request still gets exactly the tokens it would get alone.

    python examples/serve_many_requests.py [--device cuda]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrotorch_b200.models import ContinuousBatcher, LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.models.generation import GenerationConfig, generate  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--requests", type=int, default=16)
    args = ap.parse_args()
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny()
    dtype = torch.bfloat16 if args.device != "cpu" else torch.float32
    model = LlamaForCausalLM(cfg).to(device=args.device, dtype=dtype).eval()
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (int(torch.randint(4, 60, (1,), generator=g)),), generator=g).tolist()
               for _ in range(args.requests)]
    new = [int(torch.randint(4, 24, (1,), generator=g)) for _ in prompts]

    server = ContinuousBatcher(model, num_blocks=24, block_size=16, max_running=8, max_seq_len=128, prefill_chunk=32)
    requests = [server.submit(p, n) for p, n in zip(prompts, new)]
    stats = server.run()

    print("%d requests, %d prompt + %d generated tokens in %d steps (%.1f tokens per step, at most %d sequences, %d of 24 pages)"
          % (len(requests), sum(map(len, prompts)), sum(len(r.output) for r in requests), stats.steps, stats.mean_batch_tokens(),
             stats.peak_running, stats.peak_pages))
    print("preemptions: %d; steps to the first token: %s" % (stats.preemptions, [r.first_token_step - r.submit_step for r in requests]))
    if args.device == "cpu":
        for r, p, n in zip(requests[:4], prompts, new):
            alone = generate(model, torch.tensor([p]), GenerationConfig.greedy(n))[0, len(p):].tolist()
            assert alone == r.output
        print("the first four requests match a run alone")


if __name__ == "__main__":
    main()
