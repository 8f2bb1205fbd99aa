#!/usr/bin/env python
"""Train a tiny Llama for a few steps with the flat-arena trainer (CPU or one GPU).

    python examples/train_tiny_llama.py [--steps 20] [--device cuda]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrotorch_b200.data import DataLoader, SyntheticTokens  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.train.engine import FlatTrainer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()
    cfg = LlamaConfig.tiny()
    model = LlamaForCausalLM(cfg).to(a.device)
    if a.device == "cuda":
        model = model.to(torch.bfloat16)
    trainer = FlatTrainer(model, optimizer="adamw", lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    loader = DataLoader(SyntheticTokens(cfg.vocab_size, 64, length=8), batch_size=8)
    x, y = next(iter(loader))                       # one fixed batch: the loss must go down
    x, y = x.to(a.device), y.to(a.device)
    first = last = None
    for step in range(a.steps):
        last = float(trainer.step(x, y))
        first = last if first is None else first
        if step % 5 == 0:
            print("step %3d  loss %.4f" % (step, last))
    print("loss %.4f -> %.4f" % (first, last))
    assert last < first
    return first, last


if __name__ == "__main__":
    main()
