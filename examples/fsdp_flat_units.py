#!/usr/bin/env python
"""Fully sharded data parallelism with one flat buffer per unit, on four in-process ranks (no GPU):
every decoder layer of a tiny Llama is one unit; a step costs two all-gathers and one reduce-scatter per
unit, each rank keeps a quarter of the weights, and the ranks end with the weights one process would have.

    python examples/fsdp_flat_units.py
"""
import os
import sys
import threading

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrotorch_b200.models.llama import LlamaConfig, LlamaDecoderLayer, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.parallel import auto_wrap  # noqa: E402
from ferrotorch_b200.parallel.backend import SimulatedGroup  # noqa: E402


def main(world: int = 4, steps: int = 3):
    cfg = LlamaConfig.tiny()
    torch.manual_seed(0)
    protos = [LlamaForCausalLM(cfg) for _ in range(world)]
    for m in protos[1:]:
        m.load_state_dict(protos[0].state_dict())
    tokens = torch.randint(0, cfg.vocab_size, (world * 2, 17), generator=torch.Generator().manual_seed(1))
    groups = SimulatedGroup.create_group(world)
    out = {}

    def rank(r):
        model = auto_wrap(protos[r], groups[r], (LlamaDecoderLayer,))
        shards = model.sharded_parameters()
        opt = torch.optim.AdamW(shards, lr=1e-3)
        mine = tokens.chunk(world)[r]
        losses = []
        for _ in range(steps):
            opt.zero_grad()
            loss = model(mine[:, :-1], labels=mine[:, 1:])
            loss.backward()
            model.sync_gradients()
            opt.step()
            losses.append(float(groups[r].all_reduce(loss.detach().reshape(1).clone(), "mean")))
        out[r] = (losses, sum(p.numel() for p in shards), [dict(u.stats) for u in model.units])

    ts = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(300) for t in ts]
    total = sum(p.numel() for p in LlamaForCausalLM(cfg).parameters())
    losses, held, stats = out[0]
    print("mean loss per step:", ["%.4f" % v for v in losses])
    print("parameters: %d in the model, %d held by rank 0 (%.0f %%)" % (total, held, 100.0 * held / total))
    print("per unit and step: %d all-gathers, %d reduce-scatter" % (stats[0]["all_gathers"] // steps, stats[0]["reduce_scatters"] // steps))
    assert all(out[r][0] == losses for r in out) and losses[-1] < losses[0]
    return out


if __name__ == "__main__":
    main()
