#!/usr/bin/env python
"""Two ways to split one model over ranks, run here on in-process simulated ranks (threads):

* pipeline parallelism: three stages of an MLP trained with the 1F1B schedule; activations and
  gradients leave through non-blocking sends, the next micro-batch's receive is posted before
  the current one is computed; the loss and every gradient equal the unsplit model's;
* context parallelism: ring attention and Ulysses attention over a sequence split across four
  ranks, forward and backward, against attention over the whole sequence.

The same code runs over TCP processes (``TcpGroup``) or NCCL (``TorchGroup``) by passing another group.

    python examples/pipeline_and_context_parallel.py
"""
import copy
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200.ops import reference as R  # noqa: E402
from ferrotorch_b200.parallel import Pipeline  # noqa: E402
from ferrotorch_b200.parallel import context_parallel as CP  # noqa: E402
from ferrotorch_b200.parallel.backend import run_simulated  # noqa: E402


def pipeline_demo():
    torch.manual_seed(0)
    stages = [nn.Sequential(nn.Linear(16, 32), nn.Tanh()), nn.Sequential(nn.Linear(32, 32), nn.Tanh()), nn.Linear(32, 4)]
    x, y = torch.randn(16, 16), torch.randn(16, 4)
    whole = copy.deepcopy(nn.Sequential(*stages))
    want = nn.functional.mse_loss(whole(x), y)
    want.backward()

    def rank_body(g):
        stage = copy.deepcopy(stages[g.rank])
        pipe = Pipeline(stage, g, n_micro=4, schedule="1f1b", loss_fn=nn.functional.mse_loss)
        loss = pipe.train_step(x if g.rank == 0 else None, y if g.rank == 2 else None)
        return loss, [p.grad for p in stage.parameters()], pipe.stats

    res = run_simulated(3, rank_body)
    worst = max(float((g - w.grad).abs().max()) for s in range(3) for g, w in zip(res[s][1], whole[s].parameters()))
    print("pipeline 1F1B: loss %.6f (unsplit %.6f), largest gradient difference %.1e, stage 1 posted %d sends and prefetched %d receives"
          % (float(res[2][0]), float(want.detach()), worst, res[1][2]["posted_sends"], res[1][2]["prefetched_recvs"]))
    assert abs(float(res[2][0]) - float(want.detach())) < 1e-6 and worst < 1e-6


def context_demo():
    torch.manual_seed(1)
    W, B, S_loc, Hq, Hkv, D = 4, 1, 8, 8, 4, 16
    q, k, v = (torch.randn(B, W * S_loc, h, D, requires_grad=True) for h in (Hq, Hkv, Hkv))
    go = torch.randn(B, W * S_loc, Hq, D)
    full = R.attention(q, k, v, causal=True)[0]
    full.backward(go)

    def rank_body(g):
        sl = slice(g.rank * S_loc, (g.rank + 1) * S_loc)
        out = {}
        for name, fn in (("ring", CP.ring_attention), ("ulysses", CP.ulysses_attention)):
            ql, kl, vl = (t[:, sl].detach().clone().requires_grad_() for t in (q, k, v))
            o = fn(ql, kl, vl, g, True)
            o.backward(go[:, sl])
            out[name] = (float((o - full[:, sl]).abs().max()), float((ql.grad - q.grad[:, sl]).abs().max()),
                         float((kl.grad - k.grad[:, sl]).abs().max()))
        return out

    res = run_simulated(W, rank_body)
    for name in ("ring", "ulysses"):
        worst = [max(r[name][i] for r in res) for i in range(3)]
        print("%s attention over %d ranks: output / dq / dk differ from full attention by at most %.1e / %.1e / %.1e" % ((name, W) + tuple(worst)))
        assert max(worst) < 1e-4


if __name__ == "__main__":
    pipeline_demo()
    context_demo()
