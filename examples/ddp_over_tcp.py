#!/usr/bin/env python
"""Data-parallel training of a tiny Llama on CPU ranks over the C++ TCP transport (no GPU):
every rank ends every step with bitwise identical gradients and losses.

    python examples/ddp_over_tcp.py            # spawns 2 ranks on 127.0.0.1
"""
import multiprocessing as mp
import os
import socket
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def worker(rank, world, port, q, steps):
    import torch

    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.parallel import DDP, TcpGroup

    group = TcpGroup(rank, world, "127.0.0.1", port, timeout=30.0)
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny()
    # 4 MB buckets leave on a worker thread while backward is still running
    model = DDP(LlamaForCausalLM(cfg), group, bucket_size_bytes=4 << 20, overlap=True)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        t = torch.randint(0, cfg.vocab_size, (4, 33), generator=g)
        loss = model(t[:, :-1], labels=t[:, 1:])
        opt.zero_grad()
        loss.backward()
        model.sync_gradients()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        losses.append(float(group.all_reduce(loss.detach().reshape(1), "mean")))
    digest = float(sum(p.detach().double().sum() for p in model.parameters()))
    q.put((rank, losses, digest))
    group.barrier()


def main(steps: int = 5):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, 2, port, q, steps)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict((r, (l, d)) for r, l, d in (q.get(timeout=120) for _ in procs))
    for p in procs:
        p.join(30)
    assert res[0] == res[1], "ranks diverged"
    print("mean losses per step:", ["%.4f" % x for x in res[0][0]])
    print("replicas identical (parameter digest %.6f)" % res[0][1])
    return res


if __name__ == "__main__":
    main()
