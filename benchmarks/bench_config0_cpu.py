#!/usr/bin/env python
"""The CPU plumbing configuration of the benchmark spec: a tiny Llama (4 layers, d_model 256,
4 query / 2 KV heads of 64, SwiGLU 688, vocabulary 4096, fp32) trained for 20 AdamW steps
(lr 3e-4, betas 0.9 / 0.95, weight decay 0.1, gradient clip 1.0) on two CPU ranks, batch 8 x 128
uniform-random tokens per rank from seed 0.  Two arms, same model code and data:

* ``tcp``  -- this framework's host data parallelism over its native TCP transport
              (``parallel.host_ddp.DDP`` on a ``TcpGroup``: star all-reduce in rank order, 4 MB buckets
              reduced on a worker thread while backward still runs; ``tcp+sequential`` reduces after backward);
* ``gloo`` -- the same wrapper over ``torch.distributed`` / gloo (``TorchGroup``);
* ``torch_ddp`` -- ``torch.nn.parallel.DistributedDataParallel`` over gloo (the library arm).

Prints one JSON line per arm: seconds per step (max over ranks), whether the per-step losses and
the checksums of the averaged gradients agree bit for bit between the two ranks, first and last loss.

    python benchmarks/bench_config0_cpu.py [--steps 20]
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import socket
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def worker(rank: int, world: int, port: int, backend: str, steps: int, threads: int, q, overlap: bool = True, bucket_mb: int = 4) -> None:
    import torch

    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.parallel.host_ddp import DDP

    try:
        torch.set_num_threads(threads)
        backend, _, opt_ = backend.partition("+")
        overlap = overlap and opt_ != "sequential"
        if backend == "tcp":
            from ferrotorch_b200.parallel.backend import TcpGroup

            g = TcpGroup(rank, world, "127.0.0.1", port, timeout=120.0)
        else:
            import torch.distributed as dist

            from ferrotorch_b200.parallel.backend import TorchGroup

            dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
            g = TorchGroup()
        torch.manual_seed(1000 + rank)                      # different initial weights: the broadcast must fix it
        model = LlamaForCausalLM(LlamaConfig.tiny())
        if backend == "torch_ddp":
            wrapped = torch.nn.parallel.DistributedDataParallel(model)     # broadcasts rank 0's weights itself
            ddp = None
        else:
            wrapped = model
            ddp = DDP(model, g, bucket_size_bytes=bucket_mb << 20, overlap=overlap)
            ddp.broadcast_parameters(0)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
        gen = torch.Generator().manual_seed(0)
        losses, sums = [], []
        g.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            ids = torch.randint(0, 4096, (8, 129), generator=gen)
            loss = wrapped(ids[:, :-1], labels=ids[:, 1:])
            opt.zero_grad(set_to_none=True)
            loss.backward()
            if ddp is not None:
                ddp.sync_gradients()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            sums.append(torch.cat([p.grad.reshape(-1) for p in model.parameters()]).double().sum().item().hex())
            opt.step()
            losses.append(loss.item().hex())
        dt = (time.perf_counter() - t0) / steps
        q.put((rank, {"s_per_step": dt, "losses": losses, "grads": sums}))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR %r %s" % (e, traceback.format_exc())))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--threads", type=int, default=max(1, (os.cpu_count() or 2) // 2))
    ap.add_argument("--arms", default="tcp,tcp+sequential,gloo,torch_ddp")
    a = ap.parse_args()
    ctx = mp.get_context("spawn")
    for backend in a.arms.split(","):
        q, port = ctx.Queue(), _free_port()
        procs = [ctx.Process(target=worker, args=(r, 2, port, backend, a.steps, a.threads, q)) for r in range(2)]
        for p in procs:
            p.start()
        out = dict(q.get(timeout=1800) for _ in range(2))
        for p in procs:
            p.join(60)
        bad = [v for v in out.values() if isinstance(v, str)]
        if bad:
            print(json.dumps({"config": 0, "arm": backend, "error": bad[0][:400]}))
            continue
        r0, r1 = out[0], out[1]
        print(json.dumps({
            "config": 0, "arm": backend, "world": 2, "steps": a.steps, "threads_per_rank": a.threads,
            "s_per_step": max(r0["s_per_step"], r1["s_per_step"]),
            "losses_bitwise_equal": r0["losses"] == r1["losses"], "reduced_grads_bitwise_equal": r0["grads"] == r1["grads"],
            "first_loss": float.fromhex(r0["losses"][0]), "last_loss": float.fromhex(r0["losses"][-1])}))


if __name__ == "__main__":
    main()
