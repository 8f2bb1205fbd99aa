#!/usr/bin/env python
"""ResNet-50 data-parallel training throughput (the ResNet-50 config of the benchmark spec): bf16 weights and
activations with fp32 master weights, SGD momentum 0.9, wd 1e-4, lr 0.1, batch 256 per GPU,
synthetic N(0,1) images 224x224x3, uniform labels.  Gradient exchange: 25 MB buckets, each one
fused reduce + SGD update launch (``ft_ddp_reduce_update``) overlapped with backward.

    python benchmarks/bench_resnet.py --steps 10
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_resnet.py
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--impl", default="ours", choices=["ours", "torch"])
    a = ap.parse_args()
    import torch
    import torch.distributed as dist

    from ferrotorch_b200 import _native
    from ferrotorch_b200.models.resnet import resnet50
    from ferrotorch_b200.train.engine import FlatTrainer

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(rank)
    torch.backends.cudnn.benchmark = True
    model = resnet50().to(dev).to(memory_format=torch.channels_last)
    x = torch.randn(a.batch, 3, 224, 224, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (a.batch,), device=dev)
    loss_fn = lambda m, xb, yb: torch.nn.functional.cross_entropy(m(xb).float(), yb)  # noqa: E731
    if a.impl == "torch":
        ddp_model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local]) if world > 1 else model
        opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4, fused=True)

        def step():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(ddp_model(x).float(), y)
            loss.backward()
            opt.step()
            return loss
    else:
        model = model.to(torch.bfloat16)
        ddp = None
        if world > 1:
            from ferrotorch_b200.parallel.ddp import FusedDDP

            ddp = FusedDDP(dist.group.WORLD, mode=a.comm, bucket_mb=25.0)
        tr = FlatTrainer(model, optimizer="sgd", lr=0.1, momentum=0.9, weight_decay=1e-4, loss_fn=loss_fn, ddp=ddp,
                         allocator=ddp.allocator if ddp else None, no_decay=lambda n, p: False)
        if ddp is not None:
            ddp.broadcast_parameters(tr)
        step = lambda: tr.step(x, y)  # noqa: E731

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    sync()
    l0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    if rank == 0:
        print(json.dumps({"metric": "resnet50_train_images_per_s", "impl": a.impl, "value": a.batch * world * a.steps / (ms / 1e3),
                          "n_gpus": world, "ms_per_step": ms / a.steps, "batch_per_gpu": a.batch, "comm": a.comm,
                          "gpu_launches": _native.launch_count() - l0, "loss": float(loss), "dtype": "bf16",
                          "data": "synthetic"}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
