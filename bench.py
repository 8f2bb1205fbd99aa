#!/usr/bin/env python
"""Flagship benchmark: Llama-3-8B training throughput (tokens/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Config (the Llama-3-8B training config of the benchmark spec): Llama-3-8B architecture (32 layers, d 4096, 32 q / 8 kv heads
of 128, FFN 14336, vocab 128256, RoPE theta 5e5), bf16 weights and activations, fp32 AdamW
state (master weights + two moments), lr 3e-4, wd 0.1, next-token cross-entropy on synthetic
token ids uniform in [0, 128256), sequence 4096, 4 sequences per GPU (32 per step at 8 GPUs;
weak scaling).  Random-init weights ~N(0, 0.02).  Data parallel across GPUs with the bucketed
gradient all-reduce fused with the AdamW update (``ferrotorch_b200.parallel.ddp``).

Timing: W warm-up steps, then exactly K steps between a barrier + ``torch.cuda.synchronize()``
on both sides, CUDA events on the compute stream, max over ranks.  The working set (128 GB of
weights and optimizer state per GPU) is three orders of magnitude larger than the 126 MB L2, so
no explicit flush is needed between steps.  A second timed pass measures the same steps end
to end through the public API: every step copies its token ids from pinned host memory and
reads the loss back to the host.  SM clocks and throttle reasons are sampled with nvidia-smi
during the timed passes.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"])
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "llama-1b", "tiny"])
    ap.add_argument("--layers", type=int, default=None, help="override the layer count (debug only; "
                    "the JSON line then reports the reduced model and is not a headline number)")
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--batch-per-gpu", type=int, default=4)
    ap.add_argument("--micro-batches", type=int, default=2)
    ap.add_argument("--checkpoint", action="store_true", help="recompute each decoder layer in backward")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--measure-exposed", action="store_true",
                    help="record how long the compute stream waits for the gradient exchange at the end of a step")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); power.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c, w in zip(sm, power) if w > 300] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def reference_unavailable() -> None:
    why = ("reference is a Rust workspace (28 crates, no Python package, no setup.py/pyproject.toml): "
           "a pip install of its source tree into baseline/_ref has nothing to build and no "
           "cargo/rustc toolchain or vendored crates exist offline")
    print(json.dumps({"impl": "reference", "unavailable": why}))


def build_model(args, device, dtype=None):
    import torch

    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM

    if args.model == "llama3-8b":
        cfg = LlamaConfig.llama3_8b()
    elif args.model == "llama-1b":
        cfg = LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=16, num_attention_heads=32,
                          num_key_value_heads=8, head_dim=64)
    else:
        cfg = LlamaConfig.tiny()
        cfg.head_dim = 64
    if args.layers is not None:
        cfg.num_hidden_layers = args.layers
    cfg.max_position_embeddings = max(args.seq_len, 2048)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype or torch.bfloat16)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.model.checkpoint_layers = args.checkpoint
    return cfg, model


def run_torch_baseline(args, cfg, model, device, world, rank, local_rank) -> None:
    """Same model, same data, same step, in plain PyTorch on the same box: fp32 parameters with
    bf16 autocast (cuBLAS GEMMs, SDPA attention, torch RMSNorm / cross-entropy),
    ``torch.optim.AdamW(fused=True)``, DistributedDataParallel over NCCL for N > 1."""
    import contextlib

    import torch
    import torch.distributed as dist

    from ferrotorch_b200.ops import functional as F

    F.set_native(False)
    model = model.float()
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    B, S, V, mb = args.batch_per_gpu, args.seq_len, cfg.vocab_size, args.micro_batches
    gen = torch.Generator().manual_seed(rank)
    host = [torch.randint(0, V, (B, S + 1), generator=gen).pin_memory() for _ in range(3)]
    dev = [t.to(device) for t in host]
    per = B // mb

    def step(t):
        opt.zero_grad(set_to_none=True)
        total = 0.0
        for i in range(mb):
            x, y = t[i * per:(i + 1) * per, :-1], t[i * per:(i + 1) * per, 1:]
            sync = contextlib.nullcontext() if (world == 1 or i == mb - 1) else net.no_sync()
            with sync:
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = net(x, labels=y, loss_denominator=B * S)
                loss.backward()
            total = total + loss.detach()
        opt.step()
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(dev[i % 3])
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step(dev[i % 3])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    if rank == 0:
        print(json.dumps({"metric": "llama3_8b_train_tokens_per_s", "impl": "torch", "value": B * S * world * args.steps / (ms / 1e3),
                          "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": ms / args.steps, "dtype": "bf16 autocast, fp32 params", "data": "synthetic",
                          "config": {"model": "Llama-3-8B" if args.layers is None else "layers=%d" % cfg.num_hidden_layers,
                                     "global_batch": B * world, "seq_len": S, "micro_batches": mb},
                          "clocks": clocks, "loss": float(loss), "gpu_launches": 0}))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    import torch.distributed as dist

    from ferrotorch_b200 import _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus %d must be launched with torchrun (one rank per GPU)" % args.gpus)
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    torch.manual_seed(1234 + rank)
    cfg, model = build_model(args, device, dtype=torch.float32 if args.impl == "torch" else torch.bfloat16)
    model.train()

    from ferrotorch_b200.train.engine import FlatTrainer

    if args.impl == "torch":
        run_torch_baseline(args, cfg, model, device, world, rank, local_rank)
        return

    ddp = None
    if world > 1:
        from ferrotorch_b200.parallel.ddp import FusedDDP

        ddp = FusedDDP(dist.group.WORLD, mode=args.comm)
        ddp.measure_exposed = args.measure_exposed
    alloc = ddp.allocator if ddp is not None else None
    trainer = FlatTrainer(model, optimizer="adamw", lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                          micro_batches=args.micro_batches, ddp=ddp, allocator=alloc)
    torch.cuda.empty_cache()
    if ddp is not None:
        ddp.broadcast_parameters(trainer)

    B, S, V = args.batch_per_gpu, args.seq_len, cfg.vocab_size
    gen = torch.Generator().manual_seed(rank)
    n_host = max(2, min(args.steps, 4))
    host_tokens = [torch.randint(0, V, (B, S + 1), generator=gen).pin_memory() for _ in range(n_host)]
    dev_tokens = [t.to(device, non_blocking=True) for t in host_tokens]

    def step_device(i):
        t = dev_tokens[i % n_host]
        return trainer.step(t[:, :-1], t[:, 1:])

    def step_e2e(i):
        t = host_tokens[i % n_host].to(device, non_blocking=True)
        loss = trainer.step(t[:, :-1], t[:, 1:])
        return float(loss)  # device -> host read of the step's result

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k):
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        l0 = _native.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(k):
            last = fn(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = _native.launch_count() - l0
        clocks = sampler.stop()
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms, launches, clocks, last

    for i in range(args.warmup):
        step_device(i)
    ms, launches, clocks, last = timed(step_device, args.steps)
    last_loss = float(last)
    tokens_per_step = B * S * world
    value = tokens_per_step * args.steps / (ms / 1e3)

    e2e = None
    if not args.no_e2e:
        step_e2e(0)
        ms2, _, clocks2, _ = timed(step_e2e, args.steps)
        e2e = {"value": tokens_per_step * args.steps / (ms2 / 1e3), "unit": "tokens/s",
               "ms_per_step": ms2 / args.steps, "h2d_bytes_per_step": B * (S + 1) * 8 * world,
               "d2h_bytes_per_step": 4 * world, "clocks": clocks2}

    status = _native.device_status(local_rank)
    if rank == 0:
        full = args.model == "llama3-8b" and args.layers is None
        out = {
            "metric": "llama3_8b_train_tokens_per_s" if full else "train_tokens_per_s_reduced_model",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": "Llama-3-8B" if full else "%s(layers=%d)" % (args.model, cfg.num_hidden_layers),
                       "global_batch": B * world, "seq_len": S, "parallelism": "dp%d" % world,
                       "micro_batches": args.micro_batches, "activation_checkpointing": bool(args.checkpoint),
                       "optimizer": "AdamW fp32 state (master, m, v), lr 3e-4, wd 0.1",
                       "comm": args.comm if world > 1 else "none",
                       "l2": "no flush: 128 GB of weights + optimizer state per step >> 126 MB L2"},
            "clocks": clocks, "gpu_launches": launches, "loss": last_loss, "device_status": status,
            "model_flops_per_token": 6 * cfg.num_parameters() + 6 * cfg.num_hidden_layers * cfg.hidden_size * S,
            "impl": "ours",
        }
        if e2e is not None:
            out["e2e"] = e2e
        if ddp is not None and args.measure_exposed:
            ex = ddp.exposed_ms()[-args.steps:]
            out["exposed_comm_ms_per_step"] = sum(ex) / max(1, len(ex))
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
