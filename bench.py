#!/usr/bin/env python
"""Flagship benchmark: Llama-3-8B training throughput (tokens/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Config: Llama-3-8B architecture (32 layers, d 4096, 32 q / 8 kv heads of 128, FFN 14336, vocab
128256, RoPE theta 5e5), bf16 weights and activations, fp32 AdamW state (master weights + two
moments), lr 3e-4, wd 0.1, next-token cross-entropy on synthetic token ids uniform in
[0, 128256), sequence 4096, **global batch 32 sequences per optimizer step at every N** (strong
scaling: each GPU runs 32 / N sequences per step as micro-batches of ``--micro-batch-seqs``,
gradients accumulated in an fp32 arena).  Random-init weights ~N(0, 0.02).  Data parallel
across GPUs with the bucketed gradient all-reduce fused with the AdamW update
(``ferrotorch_b200.parallel.ddp``).  At 8 GPUs the line also carries the same global batch run
as one tensor + sequence-parallel replica (``tp_sp_point``).

Baseline: no reference number exists for this metric (the reference is a Rust workspace that
cannot be built here, and it publishes no Llama figure), so before the measured arm the script
runs the same model, batch and data shape in plain PyTorch on the same GPUs
(``--impl torch`` runs only that) and reports ``vs_baseline = value / torch value``.

Timing: W warm-up steps, then exactly K steps between a barrier + ``torch.cuda.synchronize()``
on both sides, CUDA events on the compute stream, max over ranks.  The working set (> 100 GB of
weights, gradients and optimizer state per GPU) is three orders of magnitude larger than the
126 MB L2, so no explicit flush is needed between steps.  A second timed pass measures the same
steps end to end through the public API: every step copies its token ids from pinned host
memory and reads the loss back to the host.  SM clocks and throttle reasons are sampled with
nvidia-smi during the timed passes.
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
    ap.add_argument("--global-batch", type=int, default=32, help="sequences per optimizer step over all GPUs")
    ap.add_argument("--micro-batch-seqs", type=int, default=2, help="sequences per forward/backward pass")
    ap.add_argument("--no-baseline", action="store_true", help="skip the same-box PyTorch arm (vs_baseline = null)")
    ap.add_argument("--baseline-steps", type=int, default=1, help="timed steps of the PyTorch arm (after 1 warm-up)")
    ap.add_argument("--e2e-steps", type=int, default=3, help="timed steps of the end-to-end pass (0 = --steps)")
    ap.add_argument("--no-tp-point", action="store_true", help="at 8 GPUs, skip the additional TP=8+SP measurement")
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
    if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also under torchrun
        print(json.dumps({"impl": "reference", "unavailable": why}))


def build_config(args):
    from ferrotorch_b200.models.llama import LlamaConfig

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
    return cfg


def build_model(args, device, dtype=None):
    import torch

    from ferrotorch_b200.models.llama import LlamaForCausalLM

    cfg = build_config(args)
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype or torch.bfloat16)
    try:
        with torch.device(device):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(prev)
    model.model.checkpoint_layers = args.checkpoint
    return cfg, model


def run_torch_arm(args, device, world, rank, local_rank, steps, warmup) -> dict | None:
    """Same model, same data, same global batch in plain PyTorch on the same box: bf16 parameters
    (no per-micro-batch weight casts), cuBLAS GEMMs, SDPA attention, torch RMSNorm / cross-entropy,
    ``torch.optim.AdamW(fused=True)`` (its state is then bf16: less optimizer traffic than the
    fp32 state of the measured arm), DistributedDataParallel over NCCL for N > 1 with
    ``no_sync`` on all but the last micro-batch.  Returns the result on every rank."""
    import contextlib

    import torch
    import torch.distributed as dist

    from ferrotorch_b200.ops import functional as F

    old = F.set_native(False)
    torch.manual_seed(1234 + rank)
    cfg, model = build_model(args, device, dtype=torch.bfloat16)
    model.train()
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank]) if world > 1 else model
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)
    B, S, V = args.global_batch // world, args.seq_len, cfg.vocab_size
    per = min(args.micro_batch_seqs, B)
    mb = B // per
    gen = torch.Generator().manual_seed(rank)
    host = [torch.randint(0, V, (B, S + 1), generator=gen).pin_memory() for _ in range(2)]
    dev = [t.to(device) for t in host]

    def step(t):
        opt.zero_grad(set_to_none=True)
        total = 0.0
        for i in range(mb):
            x, y = t[i * per:(i + 1) * per, :-1], t[i * per:(i + 1) * per, 1:]
            sync = contextlib.nullcontext() if (world == 1 or i == mb - 1) else net.no_sync()
            with sync:
                loss = net(x, labels=y, loss_denominator=B * S)
                loss.backward()
            total = total + loss.detach()
        opt.step()
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    loss = None
    for i in range(warmup):
        loss = step(dev[i % 2])
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = step(dev[i % 2])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t)
    out = {"metric": "llama3_8b_train_tokens_per_s", "impl": "torch",
           "value": B * S * world * steps / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": steps,
           "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong",
           "dtype": "bf16 parameters, torch.optim.AdamW(fused) with bf16 state", "data": "synthetic",
           "config": {"model": "Llama-3-8B" if (args.model == "llama3-8b" and args.layers is None)
                      else "%s(layers=%d)" % (args.model, cfg.num_hidden_layers),
                      "global_batch": B * world, "seq_len": S, "micro_batch_seqs": per,
                      "parallelism": "dp%d (torch DDP / NCCL)" % world,
                      "kernels": "cuBLAS, SDPA (flash), torch eager elementwise"},
           "clocks": clocks, "loss": float(loss), "gpu_launches": 0}
    del net, opt, model, dev, loss
    F.set_native(old)
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_tp_point(args, device, world, rank, local_rank, steps, warmup) -> dict:
    """The 8-GPU point as the benchmark spec words it: one model replica over all ranks with tensor +
    sequence parallelism (fused all-gather->GEMM / GEMM->reduce-scatter kernels), same global
    batch.  Returns its own result dictionary (tokens/s over the whole job)."""
    import torch
    import torch.distributed as dist

    from ferrotorch_b200 import _native
    from ferrotorch_b200.models.llama_tp import TPLlamaForCausalLM, make_tp_trainer
    from ferrotorch_b200.parallel.tensor_parallel import TPContext

    cfg = build_config(args)
    tp = TPContext(dist.group.WORLD, device)
    torch.manual_seed(1234 + rank)
    model = TPLlamaForCausalLM(cfg, tp)
    per = 4
    tr = make_tp_trainer(model, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                         micro_batches=max(1, args.global_batch // per))
    B, S = args.global_batch, args.seq_len
    g = torch.Generator().manual_seed(0)          # one replica: the same data on every rank
    host = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).pin_memory()

    def one_step():
        t = host.to(device, non_blocking=True)
        return tr.step(t[:, :-1], t[:, 1:])

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    loss = None
    for _ in range(warmup):
        loss = one_step()
    sync()
    tp.check_status()
    l0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = one_step()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t)
    tp.check_status()
    return {"value": B * S * steps / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / steps, "steps": steps,
            "warmup": warmup, "loss": float(loss), "gpu_launches": _native.launch_count() - l0,
            "config": {"global_batch": B, "seq_len": S, "micro_batch_seqs": per,
                       "parallelism": "tp%d+sp" % world},
            "timing": "end to end: token ids copied from pinned host memory every step"}


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
    if args.global_batch % world:
        raise SystemExit("--global-batch %d does not divide over %d GPUs" % (args.global_batch, world))

    if args.impl == "torch":
        out = run_torch_arm(args, device, world, rank, local_rank, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps(out))
        if world > 1:
            dist.destroy_process_group()
        return

    # Same-box baseline first (its memory is released before the measured arm is built).
    baseline = None
    if not args.no_baseline:
        try:
            baseline = run_torch_arm(args, device, world, rank, local_rank, args.baseline_steps, 1)
        except Exception as e:  # noqa: BLE001  (an out-of-memory baseline must not lose the measured arm)
            baseline = {"error": "%s: %s" % (type(e).__name__, str(e)[:200])}
            import gc

            gc.collect()
            torch.cuda.empty_cache()

    torch.cuda.reset_peak_memory_stats()
    torch.manual_seed(1234 + rank)
    cfg, model = build_model(args, device, dtype=torch.bfloat16)
    model.train()

    from ferrotorch_b200.train.engine import FlatTrainer

    ddp = None
    if world > 1:
        from ferrotorch_b200.parallel.ddp import FusedDDP

        ddp = FusedDDP(dist.group.WORLD, mode=args.comm)
        ddp.measure_exposed = args.measure_exposed
    alloc = ddp.allocator if ddp is not None else None
    B, S, V = args.global_batch // world, args.seq_len, cfg.vocab_size
    per = min(args.micro_batch_seqs, B)
    micro_batches = B // per
    trainer = FlatTrainer(model, optimizer="adamw", lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                          micro_batches=micro_batches, ddp=ddp, allocator=alloc)
    grad_dtype_name = str(trainer.arena.grads.dtype)
    torch.cuda.empty_cache()
    if ddp is not None:
        ddp.broadcast_parameters(trainer)

    gen = torch.Generator().manual_seed(rank)
    n_host = 2
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
    peak_gb = torch.cuda.max_memory_allocated() / 2 ** 30

    e2e = None
    if not args.no_e2e:
        k2 = args.steps if args.e2e_steps <= 0 else min(args.steps, args.e2e_steps)
        step_e2e(0)
        ms2, _, clocks2, _ = timed(step_e2e, k2)
        e2e = {"value": tokens_per_step * k2 / (ms2 / 1e3), "unit": "tokens/s", "steps": k2,
               "ms_per_step": ms2 / k2, "h2d_bytes_per_step": B * (S + 1) * 8 * world,
               "d2h_bytes_per_step": 4 * world, "clocks": clocks2}

    status = _native.device_status(local_rank)
    exposed = None
    if ddp is not None and args.measure_exposed:
        ex = ddp.exposed_ms()[-args.steps:]
        exposed = sum(ex) / max(1, len(ex))

    tp_point = None
    if world == 8 and not args.no_tp_point:
        # the 8-GPU point as the spec words it (TP=8 + SP), next to the data-parallel value
        try:
            del trainer, model, ddp, dev_tokens
            import gc

            gc.collect()
            torch.cuda.empty_cache()
            tp_point = run_tp_point(args, device, world, rank, local_rank, max(1, min(args.steps, 3)), 2)
        except Exception as e:  # noqa: BLE001
            tp_point = {"error": "%s: %s" % (type(e).__name__, str(e)[:200])}

    if rank == 0:
        full = args.model == "llama3-8b" and args.layers is None
        base_val = baseline.get("value") if isinstance(baseline, dict) else None
        # matmul parameters only: the embedding table is a gather, not a GEMM
        matmul_params = cfg.num_parameters() - cfg.vocab_size * cfg.hidden_size
        out = {
            "metric": "llama3_8b_train_tokens_per_s" if full else "train_tokens_per_s_reduced_model",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / base_val) if base_val else None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"model": "Llama-3-8B" if full else "%s(layers=%d)" % (args.model, cfg.num_hidden_layers),
                       "global_batch": B * world, "seq_len": S, "parallelism": "dp%d" % world,
                       "micro_batch_seqs": per, "micro_batches_per_step": micro_batches,
                       "activation_checkpointing": bool(args.checkpoint),
                       "gradient_accumulation_dtype": grad_dtype_name,
                       "optimizer": "AdamW fp32 state (master, m, v), lr 3e-4, wd 0.1",
                       "comm": args.comm if world > 1 else "none",
                       "l2": "no flush: > 100 GB of weights + optimizer state per step >> 126 MB L2"},
            "baseline": {"what": "vs_baseline = value / this: plain PyTorch on the same box, same model, batch and "
                                 "data shape (no published reference number exists for this metric)",
                         "result": baseline},
            "clocks": clocks, "gpu_launches": launches, "loss": last_loss, "device_status": status,
            "peak_mem_gb": peak_gb,
            "model_flops_per_token": 6 * matmul_params + 6 * cfg.num_hidden_layers * cfg.hidden_size * S,
            "impl": "ours",
        }
        if e2e is not None:
            out["e2e"] = e2e
        if exposed is not None:
            out["exposed_comm_ms_per_step"] = exposed
        if tp_point is not None:
            out["tp_sp_point"] = tp_point
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
