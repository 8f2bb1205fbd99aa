#!/usr/bin/env python
"""Roofline of the fused tensor-parallel kernels on the projection shapes of a Llama block.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/bench_tp_kernels.py --rows 16384

For every shape: CUDA-event time of the fused kernel (mean of ``--iters`` back-to-back launches
after warm-up, max over ranks), its TFLOP/s, the bytes that had to cross NVLink per GPU and
direction, the roofline time = max(FLOPs / measured GEMM peak, NVLink bytes / 770 GB/s) and the
achieved fraction of it.  The GEMM peak is ``--peak-tflops`` (default 1414.9: a B200's measured
sustained cuBLAS bf16 throughput under its power cap).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16384, help="token rows M (batch*seq) of the block")
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--qkv", type=int, default=6144)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=1414.9,
                    help="measured sustained cuBLAS bf16 GEMM throughput, TFLOP/s")
    ap.add_argument("--n-copy", type=int, default=0, help="copy CTAs of the all-gather GEMM (0 = default)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from ferrotorch_b200.parallel.tensor_parallel import TPContext

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    tp = TPContext(group, dev, **({"n_copy": args.n_copy} if args.n_copy else {}))
    peak = args.peak_tflops
    link = 770.0  # GB/s per direction per GPU, measured peer copy
    M, H = args.rows, args.hidden
    ms_rows = tp.rows_per_rank(M)
    lo = rank * ms_rows

    def rnd(*s):
        return (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)

    def timed(fn):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    rows = []
    x_rows = rnd(ms_rows, H)

    def ag_case(name, slot, K, N, kn):
        w = rnd(K, N) if kn else rnd(N, K)

        def run():
            tp.wait_gather_buffer_free(slot)
            tp.my_rows(slot, M, K).copy_(x_rows)
            tp.ag_gemm(slot, M, w, w_is_kn=kn)

        ms = timed(run)
        flops = 2.0 * M * N * K
        nbytes = (world - 1) / world * M * K * 2
        rows.append((name, M, N, K, ms, flops, nbytes))

    def rs_case(name, slot, K, N, kn):
        x = rnd(M, K)
        w = rnd(K, N) if kn else rnd(N, K)
        ms = timed(lambda: tp.gemm_rs(slot, x, w, w_is_kn=kn))
        flops = 2.0 * M * N * K
        nbytes = (world - 1) / world * M * N * 2
        rows.append((name, M, N, K, ms, flops, nbytes))

    W = world
    ag_case("qkv      AG->GEMM", 0, H, args.qkv // W, False)
    rs_case("o_proj   GEMM->RS", 1, args.qkv * 2 // 3 // W, H, False)
    ag_case("gate_up  AG->GEMM", 2, H, 2 * args.ffn // W, False)
    rs_case("down     GEMM->RS", 3, args.ffn // W, H, False)
    rs_case("qkv dX   GEMM->RS", 5, args.qkv // W, H, True)
    ag_case("o dX     AG->GEMM", 7, H, args.qkv * 2 // 3 // W, True)
    rs_case("gate_up dX GEMM->RS", 8, 2 * args.ffn // W, H, True)
    ag_case("down dX  AG->GEMM", 10, H, args.ffn // W, True)
    tp.check_status()
    if rank == 0:
        out = []
        print("world %d, rows %d, GEMM peak %.0f TFLOP/s (measured), link %.0f GB/s" % (world, M, peak, link))
        print("%-22s %6s %6s %6s %9s %9s %10s %10s %8s" % ("kernel", "M", "N", "K", "ms", "TFLOP/s", "NVL GB/s", "roof ms", "frac"))
        for name, m, n, k, ms, flops, nbytes in rows:
            roof = max(flops / (peak * 1e12), nbytes / (link * 1e9)) * 1e3
            print("%-22s %6d %6d %6d %9.3f %9.1f %10.1f %10.3f %8.2f" %
                  (name, m, n, k, ms, flops / ms / 1e9, nbytes / ms / 1e6, roof, roof / ms))
            out.append({"kernel": name.strip(), "M": m, "N": n, "K": k, "ms": ms, "tflops": flops / ms / 1e9,
                        "nvlink_gbs": nbytes / ms / 1e6, "roofline_ms": roof, "fraction": roof / ms})
        print(json.dumps({"world": world, "rows": M, "kernels": out}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
