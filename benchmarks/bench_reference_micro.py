#!/usr/bin/env python
"""The micro-benchmarks the reference publishes (its ``benchmarks/RESULTS.md``: creation,
elementwise, matmul, reductions, shape ops, broadcasting, MLP forward / backward / training step,
convolution, recurrent layers), run through this package's public API on ``--device cpu`` or
``cuda``, printed beside the reference's own published values (RTX 3090 / AMD CPU, other
hardware: context, not a same-box comparison).

    python benchmarks/bench_reference_micro.py --device cpu

Timing: median of ``--iters`` calls after ``--warmup`` (CUDA: events around each call after a
synchronise), microseconds.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ferrotorch_b200 as ft  # noqa: E402
from ferrotorch_b200.ops.random import DevicePhilox  # noqa: E402

# name -> (reference ferrotorch us, reference PyTorch us) as published; None where not published
PUBLISHED = {
    "cpu": {"zeros": (83, 35), "rand": (2689, 1865), "add": (907, 34), "mul": (929, 40), "relu": (125, 42), "sigmoid": (1037, 132),
            "exp": (997, 50), "log": (948, 1120), "sin": (968, 97), "cos": (984, 104), "tanh": (989, 200),
            "matmul_64": (16, 7), "matmul_256": (220, 68), "matmul_1024": (4979, 3024), "sum_all": (379, 21), "sum_dim0": (10118, 14),
            "mean_dim1": (10480, 11), "permute": (1747, 467), "chunk4": (341, 2), "cat4": (236, 70), "broadcast_add": (976, 12),
            "broadcast_mul": (2112, 49), "mlp32_fwd": (105, 53), "mlp32_bwd": (468, 355), "mlp32_train": (1525, 692),
            "mlp128_fwd": (957, 318), "mlp128_bwd": (3670, 1555), "mlp128_train": (6418, 1972), "conv2d_fwd": (1244, 102),
            "lstm_fwd": (9212, 2381)},
    "cuda": {"zeros": (334, 55), "rand": (15, 60), "add": (53, 42), "mul": (53, 42), "sub": (51, None), "div": (54, None), "relu": (54, 42),
             "sigmoid": (54, None), "tanh": (60, None), "exp": (47, None), "log": (47, None), "matmul_64": (99, 65), "matmul_256": (56, 33),
             "matmul_1024": (198, 319), "matmul_4096": (15225, 14880), "sum_all": (342, None), "sum_dim0": (143, None), "mean": (462, None),
             "softmax": (117, None), "mlp32_fwd": (165, 201), "mlp32_bwd": (None, 1219), "h2d": (285, 358), "d2h": (376, 413)},
}


def timeit(fn, dev, iters, warmup):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if dev.type == "cuda":
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        else:
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e6)
    return statistics.median(ts)


def cases(dev):
    g = torch.Generator(device=dev).manual_seed(0)
    r = lambda *s: torch.rand(*s, device=dev, generator=g) + 0.1  # noqa: E731
    a, b = r(1000, 1000), r(1000, 1000)
    # "rand" is this package's own generator (Philox-4x32-10: device kernel, threaded host fill), as the
    # reference's row is its own generator; torch's generator is the second row
    philox = DevicePhilox(0, dev)
    out = {
        "zeros": lambda: ft.zeros((1000, 1000), device=dev), "rand": lambda: philox.uniform(1000, 1000),
        "rand@torch_generator": lambda: ft.rand((1000, 1000), device=dev),
        "add": lambda: a + b, "mul": lambda: a * b, "sub": lambda: a - b, "div": lambda: a / b, "relu": lambda: torch.relu(a),
        "sigmoid": lambda: torch.sigmoid(a), "exp": lambda: torch.exp(a), "log": lambda: torch.log(a), "sin": lambda: torch.sin(a),
        "cos": lambda: torch.cos(a), "tanh": lambda: torch.tanh(a), "sum_all": lambda: a.sum(), "sum_dim0": lambda: ft.sum_dim(a, 0),
        "mean_dim1": lambda: a.mean(1), "mean": lambda: a.mean(), "permute": lambda: a.t().contiguous(), "chunk4": lambda: a.chunk(4),
        "softmax": lambda x=r(64, 256): torch.softmax(x, -1),
    }
    parts = [r(250, 1000) for _ in range(4)]
    out["cat4"] = lambda: torch.cat(parts)
    c1, c2 = r(1000, 1), r(1, 1000)
    out["broadcast_add"] = lambda: c1 + c2
    d1, d2 = r(64, 1, 256), r(1, 128, 1)
    out["broadcast_mul"] = lambda: d1 * d2
    for n in (64, 256, 1024) + ((4096,) if dev.type == "cuda" else ()):
        x, y = r(n, n), r(n, n)
        out["matmul_%d" % n] = lambda x=x, y=y: ft.matmul(x, y)
    for name, batch, dims in (("mlp32", 32, (784, 256, 10)), ("mlp128", 128, (784, 512, 256, 10))):
        layers = []
        for i, o in zip(dims[:-1], dims[1:]):
            layers += [nn.Linear(i, o), nn.ReLU()]
        mlp = nn.Sequential(*layers[:-1]).to(dev)
        x, t = r(batch, 784), torch.randint(0, 10, (batch,), device=dev)
        opt = torch.optim.Adam(mlp.parameters())

        def fwd(mlp=mlp, x=x):
            with torch.no_grad():
                return mlp(x)

        def bwd(mlp=mlp, x=x, t=t):
            mlp.zero_grad(set_to_none=True)
            nn.functional.cross_entropy(mlp(x), t).backward()

        def train(mlp=mlp, x=x, t=t, opt=opt):
            opt.zero_grad(set_to_none=True)
            nn.functional.cross_entropy(mlp(x), t).backward()
            opt.step()

        out[name + "_fwd"], out[name + "_bwd"], out[name + "_train"] = fwd, bwd, train
    conv, cx = nn.Conv2d(3, 16, 3).to(dev), r(32, 3, 32, 32)
    out["conv2d_fwd"] = lambda: conv(cx)
    lstm, lx = nn.LSTM(128, 256, batch_first=True).to(dev), r(16, 32, 128)
    out["lstm_fwd"] = lambda: lstm(lx)
    if dev.type == "cuda":
        host = torch.rand(1000, 1000).pin_memory()
        out["h2d"] = lambda: host.to(dev)
        out["d2h"] = lambda: a.cpu()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--threads", type=int, default=0)
    a = ap.parse_args()
    if a.threads:
        torch.set_num_threads(a.threads)
    dev = torch.device(a.device)
    pub = PUBLISHED[a.device]
    rows = []
    with torch.inference_mode(False):
        for name, fn in cases(dev).items():
            if name.split("@")[0] not in pub:
                continue
            us = timeit(fn, dev, a.iters, a.warmup)
            ref_ft, ref_pt = pub[name.split("@")[0]]
            rows.append({"bench": name, "us": round(us, 1), "reference_ferrotorch_us": ref_ft, "reference_pytorch_us": ref_pt,
                         "speedup_vs_reference": round(ref_ft / us, 2) if ref_ft else None})
    for r in rows:
        print(json.dumps(r))
    faster = sum(1 for r in rows if r["speedup_vs_reference"] and r["speedup_vs_reference"] >= 1.0)
    print(json.dumps({"device": a.device, "threads": torch.get_num_threads(), "benches": len(rows),
                      "at_or_above_the_reference_published_value": faster}))


if __name__ == "__main__":
    main()
