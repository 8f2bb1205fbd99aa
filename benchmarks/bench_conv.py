#!/usr/bin/env python
"""Convolution kernel and folded-ResNet inference timings on one GPU.

Per layer shape of ResNet-50 (batch 256 unless --batch): this library's convolution (``ops.conv``:
1 x 1 as a GEMM, k x k in the shifted-row form, each with its layout copies) against cuDNN through
``torch.nn.functional.conv2d``, forward and forward + backward (all three gradients), both bf16
channels-last, CUDA events, an L2 flush (a 256 MiB write) between timed iterations.  With --model: images / s of
``FusedInferenceResNet`` (batch norm folded, bias / shortcut / ReLU in the convolution epilogue)
against the eval-mode model.  One JSON line per measurement.

    python benchmarks/bench_conv.py [--batch 64] [--iters 10] [--model]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# (Cin, Cout, kernel, stride, input size): the distinct stride-1 / stride-2 shapes of ResNet-50's stages
LAYERS = [(64, 64, 1, 1, 56), (64, 64, 3, 1, 56), (64, 256, 1, 1, 56), (256, 64, 1, 1, 56), (256, 128, 1, 1, 56),
          (128, 128, 3, 2, 56), (128, 512, 1, 1, 28), (512, 128, 1, 1, 28), (128, 128, 3, 1, 28), (512, 256, 1, 1, 28),
          (256, 256, 3, 2, 28), (256, 1024, 1, 1, 14), (1024, 256, 1, 1, 14), (256, 256, 3, 1, 14), (1024, 512, 1, 1, 14),
          (512, 512, 3, 2, 14), (512, 2048, 1, 1, 7), (2048, 512, 1, 1, 7), (512, 512, 3, 1, 7)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model", action="store_true")
    a = ap.parse_args()
    import torch
    import torch.nn.functional as F

    from ferrotorch_b200.models import resnet as R
    from ferrotorch_b200.ops import conv as C

    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(a.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(a.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / a.iters

    if not a.model:
        for cin, cout, k, stride, hw in LAYERS:
            x = torch.randn(a.batch, cin, hw, hw, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
            w = (torch.randn(cout, cin, k, k, device=dev) / (cin * k * k) ** 0.5).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            pad = k // 2
            ho = C.out_size(hw, k, stride, pad, 1)
            flops = 2.0 * a.batch * ho * ho * cout * cin * k * k
            xg, wg = x.clone().requires_grad_(), w.clone().requires_grad_()
            gy = torch.randn(a.batch, cout, ho, ho, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)

            def fwd_bwd(fn):
                xg.grad = wg.grad = None
                fn(xg, wg).backward(gy)

            C.use_native_conv(True)
            ours = timed(lambda: C.conv2d(x, w, None, stride, pad))
            ours_fb = timed(lambda: fwd_bwd(lambda p, q: C.conv2d(p, q, None, stride, pad)))
            gather = timed(lambda: C.conv2d_gather(x, w, None, stride, pad)) if k > 1 else None
            C.use_native_conv(False)
            lib = timed(lambda: F.conv2d(x, w, None, stride, pad))
            lib_fb = timed(lambda: fwd_bwd(lambda p, q: F.conv2d(p, q, None, stride, pad)))
            print(json.dumps({"bench": "conv2d", "path": C.native_path(x, w, stride, pad, 1), "cin": cin, "cout": cout, "k": k,
                              "stride": stride, "hw": hw, "batch": a.batch, "fwd_ms": ours, "cudnn_fwd_ms": lib,
                              "fwd_bwd_ms": ours_fb, "cudnn_fwd_bwd_ms": lib_fb, "gather_kernel_fwd_ms": gather,
                              "fwd_tflops": flops / ours / 1e9, "cudnn_fwd_tflops": flops / lib / 1e9,
                              "fwd_bwd_tflops": 3 * flops / ours_fb / 1e9, "cudnn_fwd_bwd_tflops": 3 * flops / lib_fb / 1e9,
                              "l2_flush": "256 MiB write"}), flush=True)
        return
    model = R.resnet50().to(dev).bfloat16().to(memory_format=torch.channels_last).eval()
    x = torch.randn(a.batch, 3, 224, 224, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    fused = R.fuse_for_inference(model).to(dev)
    with torch.no_grad():
        base = timed(lambda: model(x))
        C.use_native_conv(False)
        folded = timed(lambda: fused(x))
        C.use_native_conv(True)
        native = timed(lambda: fused(x))
    for name, ms in (("eval_model", base), ("folded_cudnn", folded), ("folded_native", native)):
        print(json.dumps({"bench": "resnet50_inference", "variant": name, "batch": a.batch, "ms": ms,
                          "images_per_s": a.batch / ms * 1e3, "dtype": "bf16", "l2_flush": "256 MiB write"}), flush=True)


if __name__ == "__main__":
    main()
