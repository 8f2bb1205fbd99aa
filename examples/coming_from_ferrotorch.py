#!/usr/bin/env python
"""A tour of the reference's API names as they resolve in this package: the flat tensor API and
prelude, optimizer config objects, function-style collectives over in-process ranks, post-training
quantisation, a ResNet folded for inference, and the JIT back-ends.  Runs on CPU in seconds.

    python examples/coming_from_ferrotorch.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import ferrotorch_b200 as ft  # noqa: E402
from ferrotorch_b200.prelude import *  # noqa: E402,F401,F403


def main():
    torch.manual_seed(0)
    # flat tensor API: the reference's spellings, then torch's
    x = ft.from_slice(range(12), [3, 4])
    print("sum_dim:", ft.sum_dim(x, 1, False).tolist(), "| max_with_dim:", ft.max_with_dim(x, 0)[1].tolist())
    print("fft2_norm ortho energy:", float(ft.fft2_norm(x, norm=ft.FftNorm.Ortho).abs().square().sum()), "=", float(x.square().sum()))

    # prelude names + optimizer config objects
    net = Sequential(Linear(4, 8), ReLU(), Linear(8, 2))            # noqa: F405
    opt = ft.optim.AdamWConfig(lr=1e-2, weight_decay=0.0).build(net.parameters())
    for _ in range(50):
        loss = MSELoss()(net(x), x[:, :2])                           # noqa: F405
        opt.zero_grad()
        loss.backward()
        opt.step()
    print("fit loss after 50 AdamW steps: %.4f" % loss.item())

    # function-style collectives with the group as an argument (three ranks as threads)
    def rank_fn(group):
        t = torch.full((2,), float(group.rank + 1))
        return ft.distributed.allreduce(t, group, ft.distributed.ReduceOp.Mean)

    print("allreduce(mean) over 3 simulated ranks:", ft.distributed.run_simulated(3, rank_fn)[0].tolist())

    # post-training quantisation with a calibrated range
    w = torch.randn(64, 64)
    obs = ft.HistogramObserver(512, 0.999)
    obs.observe(w)
    q = ft.quantize(w, qparams=obs.calculate_qparams())
    print("int8 PTQ error (rms): %.4f" % float((ft.ops.ptq.dequantize(q) - w).square().mean().sqrt()))

    # a ResNet folded for inference: batch norm inside the convolutions, ReLU / shortcut in their epilogues
    model = ft.vision.get_model("resnet18", num_classes=10).eval()
    fused = ft.models.resnet.fuse_for_inference(model)
    img = torch.randn(1, 3, 64, 64)
    with torch.no_grad():
        print("folded ResNet max deviation: %.2e" % float((fused(img) - model(img)).abs().max()))

    # JIT: one optimised graph, three ways to run it
    fn = lambda a, b: torch.sigmoid(torch.relu(a * 2.0 + b)) * b     # noqa: E731
    a, b = torch.randn(4, 8), torch.randn(8)
    g = ft.jit.trace(fn, (a, b))
    ft.jit.optimize(g)
    for backend in (ft.jit.InterpreterBackend(), ft.jit.NativeBackend(), ft.jit.InductorBackend()):
        out = backend.compile(g)([a, b])[0]
        print("%-12s max deviation from eager: %.1e" % (backend.name, float((out - fn(a, b)).abs().max())))


if __name__ == "__main__":
    main()
