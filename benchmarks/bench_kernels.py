#!/usr/bin/env python
"""Per-kernel micro-benchmarks with roofline fractions against a measured copy bandwidth and
cuBLAS bf16 throughput (``--hbm-gbs``, ``--bf16-tflops``; defaults are a B200's measured values).

    python benchmarks/bench_kernels.py [--small] [--only gemm,attn,norm,optim,decode,quant,jit,bn,tp]

Timing: CUDA events, 3+ warm-up runs, a 256 MiB buffer is rewritten between timed runs to flush
the 126 MB L2, median of the timed runs.  ``--small`` keeps every case to a few launches and
under ~2 GB (the shape used under ncu).  Prints one JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ferrotorch_b200 import _native  # noqa: E402
from ferrotorch_b200.ops import functional as F  # noqa: E402
from ferrotorch_b200.ops.attention import flash_attention  # noqa: E402


# Roofline denominators: a STREAM-style copy and a cuBLAS bf16 GEMM burst measured on a B200
# (6553 GB/s, 1681.7 TFLOP/s); override with --hbm-gbs / --bf16-tflops for another part.
PEAKS = {"hbm_gbs": 6553.0, "bf16_tflops": 1681.7}


def peaks():
    return PEAKS["hbm_gbs"], PEAKS["bf16_tflops"], "measured"


ITERS, WARM = 10, 3


def bench(fn, iters=None, warm=None):
    iters, warm = iters or ITERS, warm or WARM
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def emit(name, ms, flops=None, nbytes=None, **extra):
    hbm, tf, kind = peaks()
    out = {"kernel": name, "ms": round(ms, 4), **extra}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_%s_bf16_peak" % kind] = round(flops / ms / 1e9 / tf, 3)
    if nbytes:
        out["gbs"] = round(nbytes / ms / 1e6, 1)
        out["frac_of_%s_hbm" % kind] = round(nbytes / ms / 1e6 / hbm, 3)
    print(json.dumps(out), flush=True)


def r(*s):
    return torch.randn(*s, device="cuda", dtype=torch.bfloat16)


def run_gemm(small):
    shapes = [(4096, 4096, 4096)] if small else [(8192, 8192, 8192), (4096, 6144, 4096), (4096, 28672, 4096),
                                                 (4096, 4096, 14336), (16384, 4096, 4096), (64, 28672, 4096)]
    for M, N, K in shapes:
        a, b, c = r(M, K), r(N, K), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        emit("gemm_nt %dx%dx%d" % (M, N, K), bench(lambda: F.gemm_nt(a, b, out=c)), fl)
        if not small:
            emit("gemm_nt one-CTA kernel %dx%dx%d" % (M, N, K), bench(lambda: F.gemm_nt(a, b, out=c, bn=-256)), fl)
            emit("torch.matmul %dx%dx%d" % (M, N, K), bench(lambda: torch.matmul(a, b.t(), out=c)), fl)
            bt, at = r(K, N).t(), r(K, M).t()
            emit("gemm_nn(dgrad) %dx%dx%d" % (M, N, K), bench(lambda: F.gemm_nt(a, bt, out=c)), fl)
            emit("gemm_tn(wgrad) %dx%dx%d" % (M, N, K), bench(lambda: F.gemm_nt(at, bt, out=c)), fl)


def run_attn(small):
    B, S, Hq, Hkv, D = (1, 2048, 16, 4, 128) if small else (4, 4096, 32, 8, 128)
    q, k, v = r(B, S, Hq, D).requires_grad_(), r(B, S, Hkv, D).requires_grad_(), r(B, S, Hkv, D).requires_grad_()
    fl = 4.0 * B * Hq * S * S * D / 2
    emit("flash_fwd B%d S%d" % (B, S), bench(lambda: F.flash_attn_fwd(q, k, v, True)), fl)
    o = flash_attention(q, k, v, causal=True)
    do = r(B, S, Hq, D)
    emit("flash_bwd B%d S%d" % (B, S), bench(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True)), 2.5 * fl)
    if not small:
        qt, kt, vt = (x.detach().transpose(1, 2) for x in (q, k, v))
        emit("sdpa_fwd (library)", bench(lambda: torch.nn.functional.scaled_dot_product_attention(
            qt, kt, vt, is_causal=True, enable_gqa=True)), fl)


def run_norm(small):
    T, H, Fd = (16384, 4096, 14336) if not small else (8192, 4096, 14336)
    x, w = r(T, H), r(H)
    emit("rmsnorm_fwd %dx%d" % (T, H), bench(lambda: F.rmsnorm(x, w)), nbytes=4.0 * T * H)
    gu = r(T, 2 * Fd)
    emit("swiglu_fwd %dx%d" % (T, Fd), bench(lambda: F.swiglu(gu)), nbytes=6.0 * T * Fd)
    gur = gu.clone().requires_grad_()
    act_out = F.swiglu(gur)
    dact = r(T, Fd)
    emit("swiglu_bwd %dx%d" % (T, Fd), bench(lambda: torch.autograd.grad(act_out, gur, dact, retain_graph=True)),
         nbytes=14.0 * T * Fd)
    qkv = r(T, 48, 128)
    cos, sin = (t.cuda() for t in __import__("ferrotorch_b200.ops.reference", fromlist=["x"]).rope_tables(128, 4096, 5e5))
    emit("rope %d tokens" % T, bench(lambda: F._rope_launch(qkv, cos, sin, None, 40, 4096, 0, False, False)),
         nbytes=4.0 * T * 40 * 128)
    V = 128256
    z, tgt = r(2048, V), torch.randint(0, V, (2048,), device="cuda")
    emit("cross_entropy 2048x%d" % V, bench(lambda: F.cross_entropy_fwd_bwd_(z, tgt, 1.0)), nbytes=6.0 * 2048 * V)


def run_optim(small):
    n = (1 << 26) if small else (1 << 29)
    lib = _native.kernels()
    p, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    g, lp = torch.zeros(n, device="cuda", dtype=torch.bfloat16), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    st = torch.cuda.current_stream().cuda_stream
    emit("adamw_flat %d" % n, bench(lambda: lib.ft_adamw_flat(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                                             lp.data_ptr(), n, 0, None, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 0, 0, st)),
         nbytes=28.0 * n)


def run_decode(small):
    from ferrotorch_b200.nn.paged import PagedAttentionManager, PagedKVCache

    B, ctx, Hq, Hkv, D = (16, 1024, 32, 8, 128) if small else (64, 2304, 32, 8, 128)
    cache = PagedKVCache(1, Hkv, D, num_blocks=B * (ctx // 16 + 1), max_seqs=B, max_seq_len=ctx + 16)
    mgr = PagedAttentionManager(cache)
    for _ in range(B):
        mgr.add_sequence(ctx)
    cache.k[0].normal_()
    cache.v[0].normal_()
    q = r(B, Hq, D)
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    emit("paged_decode B%d ctx%d" % (B, ctx), bench(lambda: cache.decode(0, q, lens)), nbytes=4.0 * B * ctx * Hkv * D)
    # the four projections of a Llama-3-8B block at decode batch size: weight bytes / time
    for N, K in ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)):
        x, w, out = r(B, K), r(N, K), torch.empty(B, N, device="cuda", dtype=torch.bfloat16)
        nb = 2.0 * N * K + 2.0 * B * (N + K)
        emit("gemm_small_m %dx%dx%d" % (B, N, K), bench(lambda: F.gemm_small_m(x, w, out=out)), 2.0 * B * N * K, nbytes=nb)
        emit("gemm (128-row batch tile) %dx%dx%d" % (B, N, K), bench(lambda: F.gemm_nt(x, w, out=out, bn=-128)), 2.0 * B * N * K, nbytes=nb)
        emit("torch.matmul %dx%dx%d" % (B, N, K), bench(lambda: torch.matmul(x, w.t(), out=out)), 2.0 * B * N * K, nbytes=nb)


def run_quant(small):
    from ferrotorch_b200.ops import quant as Q

    M, N, K = (256, 4096, 4096) if small else (64, 28672, 8192)
    x, w = r(M, K), r(N, K) * 0.05
    nib, sc = Q.requantize_q4_0(w.float().cpu())
    nib, sc = nib.cuda(), sc.cuda()
    # weight-bound at small M: bytes = the 4-bit weight + its scales
    emit("q4_0_gemm %dx%dx%d" % (M, N, K), bench(lambda: Q.q4_0_linear(x, nib, sc)), 2.0 * M * N * K,
         nbytes=N * K * 0.5 + N * (K // 32) * 2 + 2.0 * M * (N + K))
    vals, meta = Q.pack_2_4(Q.apply_2_4_mask(w.float().cpu()).to(torch.bfloat16))
    vals, meta = vals.cuda(), meta.cuda()
    emit("sparse24_gemm %dx%dx%d" % (M, N, K), bench(lambda: Q.sparse24_linear(x, vals, meta)), 2.0 * M * N * K,
         nbytes=N * K * 1.0 + N * K / 8 + 2.0 * M * (N + K))
    emit("gemm_nt (dense bf16 weight) %dx%dx%d" % (M, N, K), bench(lambda: F.gemm_nt(x, w)), 2.0 * M * N * K,
         nbytes=2.0 * N * K + 2.0 * M * (N + K))


def run_jit(small):
    from ferrotorch_b200 import jit

    n = (1 << 24) if small else (1 << 27)
    a, b = r(n), r(n)

    def chain(x, y):
        return torch.nn.functional.silu(x * 1.5 + y) * y - torch.tanh(x)

    fn = jit.compile(chain, (a, b))
    fn(a, b)
    emit("jit fused elementwise (5 ops) n=%d" % n, bench(lambda: fn(a, b)), nbytes=6.0 * n)
    emit("eager torch, same chain n=%d" % n, bench(lambda: chain(a, b)), nbytes=6.0 * n)


def run_bn(small):
    from torch import nn

    from ferrotorch_b200.ops.batchnorm import batch_norm_act

    N, C, H = (64, 256, 56) if small else (256, 256, 56)
    x = r(N, C, H, H).contiguous(memory_format=torch.channels_last)
    res, dy = torch.randn_like(x), torch.randn_like(x)
    bn = nn.BatchNorm2d(C).cuda().to(torch.bfloat16)
    tot = 2.0 * x.numel()
    emit("bn+relu fwd %dx%dx%dx%d" % (N, C, H, H), bench(lambda: batch_norm_act(x, bn, None, True)), nbytes=3 * tot)
    emit("bn+add+relu fwd", bench(lambda: batch_norm_act(x, bn, res, True)), nbytes=4 * tot)
    xs = x.clone().requires_grad_()
    y = batch_norm_act(xs, bn, None, True)
    emit("bn+relu bwd", bench(lambda: torch.autograd.grad(y, xs, dy, retain_graph=True)), nbytes=5 * tot)
    emit("torch bn+relu fwd (library)", bench(lambda: torch.relu(bn(x))), nbytes=3 * tot)


def run_tp(small):
    """The fused tensor-parallel kernels at world size 1 (collective parts idle): their GEMM core."""
    from ferrotorch_b200.parallel.tensor_parallel import TPContext

    tp = TPContext(None, torch.device("cuda", 0))
    M, N, K = (4096, 4096, 4096) if small else (16384, 6144, 4096)
    x, w, wk = r(M, K), r(N, K), r(K, N)
    tp.my_rows(0, M, K).copy_(x)
    fl = 2.0 * M * N * K
    emit("tp ag_gemm (W=1) %dx%dx%d" % (M, N, K), bench(lambda: tp.ag_gemm(0, M, w)), fl)
    emit("tp ag_gemm [K,N] weight (W=1)", bench(lambda: tp.ag_gemm(0, M, wk, w_is_kn=True)), fl)
    emit("tp gemm_rs (W=1) %dx%dx%d" % (M, N, K), bench(lambda: tp.gemm_rs(1, x, w)), fl)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--only", default="gemm,attn,norm,optim,decode")
    ap.add_argument("--iters", type=int, default=10, help="timed runs per case (1-2 under ncu)")
    ap.add_argument("--warm", type=int, default=3)
    ap.add_argument("--hbm-gbs", type=float, default=PEAKS["hbm_gbs"], help="measured copy bandwidth, GB/s")
    ap.add_argument("--bf16-tflops", type=float, default=PEAKS["bf16_tflops"],
                    help="measured cuBLAS bf16 GEMM throughput (burst), TFLOP/s")
    a = ap.parse_args()
    ITERS, WARM = a.iters, a.warm
    PEAKS.update(hbm_gbs=a.hbm_gbs, bf16_tflops=a.bf16_tflops)
    for name in a.only.split(","):
        {"gemm": run_gemm, "attn": run_attn, "norm": run_norm, "optim": run_optim, "decode": run_decode,
         "quant": run_quant, "jit": run_jit, "bn": run_bn, "tp": run_tp}[name](a.small)
    print(json.dumps({"device_status": _native.device_status(0)}))
