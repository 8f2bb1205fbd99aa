"""Parity sweep: run an op of this framework against its fp32 PyTorch oracle over a grid of
shapes and report the worst error per op.

The reference ships a CLI that sweeps one op against a PyTorch oracle
(tools/parity-sweep/runner, tools/parity-sweep/oracle.py); this is the same idea over the native
kernels.  ``python -m ferrotorch_b200.utils.parity [--device cuda] [--ops rmsnorm,swiglu]
[--extended] [--random 8] [--out parity_audit.json]``.  ``--extended`` adds the gradient cases and
the remaining ops (rope, fused linear + cross-entropy, GEMM epilogues, Q4_0 and 2:4 linears);
``--random N`` appends N shapes per op drawn around tile edges (multiples of 128 plus or minus a
few rows); ``--out`` writes the rows as the audit file (tools/parity-sweep/parity_audit.json).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass
from typing import Callable

import torch


@dataclass
class OpCase:
    name: str
    make: Callable[[torch.device, torch.dtype, tuple], tuple]     # -> inputs
    ours: Callable[..., torch.Tensor]
    oracle: Callable[..., torch.Tensor]                           # on fp32 copies of the inputs
    shapes: list[tuple]
    rtol: float = 2e-2


def _registry() -> dict[str, OpCase]:
    from ..ops import functional as F
    from ..ops import reference as ref

    def rnd(dev, dt, *shape, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dt)

    cases = [
        OpCase("linear", lambda d, t, s: (rnd(d, t, s[0], s[2]), rnd(d, t, s[1], s[2], scale=0.05)),
               lambda x, w: F.linear(x, w), lambda x, w: x @ w.t(),
               [(128, 256, 512), (300, 264, 320), (1024, 768, 64)]),
        OpCase("rmsnorm", lambda d, t, s: (rnd(d, t, *s), rnd(d, t, s[-1]) + 1.0),
               lambda x, w: F.rmsnorm(x, w, 1e-5), lambda x, w: ref.rmsnorm(x, w, 1e-5),
               [(64, 256), (1000, 4096), (7, 8192)]),
        OpCase("swiglu", lambda d, t, s: (rnd(d, t, *s),), lambda g: F.swiglu(g), lambda g: ref.swiglu(g, 0),
               [(64, 512), (333, 2 * 1408), (16, 2 * 14336)]),
        OpCase("embedding", lambda d, t, s: (torch.randint(0, s[0], (s[2],), device=d), rnd(d, t, s[0], s[1])),
               lambda i, w: F.embedding(i, w), lambda i, w: w[i], [(1000, 64, 77), (4096, 512, 300)], rtol=0.0),
        OpCase("attention", lambda d, t, s: tuple(rnd(d, t, s[0], s[1], h, s[4]) for h in (s[2], s[3], s[3])),
               lambda q, k, v: __import__("ferrotorch_b200.ops.attention", fromlist=["x"]).flash_attention(q, k, v, causal=True),
               lambda q, k, v: ref.attention(q, k, v, True, None, 0)[0],
               [(2, 128, 4, 2, 64), (1, 300, 8, 8, 128), (2, 1024, 8, 2, 128)]),
    ]
    return {c.name: c for c in cases}


def _grads(fn, wrt):
    """``fn(*inputs) -> tensor`` turned into ``-> concatenated gradients`` of a fixed random
    projection of the output with respect to the inputs listed in ``wrt``."""
    def run(*inputs):
        leaves = [t.detach().clone().requires_grad_(i in wrt) if t.is_floating_point() else t for i, t in enumerate(inputs)]
        y = fn(*leaves)
        g = torch.Generator(device="cpu").manual_seed(7)
        w = torch.randn(y.shape, generator=g).to(y.device, y.dtype)
        gs = torch.autograd.grad((y.float() * w.float()).sum(), [leaves[i] for i in wrt])
        return torch.cat([x.float().reshape(-1) / x.float().abs().max().clamp_min(1e-6) for x in gs])
    return run


def _extended() -> dict[str, OpCase]:
    from ..ops import attention as A
    from ..ops import functional as F
    from ..ops import quant as Q
    from ..ops import reference as ref

    def rnd(dev, dt, *shape, scale=1.0):
        return (torch.randn(*shape, device=dev) * scale).to(dt)

    def rope_inputs(d, t, s):
        T, H, D = s
        cos, sin = ref.rope_tables(D, 4096, 10000.0, None, device=d)
        return rnd(d, t, T, H, D), cos, sin, torch.randint(0, 4096, (T,), device=d, dtype=torch.int32)

    def lce_inputs(d, t, s):
        T, V, H = s
        return rnd(d, t, T, H), rnd(d, t, V, H, scale=0.05), torch.randint(0, V, (T,), device=d)

    def q4_inputs(d, t, s):
        M, N, K = s
        nib, sc = Q.quantize_q4_0_planes(torch.randn(N, K, device=d) * 0.05)
        return rnd(d, t, M, K), nib, sc

    def sp_inputs(d, t, s):
        M, N, K = s
        return rnd(d, t, M, K), Q.apply_2_4_mask(torch.randn(N, K, device=d) * 0.05).to(t)

    lin = lambda x, w: F.linear(x, w)                                        # noqa: E731
    att = lambda q, k, v: A.flash_attention(q, k, v, causal=True)            # noqa: E731
    cases = [
        OpCase("linear_bwd", lambda d, t, s: (rnd(d, t, s[0], s[2]), rnd(d, t, s[1], s[2], scale=0.05)),
               _grads(lin, (0, 1)), _grads(lambda x, w: x @ w.t(), (0, 1)), [(128, 256, 512), (300, 264, 320)], rtol=3e-2),
        OpCase("rmsnorm_bwd", lambda d, t, s: (rnd(d, t, *s), rnd(d, t, s[-1]) + 1.0),
               _grads(lambda x, w: F.rmsnorm(x, w, 1e-5), (0, 1)), _grads(lambda x, w: ref.rmsnorm(x, w, 1e-5), (0, 1)),
               [(64, 256), (333, 4096)], rtol=3e-2),
        OpCase("swiglu_bwd", lambda d, t, s: (rnd(d, t, *s),), _grads(lambda g: F.swiglu(g), (0,)),
               _grads(lambda g: ref.swiglu(g, 0), (0,)), [(64, 512), (333, 2 * 1408)], rtol=3e-2),
        OpCase("attention_bwd", lambda d, t, s: tuple(rnd(d, t, s[0], s[1], h, s[4]) for h in (s[2], s[3], s[3])),
               _grads(att, (0, 1, 2)), _grads(lambda q, k, v: ref.attention(q, k, v, True, None, 0)[0], (0, 1, 2)),
               [(2, 128, 4, 2, 64), (1, 300, 8, 8, 128)], rtol=4e-2),
        OpCase("rope", rope_inputs, lambda x, c, s_, p: F.rope_(x.clone(), c, s_, positions=p),
               lambda x, c, s_, p: ref.rope(x, c, s_, p.long()), [(77, 4, 64), (512, 8, 128)]),
        OpCase("linear_cross_entropy", lce_inputs, lambda h, w, y: F.linear_cross_entropy(h, w, y).reshape(1),
               lambda h, w, y: torch.nn.functional.cross_entropy(h @ w.t(), y).reshape(1), [(96, 1000, 64), (300, 4096, 128)]),
        OpCase("gemm_bias_gelu", lambda d, t, s: (rnd(d, t, s[0], s[2]), rnd(d, t, s[1], s[2], scale=0.05), rnd(d, t, s[1])),
               lambda a, b, c: F.gemm_nt(a, b, bias=c, activation="gelu") if a.is_cuda else torch.nn.functional.gelu(a @ b.t() + c),
               lambda a, b, c: torch.nn.functional.gelu(a @ b.t() + c), [(128, 256, 512), (300, 264, 320)]),
        OpCase("q4_0_linear", q4_inputs, lambda x, n, s_: Q.q4_0_linear(x, n, s_),
               lambda x, n, s_: x @ Q.dequant_q4_0_planes(n, s_).float().t(), [(64, 256, 512), (17, 1024, 2048)]),
        OpCase("sparse24_linear", sp_inputs, lambda x, w: Q.sparse24_linear(x, *Q.pack_2_4(w)),
               lambda x, w: x @ w.t(), [(64, 256, 512), (33, 512, 1024)]),
    ]
    return {c.name: c for c in cases}


def _edge_shapes(template: tuple, n: int, seed: int) -> list[tuple]:
    """``n`` variations of a shape with every size above 32 moved to a multiple of 128 plus a small
    offset in [-3, 3] (kept a multiple of 8 where the template is): where tile remainders hide."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        shp = []
        for v in template:
            if v <= 32:
                shp.append(v)
                continue
            base = 128 * int(torch.randint(1, max(2, v // 128 + 2), (1,), generator=g))
            off = int(torch.randint(-3, 4, (1,), generator=g))
            step = 8 if v % 8 == 0 else 1
            shp.append(max(step, (base + off * step)))
        out.append(tuple(shp))
    return out


def sweep(ops: list[str] | None = None, device: str = "cpu", dtype: torch.dtype | None = None, seed: int = 0,
          extended: bool = False, random_shapes: int = 0) -> list[dict]:
    dev = torch.device(device)
    dtype = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
    reg = _registry()
    if extended or (ops and any(o not in reg for o in ops)):
        reg = {**reg, **_extended()}
    unknown = [o for o in (ops or []) if o not in reg]
    if unknown:
        raise KeyError("unknown op(s) %s; known: %s" % (unknown, ", ".join(sorted(reg))))
    out = []
    for name in ops or list(reg):
        case = reg[name]
        worst, where = 0.0, None
        shapes = list(case.shapes) + (_edge_shapes(case.shapes[0], random_shapes, seed) if random_shapes and name not in
                                      ("attention", "attention_bwd", "rope", "q4_0_linear", "sparse24_linear") else [])
        for shape in shapes:
            torch.manual_seed(seed)
            inputs = case.make(dev, dtype, shape)
            got = case.ours(*inputs).float()
            want = case.oracle(*[i.float() if i.is_floating_point() else i for i in inputs]).float()
            err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-6))
            if err >= worst:
                worst, where = err, shape
        out.append({"op": name, "shapes": len(shapes), "worst_rel_err": worst, "at": list(where),
                    "tolerance": case.rtol, "ok": worst <= case.rtol, "dtype": str(dtype), "device": str(dev)})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--ops", default="")
    ap.add_argument("--extended", action="store_true", help="gradient cases and the remaining ops as well")
    ap.add_argument("--random", type=int, default=0, help="extra tile-edge shapes per op")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", default="", help="write the rows to this JSON file")
    a = ap.parse_args()
    rows = sweep([o for o in a.ops.split(",") if o] or None, a.device, seed=a.seed, extended=a.extended,
                 random_shapes=a.random)
    for r in rows:
        print(json.dumps(r))
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"device": a.device, "seed": a.seed, "rows": rows}, f, indent=1)
    raise SystemExit(0 if all(r["ok"] for r in rows) else 1)


if __name__ == "__main__":
    main()
