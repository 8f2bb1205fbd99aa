"""Parity sweep: run an op of this framework against its fp32 PyTorch oracle over a grid of
shapes and report the worst error per op.

The reference ships a CLI that sweeps one op against a PyTorch oracle
(tools/parity-sweep/runner, tools/parity-sweep/oracle.py); this is the same idea over the native
kernels.  ``python -m ferrotorch_b200.utils.parity [--device cuda] [--ops rmsnorm,swiglu]``.
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


def sweep(ops: list[str] | None = None, device: str = "cpu", dtype: torch.dtype | None = None, seed: int = 0) -> list[dict]:
    dev = torch.device(device)
    dtype = dtype or (torch.bfloat16 if dev.type == "cuda" else torch.float32)
    reg = _registry()
    out = []
    for name in ops or list(reg):
        case = reg[name]
        worst, where = 0.0, None
        for shape in case.shapes:
            torch.manual_seed(seed)
            inputs = case.make(dev, dtype, shape)
            got = case.ours(*inputs).float()
            want = case.oracle(*[i.float() if i.is_floating_point() else i for i in inputs]).float()
            err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-6))
            if err >= worst:
                worst, where = err, shape
        out.append({"op": name, "shapes": len(case.shapes), "worst_rel_err": worst, "at": list(where),
                    "tolerance": case.rtol, "ok": worst <= case.rtol, "dtype": str(dtype), "device": str(dev)})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--ops", default="")
    a = ap.parse_args()
    rows = sweep([o for o in a.ops.split(",") if o] or None, a.device)
    for r in rows:
        print(json.dumps(r))
    raise SystemExit(0 if all(r["ok"] for r in rows) else 1)


if __name__ == "__main__":
    main()
