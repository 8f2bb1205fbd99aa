"""Out-of-bounds and race checks that need no sanitizer: canary zones around a kernel's output,
poison fill to see what a kernel really wrote, and a run-twice bitwise comparison.

The reference leans on Rust's checked indexing and per-launch validation and has no sanitizer lane
(ferrotorch-gpu/src/shape_math.rs, kernels.rs:16289-16333).  For hand-written CUDA the equivalent
is to hand a kernel a view into a larger buffer whose borders hold a known pattern and to look at
the borders afterwards: a store outside the view shows up as a changed canary, on any device,
without instrumenting the kernel.  Works for CPU and CUDA tensors alike.
"""
from __future__ import annotations

import torch

CANARY_BYTE = 0xA5
POISON_BYTE = 0xCD          # 0xCDCD is a bf16 / fp16 NaN-free large negative; 0xCDCDCDCD a float of about -4.3e8


class GuardViolation(AssertionError):
    pass


class GuardedBuffer:
    """``pad`` canary bytes, the payload (poison-filled), ``pad`` canary bytes.  ``view`` is the
    payload as a tensor of the requested shape and dtype; give it to a kernel as its output, then
    call :meth:`check`."""

    def __init__(self, shape, dtype=torch.float32, device="cpu", pad: int = 4096, align: int = 256):
        if pad % align or pad <= 0:
            raise ValueError("GuardedBuffer: pad must be a positive multiple of the alignment")
        self.shape, self.dtype, self.pad = tuple(shape), dtype, pad
        n = 1
        for d in self.shape:
            n *= int(d)
        self.nbytes = n * torch.empty(0, dtype=dtype).element_size()
        body = (self.nbytes + align - 1) // align * align                   # the tail slack is canary too
        self.raw = torch.full((pad + body + pad,), CANARY_BYTE, dtype=torch.uint8, device=device)
        self.raw[pad:pad + self.nbytes] = POISON_BYTE
        self.view = self.raw[pad:pad + self.nbytes].view(dtype).view(self.shape)

    def canaries_intact(self) -> bool:
        lo, hi = self.raw[:self.pad], self.raw[self.pad + self.nbytes:]
        return bool((lo == CANARY_BYTE).all()) and bool((hi == CANARY_BYTE).all())

    def first_violation(self) -> int | None:
        """Byte offset relative to the payload start (negative = before it) of the first changed canary."""
        bad = (self.raw != CANARY_BYTE)
        bad[self.pad:self.pad + self.nbytes] = False
        idx = bad.nonzero()
        return None if idx.numel() == 0 else int(idx[0]) - self.pad

    def unwritten_bytes(self) -> int:
        """Payload bytes that still hold the poison pattern (an upper bound on what the kernel skipped:
        a value whose bytes happen to equal the pattern counts too)."""
        return int((self.raw[self.pad:self.pad + self.nbytes] == POISON_BYTE).sum())

    def check(self, fully_written: bool = False) -> None:
        if not self.canaries_intact():
            raise GuardViolation("write outside the output: first changed byte at offset %d of a %d-byte payload"
                                 % (self.first_violation(), self.nbytes))
        if fully_written:
            # a run of poison as long as an element of the widest dtype in play marks an element the kernel never stored
            width = max(4, torch.empty(0, dtype=self.dtype).element_size())
            body = (self.raw[self.pad:self.pad + self.nbytes] == POISON_BYTE)
            usable = body.numel() // width * width
            if usable and bool(body[:usable].view(-1, width).all(dim=1).any()):
                raise GuardViolation("the kernel left part of its output unwritten (%d poison bytes remain)" % self.unwritten_bytes())


def guarded_like(t: torch.Tensor, pad: int = 4096) -> GuardedBuffer:
    """A guarded buffer holding a copy of ``t`` (for in-place kernels: run them on ``.view``)."""
    g = GuardedBuffer(t.shape, t.dtype, t.device, pad)
    g.view.copy_(t)
    return g


def run_twice_bitwise(fn, *args, **kw):
    """Call ``fn`` twice on the same inputs and require bit-identical results -- a cheap detector
    of races and of reads of uninitialised memory in kernels that are meant to be deterministic.
    Returns the (first) result."""
    def flat(o):
        if isinstance(o, torch.Tensor):
            return [o]
        if isinstance(o, (list, tuple)):
            return [t for x in o for t in flat(x)]
        return []

    a = fn(*args, **kw)
    a_saved = [t.detach().clone() for t in flat(a)]
    b = fn(*args, **kw)
    for i, (x, y) in enumerate(zip(a_saved, flat(b))):
        same = x.shape == y.shape and x.dtype == y.dtype and bool(
            (x.contiguous().view(torch.uint8) == y.contiguous().view(torch.uint8)).all()) if x.numel() else True
        if not same:
            diff = int((x != y).sum()) if x.shape == y.shape else -1
            raise GuardViolation("output %d differs between two identical runs (%d elements)" % (i, diff))
    return a
