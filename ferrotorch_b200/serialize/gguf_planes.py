"""GGUF blocks as separate planes (scales, minima, high-bit words, payload words) and their
expansion on any torch device.

The reference's portable GPU crate splits a block stream on the host into typed arrays, uploads
them and expands them with one kernel per block type (ferrotorch-cubecl/src/quant.rs:
``GgufBlockKind`` :74, ``split_q4_0_blocks`` :130 ... ``split_q8_1_blocks`` :301,
``dequantize_q4_0_to_gpu`` :536 and its five siblings).  The fast path of this package does not
split: ``csrc/gguf_dequant.cu`` decodes the raw blocks on the device and ``csrc/quant_gemm.cu``
consumes Q4_0 inside the GEMM.  The plane form is kept for code written against the reference's
API and as an independent oracle: the split is numpy slicing, the expansion a handful of torch
ops that run wherever the planes live.

Block layouts (32 elements each; ``d``, ``m`` fp16 unless stated):

====== ===== ==========================================================
kind   bytes fields
====== ===== ==========================================================
Q4_0   18    d, 16 nibble bytes                  ``(q - 8) * d``
Q4_1   20    d, m, 16 nibble bytes               ``q * d + m``
Q5_0   22    d, 4 high-bit bytes, 16 nibble bytes ``(q - 16) * d``
Q5_1   24    d, m, 4 high-bit bytes, 16 nibble    ``q * d + m``
Q8_0   34    d, 32 int8                          ``q * d``
Q8_1   36    d, s (fp16 sum, unused), 32 int8    ``q * d``
====== ===== ==========================================================

``nibble_order`` is the element order of the 4- and 5-bit kinds: ``"ggml"`` (byte ``j`` holds
elements ``j`` and ``j + 16``, what the file format says) or ``"interleaved"`` (elements ``2j`` and
``2j + 1``, what the reference's decoders emit).
"""
from __future__ import annotations

import enum

import numpy as np
import torch

from .gguf import GGML_Q4_0, GGML_Q4_1, GGML_Q5_0, GGML_Q5_1, GGML_Q8_0, GGML_Q8_1, _order_flag


class GgufBlockKind(enum.IntEnum):
    Q4_0 = GGML_Q4_0
    Q4_1 = GGML_Q4_1
    Q5_0 = GGML_Q5_0
    Q5_1 = GGML_Q5_1
    Q8_0 = GGML_Q8_0
    Q8_1 = GGML_Q8_1

    @property
    def block_elements(self) -> int:
        return 32

    @property
    def block_bytes(self) -> int:
        return {GGML_Q4_0: 18, GGML_Q4_1: 20, GGML_Q5_0: 22, GGML_Q5_1: 24, GGML_Q8_0: 34, GGML_Q8_1: 36}[int(self)]

    @property
    def has_min(self) -> bool:
        return self in (GgufBlockKind.Q4_1, GgufBlockKind.Q5_1)

    @property
    def has_high_bits(self) -> bool:
        return self in (GgufBlockKind.Q5_0, GgufBlockKind.Q5_1)


def _as_bytes(raw) -> np.ndarray:
    if isinstance(raw, torch.Tensor):
        return raw.detach().cpu().contiguous().view(torch.uint8).numpy().reshape(-1)
    return np.frombuffer(bytes(raw), dtype=np.uint8)


def split_blocks(raw, kind: GgufBlockKind, num_blocks: int) -> dict[str, torch.Tensor]:
    """Planes of ``num_blocks`` blocks: ``scales`` fp32 ``[nb]``; ``mins`` fp32 ``[nb]`` (Q4_1, Q5_1);
    ``qh`` int64 ``[nb]`` holding the 32 high bits as an unsigned word (Q5_*); ``words`` int64
    ``[nb, 4]`` (4- and 5-bit kinds: the 16 nibble bytes as little-endian 32-bit words) or
    ``[nb, 8]`` (8-bit kinds: the 32 int8 values, four per word).  Words are stored in int64 so that
    their unsigned value survives on devices without unsigned arithmetic."""
    kind = GgufBlockKind(kind)
    b = _as_bytes(raw)
    need = num_blocks * kind.block_bytes
    if b.size < need:
        raise ValueError("split_blocks: need %d bytes for %d %s blocks, got %d" % (need, num_blocks, kind.name, b.size))
    blk = b[:need].reshape(num_blocks, kind.block_bytes)
    off = 0
    out = {"scales": torch.from_numpy(blk[:, 0:2].copy().view(np.float16).astype(np.float32).reshape(-1))}
    off = 2
    if kind.has_min:
        out["mins"] = torch.from_numpy(blk[:, 2:4].copy().view(np.float16).astype(np.float32).reshape(-1))
        off = 4
    elif kind == GgufBlockKind.Q8_1:
        off = 4                                                    # the stored block sum is not needed to decode
    if kind.has_high_bits:
        out["qh"] = torch.from_numpy(blk[:, off:off + 4].copy().view("<u4").astype(np.int64).reshape(-1))
        off += 4
    out["words"] = torch.from_numpy(blk[:, off:].copy().view("<u4").astype(np.int64))
    return out


def expand_planes(kind: GgufBlockKind, planes: dict[str, torch.Tensor], num_elements: int, device=None, dtype=torch.float32,
                  nibble_order: str = "ggml") -> torch.Tensor:
    """fp32 (or ``dtype``) ``[num_elements]`` on ``device`` (default: where the planes are).  Only the
    planes cross to the device; the expansion is shifts, masks and one multiply-add there."""
    kind = GgufBlockKind(kind)
    interleaved = bool(_order_flag(nibble_order))
    dev = torch.device(device) if device is not None else planes["words"].device
    p = {k: v.to(dev, non_blocking=True) for k, v in planes.items()}
    nb = p["scales"].numel()
    if num_elements != nb * 32:
        raise ValueError("expand_planes: %d blocks hold %d elements, %d asked for" % (nb, nb * 32, num_elements))
    sh8 = torch.arange(4, device=dev) * 8
    by = ((p["words"][:, :, None] >> sh8) & 0xFF).reshape(nb, -1)                      # the payload bytes again
    if kind in (GgufBlockKind.Q8_0, GgufBlockKind.Q8_1):
        q = torch.where(by > 127, by - 256, by)
    else:
        lo, hi = by & 0xF, by >> 4                                                     # [nb, 16] each
        q = torch.stack([lo, hi], 2).reshape(nb, 32) if interleaved else torch.cat([lo, hi], 1)
        if kind.has_high_bits:
            bits = (p["qh"][:, None] >> torch.arange(32, device=dev)) & 1              # bit e belongs to element e
            q = q | (bits << 4)
        if kind == GgufBlockKind.Q4_0:
            q = q - 8
        elif kind == GgufBlockKind.Q5_0:
            q = q - 16
    out = q.to(torch.float32) * p["scales"][:, None]
    if kind.has_min:
        out = out + p["mins"][:, None]
    return out.reshape(-1).to(dtype)


def _split_fn(kind: GgufBlockKind):
    order = ["scales"] + (["mins"] if kind.has_min else []) + (["qh"] if kind.has_high_bits else []) + ["words"]

    def split(raw, num_blocks: int):
        planes = split_blocks(raw, kind, num_blocks)
        return tuple(planes[k] for k in order)
    split.__name__ = "split_%s_blocks" % kind.name.lower()
    split.__doc__ = "``(%s)`` of ``num_blocks`` %s blocks; see :func:`split_blocks`." % (", ".join(order), kind.name)

    def to_gpu(*args, device="cuda", dtype=torch.float32, nibble_order: str = "ggml"):
        *planes, num_elements = args
        if len(planes) != len(order):
            raise TypeError("dequantize_%s_to_gpu takes (%s, num_elements)" % (kind.name.lower(), ", ".join(order)))
        return expand_planes(kind, dict(zip(order, planes)), int(num_elements), device, dtype, nibble_order)
    to_gpu.__name__ = "dequantize_%s_to_gpu" % kind.name.lower()
    to_gpu.__doc__ = ("Upload the planes of :func:`split_%s_blocks` to ``device`` and expand them there; the result stays "
                      "on the device." % kind.name.lower())
    return split, to_gpu


split_q4_0_blocks, dequantize_q4_0_to_gpu = _split_fn(GgufBlockKind.Q4_0)
split_q4_1_blocks, dequantize_q4_1_to_gpu = _split_fn(GgufBlockKind.Q4_1)
split_q5_0_blocks, dequantize_q5_0_to_gpu = _split_fn(GgufBlockKind.Q5_0)
split_q5_1_blocks, dequantize_q5_1_to_gpu = _split_fn(GgufBlockKind.Q5_1)
split_q8_0_blocks, dequantize_q8_0_to_gpu = _split_fn(GgufBlockKind.Q8_0)
split_q8_1_blocks, dequantize_q8_1_to_gpu = _split_fn(GgufBlockKind.Q8_1)
