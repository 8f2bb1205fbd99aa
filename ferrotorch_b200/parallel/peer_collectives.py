"""Stand-alone collectives over NVLink peer memory (this framework's kernels, not NCCL):
all-gather, all-to-all (even and uneven) and all-reduce on symmetric buffers, every device-side
wait bounded.

The reference's GPU collectives are NCCL calls (ferrotorch-distributed/src/gpu_collective.rs,
nccl_backend.rs); its all_to_all / uneven all_to_all are host loops (collective.rs:464-667).
Here one pull kernel (``ft_peer_exchange``) serves all-gather and all-to-all: every rank copies
its input into a symmetric send buffer, raises a ready flag, and pulls its pieces from the peers'
buffers with plain loads; the all-reduce reuses the data-parallel bucket kernel in reduce-only
mode (each rank sums 1/W of the buffer in rank order and writes the result to every rank, so all
ranks end up with bitwise identical values).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from .. import _native
from .ddp import CommTimeout, SymmetricBuffer

_i, _ll, _f, _vp, _u = _native._i, _native._ll, _native._f, _native._vp, ctypes.c_uint
_native.register_protos({
    "ft_peer_exchange": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _u, _i, _ll, _i, _vp]),
})

_SLOT_EXCHANGE, _SLOT_REDUCE, _N_SLOTS = 0, 1, 2


def _align(n: int, a: int = 16) -> int:
    return (n + a - 1) // a * a


class PeerCollectives:
    """``max_bytes``: capacity of the symmetric send buffer (the largest input of any call)."""

    def __init__(self, group=None, device=None, max_bytes: int = 64 << 20, timeout_ms: int | None = None,
                 blocks: int = 0):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.timeout_ms = timeout_ms or int(os.environ.get("FT_COMM_TIMEOUT_MS", "30000"))
        self.blocks = blocks
        pad = 16 * 8 * self.world
        self.capacity = (max_bytes + pad - 1) // pad * pad
        lib = _native.kernels()
        self.send = SymmetricBuffer(self.capacity, torch.uint8, self.group, self.device)
        self.flags = SymmetricBuffer(int(lib.ft_comm_flag_count(_N_SLOTS)), torch.int32, self.group, self.device)
        self.counters = torch.zeros(_N_SLOTS, device=self.device, dtype=torch.int32)
        self.epoch = [0] * _N_SLOTS
        dist.barrier(self.group)

    # ------------------------------------------------------------------ plumbing
    def _wait_done(self, slot: int) -> None:
        """The peers have finished reading this rank's send buffer from the previous call."""
        if self.epoch[slot] == 0:
            return
        rc = _native.kernels().ft_comm_wait(self.flags.ptrs[self.rank], 1, slot, 1, _N_SLOTS, self.world,
                                            self.epoch[slot], self.timeout_ms, self.device.index,
                                            torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ft_comm_wait")

    def _exchange(self, out: torch.Tensor, src_off, dst_off, nbytes) -> None:
        arr = lambda xs: (ctypes.c_longlong * 8)(*list(xs) + [0] * (8 - len(xs)))  # noqa: E731
        self.epoch[_SLOT_EXCHANGE] += 1
        rc = _native.kernels().ft_peer_exchange(
            self.send.ptr_array, out.data_ptr(), arr(src_off), arr(dst_off), arr(nbytes), self.flags.ptr_array,
            self.counters.data_ptr(), _SLOT_EXCHANGE, _N_SLOTS, self.rank, self.world, self.epoch[_SLOT_EXCHANGE],
            self.blocks, self.timeout_ms, self.device.index, torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ft_peer_exchange")

    def _stage(self, x: torch.Tensor, offset: int = 0) -> None:
        b = x.contiguous().view(torch.uint8).reshape(-1)
        self.send.tensor[offset:offset + b.numel()].copy_(b)

    # ------------------------------------------------------------------ collectives
    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """``[n, ...]`` on every rank -> ``[world * n, ...]`` in rank order."""
        nb = x.numel() * x.element_size()
        step = _align(nb)
        assert step <= self.capacity, "input larger than the symmetric buffer"
        self._wait_done(_SLOT_EXCHANGE)
        self._stage(x)
        out = torch.empty(self.world * step, device=self.device, dtype=torch.uint8)
        self._exchange(out, [0] * self.world, [r * step for r in range(self.world)], [step] * self.world)
        if step == nb:
            return out.view(x.dtype).view((self.world * x.shape[0],) + tuple(x.shape[1:]))
        return torch.cat([out[r * step:r * step + nb].view(x.dtype).view(x.shape) for r in range(self.world)])

    def all_to_all(self, x: torch.Tensor, send_counts=None, recv_counts=None) -> torch.Tensor:
        """Rows ``[sum(send_counts), ...]`` split by ``send_counts`` go to ranks 0..W-1; returns the
        rows received, ordered by source rank (``recv_counts[r]`` rows from rank r).  Without
        counts the rows are split evenly."""
        W = self.world
        if send_counts is None:
            assert x.shape[0] % W == 0, "dim 0 must divide by the world size"
            send_counts = recv_counts = [x.shape[0] // W] * W
        assert len(send_counts) == W and len(recv_counts) == W and sum(send_counts) == x.shape[0]
        row = math.prod(x.shape[1:]) * x.element_size()
        slot_bytes = self.capacity // W // 16 * 16
        assert max(send_counts) * row <= slot_bytes and max(recv_counts) * row <= slot_bytes, \
            "a piece is larger than its share of the symmetric buffer"
        self._wait_done(_SLOT_EXCHANGE)
        off = 0
        for d in range(W):                      # piece for rank d sits in slot d of the send buffer
            if send_counts[d]:
                self._stage(x[off:off + send_counts[d]], d * slot_bytes)
            off += send_counts[d]
        steps = [_align(c * row) for c in recv_counts]
        dst, o = [], 0
        for s in steps:
            dst.append(o)
            o += s
        out = torch.empty(max(o, 16), device=self.device, dtype=torch.uint8)
        self._exchange(out, [self.rank * slot_bytes] * W, dst, steps)
        pieces = [out[dst[r]:dst[r] + recv_counts[r] * row].view(x.dtype).view((recv_counts[r],) + tuple(x.shape[1:]))
                  for r in range(W)]
        return torch.cat(pieces) if len(pieces) > 1 else pieces[0].clone()

    def all_reduce_(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """In-place sum / mean of a bf16 or fp32 tensor across ranks."""
        assert x.dtype in (torch.bfloat16, torch.float32) and op in ("sum", "avg", "mean")
        nb = x.numel() * x.element_size()
        unit = 8 * self.world * x.element_size()
        padded = (nb + unit - 1) // unit * unit
        assert padded <= self.capacity, "input larger than the symmetric buffer"
        self._wait_done(_SLOT_EXCHANGE)          # the send buffer is shared with the exchanges
        self._wait_done(_SLOT_REDUCE)
        if padded > nb:
            self.send.tensor[nb:padded].zero_()
        self._stage(x)
        self.epoch[_SLOT_REDUCE] += 1
        lib = _native.kernels()
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.ft_ddp_reduce_update(
            self.send.ptr_array, None, self.flags.ptr_array, None, None, None, self.counters.data_ptr(), 0,
            padded // x.element_size(), self.rank, self.world, _SLOT_REDUCE, _N_SLOTS, self.epoch[_SLOT_REDUCE],
            1.0 if op == "sum" else 1.0 / self.world, int(x.dtype == torch.float32), 0, 0.0, 0.9, 0.999, 1e-8, 0.0,
            1, 0.0, 0.0, 0, self.blocks, self.timeout_ms, self.device.index, stream)
        _native.check(rc, "ft_ddp_reduce_update")
        # every peer has written its slice of the result into this rank's buffer
        rc = lib.ft_comm_wait(self.flags.ptrs[self.rank], 1, _SLOT_REDUCE, 1, _N_SLOTS, self.world,
                              self.epoch[_SLOT_REDUCE], self.timeout_ms, self.device.index, stream)
        _native.check(rc, "ft_comm_wait")
        x.copy_(self.send.tensor[:nb].view(x.dtype).view(x.shape))
        return x

    def reduce_scatter(self, x: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """``[world * n, ...]`` -> this rank's ``[n, ...]`` of the sum (all-reduce, then the slice)."""
        assert x.shape[0] % self.world == 0
        full = self.all_reduce_(x.clone(), op)
        n = x.shape[0] // self.world
        return full[self.rank * n:(self.rank + 1) * n].contiguous()

    def check_status(self) -> None:
        code = _native.device_status(self.device.index)
        if code != 0:
            raise CommTimeout("a device-side wait on a peer ran out (status %d)" % code)
