"""Data-parallel training with the gradient all-reduce fused into the optimizer update.

``FusedDDP`` plugs into :class:`ferrotorch_b200.train.engine.FlatTrainer`.  The parameter and
gradient arenas are allocated in symmetric memory (every rank can address every peer's copy
over NVLink).  The arena is cut into buckets in reverse parameter order like the reference's
``compute_buckets`` (ferrotorch-distributed/src/ddp.rs:230-258, 25 MB default there); when the
last weight-gradient kernel of a bucket has been enqueued, one ``ft_ddp_reduce_update`` launch
on a side stream pulls this rank's 1/W slice of the bucket from every rank, averages it in fp32
in rank order, applies AdamW / SGD to the fp32 master weights and moments of the slice and pushes
the new bf16 weights to every rank -- overlapped with the rest of backward.  Every element is
reduced and updated by exactly one rank, so replicas stay bitwise identical.

``mode="nccl"`` is the baseline path: bucketed ``all_reduce`` (average) through NCCL on the
side stream, then the local full-arena update.

The reference's DDP synchronises after ``backward()`` returns, through host memory
(ddp.rs:117-123, 265-311); ``broadcast_parameters`` mirrors ddp.rs:176-186.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native

_i, _ll, _f, _vp, _u = _native._i, _native._ll, _native._f, _native._vp, ctypes.c_uint
_native.register_protos({
    "ft_comm_flag_count": (_ll, [_i]),
    "ft_ddp_reduce_update": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _i, _i, _i, _i, _u, _f, _i, _i,
                                  _f, _f, _f, _f, _f, _i, _f, _f, _i, _i, _ll, _i, _vp]),
    "ft_comm_wait": (_i, [_vp, _i, _i, _i, _i, _i, _u, _ll, _i, _vp]),
    "ft_comm_signal": (_i, [_vp, _i, _i, _i, _i, _i, _u, _i, _vp]),
    "ft_allgather": (_i, [_vp, _vp, _ll, _vp, _i, _i, _i, _i, _u, _ll, _i, _vp]),
})


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * 8)()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class SymmetricBuffer:
    """A tensor in symmetric memory plus the table of peer pointers to it."""

    def __init__(self, numel: int, dtype: torch.dtype, group, device):
        import torch.distributed._symmetric_memory as symm

        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm.rendezvous(self.tensor, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.ptr_array = _ptr_array(self.ptrs)


def compute_buckets(ranges, slots, bucket_elems: int, align: int):
    """Cut the arena ranges into buckets of ``bucket_elems`` elements (boundaries multiples of
    ``align``; a bucket never straddles a parameter-group boundary).  Returned in reverse arena
    order -- the order in which backward produces gradients -- each with the parameters that
    overlap it (a large parameter belongs to several buckets)."""
    cuts = []
    for _, (s, e) in ranges.items():
        lo = s
        while lo < e:
            hi = min(e, lo + bucket_elems)
            cuts.append((lo, hi))
            lo = hi
    out = []
    for lo, hi in sorted(cuts, reverse=True):
        assert lo % align == 0 and (hi - lo) % align == 0, "arena ranges must be multiples of %d" % align
        members = [p for _, p, o, k in slots if o < hi and o + k > lo]
        out.append({"lo": lo, "hi": hi, "params": members})
    return out


class FusedDDP:
    def __init__(self, group=None, mode: str = "fused", bucket_mb: float = 256.0, comm_blocks: int = 32,
                 timeout_ms: int | None = None, late_params=(), tail_blocks: int | None = None):
        assert mode in ("fused", "nccl")
        self.group = group if group is not None else dist.group.WORLD
        self.mode = mode
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.bucket_mb = bucket_mb
        self.comm_blocks = comm_blocks
        # While backward runs, a bucket kernel is kept to ``comm_blocks`` CTAs so that it does not
        # take SMs from the GEMMs; buckets that are still unlaunched when backward has ended (the
        # embedding table's, whose gradient is produced last) get ``tail_blocks`` CTAs: every SM.
        self.tail_blocks = tail_blocks or torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self.timeout_ms = timeout_ms or int(os.environ.get("FT_COMM_TIMEOUT_MS", "30000"))
        self.fused_update = mode == "fused"
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.stream = torch.cuda.Stream(self.device)
        self.epoch = 0
        self._symm: list[SymmetricBuffer] = []
        self.late = {id(p) for p in late_params}
        self.last_micro_batch = True
        # with measure_exposed the time the compute stream spends blocked on the exchange at the
        # end of a step is recorded with CUDA events (read it with exposed_ms())
        self.measure_exposed = False
        self._exposed_events: list = []
        self.reduce_only = False
        self._limited = False

    # the trainer allocates its arenas through this (symmetric memory in fused mode)
    def allocator(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        if self.mode != "fused":
            return torch.zeros(numel, device=self.device, dtype=dtype)
        pad = 8 * self.world * 64
        n = (numel + pad - 1) // pad * pad
        buf = SymmetricBuffer(n, dtype, self.group, self.device)
        self._symm.append(buf)
        return buf.tensor[:numel]

    def _symm_of(self, t: torch.Tensor) -> SymmetricBuffer:
        for b in self._symm:
            if b.tensor.data_ptr() == t.data_ptr():
                return b
        raise KeyError("tensor is not one of this DDP's symmetric buffers")

    def attach(self, trainer) -> None:
        a = trainer.arena
        self.trainer = trainer
        if self.mode == "fused" and trainer.max_grad_norm:
            # Global-norm clipping needs the norm of the fully reduced gradient before any element
            # is updated, so the bucket kernels only reduce (the averaged gradient lands in every
            # rank's arena, still overlapped with backward) and the norm + clipped update run
            # locally afterwards.  Every value is still produced by exactly one rank, so the
            # replicas stay bitwise identical.
            self.reduce_only = True
            self.fused_update = False
        align = 8 * self.world
        elems = max(align, int(self.bucket_mb * 1024 * 1024 / a.params.element_size()) // align * align)
        self.buckets = compute_buckets(a.ranges, a.slots, elems, align)
        self.n_slots = len(self.buckets)
        assert 64 % align == 0, "fused data parallelism needs a world size of 1, 2, 4 or 8"
        self._buckets_of: dict[int, list[int]] = {}
        for bi, b in enumerate(self.buckets):
            for p in b["params"]:
                self._buckets_of.setdefault(id(p), []).append(bi)
                p.grad_ready_hook = self._on_grad_ready
        # parameters whose gradient comes from a plain torch op (no main_grad epilogue): fold
        # ``.grad`` into the arena as soon as autograd has accumulated it, then count it as ready
        def _fold(p):
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
                self._on_grad_ready(p)

        for p in {id(q): q for b in self.buckets for q in b["params"]}.values():
            p.register_post_accumulate_grad_hook(_fold)
        if self.mode == "fused":
            lib = _native.kernels()
            self.p_buf, self.g_buf = self._symm_of(a.params), self._symm_of(a.grads)
            self.flags = SymmetricBuffer(int(lib.ft_comm_flag_count(self.n_slots)), torch.int32, self.group,
                                         self.device)
            self.counters = torch.zeros(self.n_slots, device=self.device, dtype=torch.int32)
        dist.barrier(self.group)

    # ------------------------------------------------------------------ per step
    def begin_step(self) -> None:
        self.epoch += 1
        self._pending = [len([p for p in b["params"] if id(p) not in self.late]) for b in self.buckets]
        self._launched = [False] * self.n_slots
        self.last_micro_batch = self.trainer.micro_batches == 1
        self._mb_seen = 0

    def note_micro_batch(self, index: int, total: int) -> None:
        self.last_micro_batch = index == total - 1

    def _on_grad_ready(self, p) -> None:
        if not self.last_micro_batch or id(p) in self.late:
            return
        for bi in self._buckets_of[id(p)]:
            self._pending[bi] -= 1
            if self._pending[bi] == 0 and not self._launched[bi]:
                self._launch(bi)

    def _launch(self, bi: int, blocks: int | None = None) -> None:
        self._launched[bi] = True
        if blocks is None and self.mode == "fused" and not self._limited:
            # From the first bucket on, the bucket kernels (clusters of two CTAs, so they take
            # whole SM pairs) hold ``comm_blocks`` SMs until backward ends: keep the persistent
            # GEMMs of the rest of backward to the SMs that stay free.
            from ..ops import functional as F

            F.set_gemm_cta_limit(max(2, (self.tail_blocks - self.comm_blocks) // 2 * 2))
            self._limited = True
        b = self.buckets[bi]
        tr = self.trainer
        cur = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        self.stream.wait_event(ev)
        lo, hi = b["lo"], b["hi"]
        n_pad = hi - lo
        if self.mode == "nccl":
            with torch.cuda.stream(self.stream):
                dist.all_reduce(tr.arena.grads[lo:hi], op=dist.ReduceOp.AVG, group=self.group)
            return
        wd = tr.weight_decay if self._group_of(lo) == "decay" else 0.0
        kind = 0 if self.reduce_only else {"adamw": 1, "adam": 2, "sgd": 3}[tr.kind]
        lib = _native.kernels()
        rc = lib.ft_ddp_reduce_update(
            self.g_buf.ptr_array, self.p_buf.ptr_array, self.flags.ptr_array,
            tr.master.data_ptr(), tr.exp_avg.data_ptr() if tr.exp_avg is not None else None,
            tr.exp_avg_sq.data_ptr() if tr.exp_avg_sq is not None else None, self.counters.data_ptr(),
            lo, n_pad, self.rank, self.world, bi, self.n_slots, self.epoch, 1.0 / self.world,
            int(tr.arena.grads.dtype == torch.float32), kind, tr.lr, tr.betas[0], tr.betas[1], tr.eps, wd,
            tr.step_count + 1, tr.momentum, tr.dampening, int(tr.nesterov), blocks or self.comm_blocks,
            self.timeout_ms, self.device.index, self.stream.cuda_stream)
        _native.check(rc, "ft_ddp_reduce_update")

    def _group_of(self, offset: int) -> str:
        for g, (s, e) in self.trainer.arena.ranges.items():
            if s <= offset < e:
                return g
        return "decay"

    def finish_step(self, trainer) -> None:
        """Launch what backward did not trigger, then make the compute stream wait for the
        whole exchange (all peers' slices written into this rank's parameter arena)."""
        self.last_micro_batch = True
        if self._limited:
            from ..ops import functional as F

            F.set_gemm_cta_limit(0)
            self._limited = False
        for bi in range(self.n_slots):
            if not self._launched[bi]:
                self._launch(bi, self.tail_blocks)       # backward is over: nothing left to share the SMs with
        if self.mode == "fused":
            lib = _native.kernels()
            rc = lib.ft_comm_wait(self.flags.ptrs[self.rank], 1, 0, self.n_slots, self.n_slots, self.world,
                                  self.epoch, self.timeout_ms, self.device.index, self.stream.cuda_stream)
            _native.check(rc, "ft_comm_wait")
        ev = torch.cuda.Event()
        ev.record(self.stream)
        cur = torch.cuda.current_stream(self.device)
        if self.measure_exposed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(cur)
            cur.wait_event(ev)
            e1.record(cur)
            self._exposed_events.append((e0, e1))
        else:
            cur.wait_event(ev)

    def exposed_ms(self) -> list[float]:
        """Per finished step: milliseconds the compute stream waited for the gradient exchange
        after backward had ended (synchronises; needs ``measure_exposed = True``)."""
        torch.cuda.synchronize(self.device)
        return [a.elapsed_time(b) for a, b in self._exposed_events]

    def broadcast_parameters(self, trainer, root: int = 0) -> None:
        """Make every replica start from rank ``root``'s weights and optimizer state."""
        for t in (trainer.arena.params, trainer.master, trainer.exp_avg, trainer.exp_avg_sq):
            if t is not None:
                dist.broadcast(t, src=dist.get_global_rank(self.group, root), group=self.group)
        torch.cuda.synchronize()

    def check_status(self) -> None:
        code = _native.device_status(self.device.index)
        if code != 0:
            raise CommTimeout("a device-side wait on a peer ran out (status %d)" % code)


class CommTimeout(RuntimeError):
    """A bounded device-side wait on a peer's flag ran out (mirrors the reference's
    ``DistributedError::Timeout``, ferrotorch-distributed/src/error.rs:21-66)."""
