"""Tensor / sequence parallelism on the fused collective GEMM kernels (``csrc/tp_gemm.cu``).

The reference only names these layers in a design document
(.design/phase-7-distributed.md:269-307: column-parallel, row-parallel, parallel embedding); its
``Placement`` vocabulary is in ferrotorch-distributed/src/dtensor.rs:56-67.  Megatron layout:

* activations between blocks are **sequence-sharded** (rank r holds rows ``[r*Ms, (r+1)*Ms)``);
* ``ColumnParallelLinear`` (QKV, gate/up: weight rows sharded) consumes them through
  :func:`TPContext.ag_gemm` -- all-gather fused into the GEMM;
* ``RowParallelLinear`` (o_proj, down_proj: weight columns sharded) produces them through
  :func:`TPContext.gemm_rs` -- reduce-scatter (+ residual add) fused into the GEMM.

``TPContext`` owns the symmetric buffers (gathered-activation buffers, staging buffers, flags)
and the per-slot epochs; every call is stream-ordered and never synchronises with the host.
With ``world_size == 1`` the same kernels run with the collective parts compiled out of the
control flow, which is how single-GPU tests exercise them.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native
from .ddp import SymmetricBuffer, _ptr_array, CommTimeout

_i, _ll, _f, _vp, _u = _native._i, _native._ll, _native._f, _native._vp, ctypes.c_uint
_native.register_protos({
    "ft_tp_counter_words": (_ll, [_i]),
    "ft_tp_ag_gemm": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _vp, _vp, _i, _i, _u, _vp,
                           _i, _ll, _i, _vp]),
    "ft_tp_gemm_rs": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _i, _i, _vp, _vp, _i,
                           _i, _u, _vp, _ll, _i, _vp]),
    "ft_tp_ag_gemm2": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _vp, _vp, _i, _i, _u, _vp,
                            _i, _ll, _i, _vp]),
    "ft_tp_gemm_rs2": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _i, _i, _i, _i, _vp, _vp,
                            _i, _i, _u, _vp, _ll, _i, _vp]),
    "ft_comm_signal_dev": (_i, [_vp, _i, _i, _i, _i, _i, _vp, _i, _vp]),
    "ft_comm_wait_dev": (_i, [_vp, _i, _i, _i, _i, _vp, _ll, _i, _vp]),
})


class _LocalBuffer:
    """World-size-1 stand-in for :class:`SymmetricBuffer`."""

    def __init__(self, numel, dtype, device):
        self.tensor = torch.zeros(numel, dtype=dtype, device=device)
        self.ptrs = [self.tensor.data_ptr()]
        self.ptr_array = _ptr_array(self.ptrs)


class TPContext:
    N_SLOTS = 16

    def __init__(self, group=None, device=None, timeout_ms: int | None = None, n_copy: int = 32):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.timeout_ms = timeout_ms or int(os.environ.get("FT_COMM_TIMEOUT_MS", "30000"))
        self.n_copy = n_copy
        lib = _native.kernels()
        self.flags = self._alloc(int(2 * self.N_SLOTS * 8), torch.int32)
        # per-slot epochs live in device memory: the kernels advance them themselves, so a captured
        # CUDA graph of a decode step replays correctly (a host-side epoch would be frozen in it)
        self.epochs = torch.zeros(self.N_SLOTS, device=self.device, dtype=torch.int32)
        self._buffers: dict = {}
        self._counters: dict = {}
        self._side_stream = None
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count

    @property
    def side_stream(self) -> "torch.cuda.Stream":
        """Stream for collectives that overlap a GEMM on the main stream (backward re-gathers)."""
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        return self._side_stream

    def _alloc(self, numel: int, dtype):
        if self.world == 1:
            return _LocalBuffer(numel, dtype, self.device)
        return SymmetricBuffer(numel, dtype, self.group, self.device)

    def buffer(self, key, numel: int, dtype=torch.bfloat16):
        """A symmetric buffer identified by ``key`` (allocated collectively on first use: every
        rank must request the same keys in the same order)."""
        b = self._buffers.get(key)
        if b is None or b.tensor.numel() < numel:
            b = self._alloc(numel, dtype)
            self._buffers[key] = b
        return b

    def counters(self, key, M: int) -> torch.Tensor:
        lib = _native.kernels()
        n = int(lib.ft_tp_counter_words(M))
        c = self._counters.get(key)
        if c is None or c.numel() < n:
            c = torch.zeros(n, device=self.device, dtype=torch.int32)
            self._counters[key] = c
        return c

    def rows_per_rank(self, M: int) -> int:
        return (M + self.world - 1) // self.world

    # ------------------------------------------------------------------ all-gather -> GEMM
    def gather_buffer(self, slot: int, M: int, K: int) -> torch.Tensor:
        """The ``[M, K]`` gathered-activation buffer of ``slot``; the caller writes its own rows
        ``[rank*Ms, (rank+1)*Ms)`` into it (see :meth:`my_rows`) and then calls :meth:`ag_gemm`."""
        return self.buffer(("xg", slot), M * K).tensor[: M * K].view(M, K)

    def my_rows(self, slot: int, M: int, K: int) -> torch.Tensor:
        ms = self.rows_per_rank(M)
        lo = self.rank * ms
        return self.gather_buffer(slot, M, K)[lo:min(M, lo + ms)]

    def wait_gather_buffer_free(self, slot: int) -> None:
        """Enqueue a wait until every peer has finished reading this rank's rows from the previous
        :meth:`ag_gemm` on ``slot`` (call before overwriting :meth:`my_rows`)."""
        if self.world == 1:
            return
        lib = _native.kernels()
        rc = lib.ft_comm_wait_dev(self.flags.ptrs[self.rank], 1, slot, self.N_SLOTS, self.world,
                                  self._epoch_ptr(slot), self.timeout_ms, self.device.index,
                                  torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ft_comm_wait_dev")

    def _epoch_ptr(self, slot: int) -> int:
        return self.epochs.data_ptr() + 4 * slot

    def ag_gemm(self, slot: int, M: int, w: torch.Tensor, bias: torch.Tensor | None = None,
                out: torch.Tensor | None = None, w_is_kn: bool = False) -> torch.Tensor:
        """``allgather_rows(X) @ w.T`` where this rank's rows of X are already in the gather buffer
        of ``slot``.  ``w``: ``[N_loc, K]``, or ``[K, N_loc]`` with ``w_is_kn`` (then the product
        is ``allgather_rows(X) @ w``, the form the backward GEMMs need).  Returns ``[M, N_loc]``."""
        if w_is_kn:
            K, N = w.shape
        else:
            N, K = w.shape
        assert w.stride(1) == 1
        lib = _native.kernels()
        stream = torch.cuda.current_stream().cuda_stream
        xg = self.buffer(("xg", slot), M * K)
        rc = lib.ft_comm_signal_dev(self.flags.ptr_array, 0, slot, self.N_SLOTS, self.rank, self.world,
                                    self._epoch_ptr(slot), self.device.index, stream)
        _native.check(rc, "ft_comm_signal_dev")
        if out is None:
            out = torch.empty((M, N), device=self.device, dtype=torch.bfloat16)
        rc = lib.ft_tp_ag_gemm2(xg.ptr_array, w.data_ptr(), out.data_ptr(), bias.data_ptr() if bias is not None else None,
                                M, N, K, K, w.stride(0), out.stride(0), int(w_is_kn), self.rank, self.world,
                                self.rows_per_rank(M), self.counters(("ag", slot), M).data_ptr(),
                                self.flags.ptr_array, slot, self.N_SLOTS, 0, self._epoch_ptr(slot), self.n_copy,
                                self.timeout_ms, self.device.index, stream)
        _native.check(rc, "ft_tp_ag_gemm2")
        return out

    def all_gather_rows(self, slot: int, M: int, K: int) -> torch.Tensor:
        """Gather every rank's rows of the ``slot`` buffer into the local copy (the copy CTAs of
        the fused kernel running alone); this rank's rows must already be in :meth:`my_rows`.
        Returns the full ``[M, K]`` buffer."""
        lib = _native.kernels()
        stream = torch.cuda.current_stream().cuda_stream
        xg = self.buffer(("xg", slot), M * K)
        rc = lib.ft_comm_signal_dev(self.flags.ptr_array, 0, slot, self.N_SLOTS, self.rank, self.world,
                                    self._epoch_ptr(slot), self.device.index, stream)
        _native.check(rc, "ft_comm_signal_dev")
        rc = lib.ft_tp_ag_gemm2(xg.ptr_array, None, None, None, M, 0, K, K, 0, 0, 0, self.rank, self.world,
                                self.rows_per_rank(M), self.counters(("ag", slot), M).data_ptr(),
                                self.flags.ptr_array, slot, self.N_SLOTS, 0, self._epoch_ptr(slot), self.n_copy,
                                self.timeout_ms, self.device.index, stream)
        _native.check(rc, "ft_tp_ag_gemm2")
        return xg.tensor[: M * K].view(M, K)

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, slot: int, x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, w_is_kn: bool = False, max_ctas: int = 0) -> torch.Tensor:
        """``reduce_scatter_rows(x @ w.T) (+ residual)``: ``x [M, K_loc]``, ``w [N, K_loc]`` (or
        ``[K_loc, N]`` with ``w_is_kn``: the product is ``x @ w``); returns this rank's ``[Ms, N]``
        rows.  ``out`` may be this rank's rows of a gather buffer."""
        M, K = x.shape
        N = w.shape[1] if w_is_kn else w.shape[0]
        assert w.shape[0 if w_is_kn else 1] == K and w.stride(1) == 1 and x.stride(1) == 1
        ms = self.rows_per_rank(M)
        lib = _native.kernels()
        stage = self.buffer(("stage", slot), self.world * ms * N)
        rows = max(0, min(ms, M - self.rank * ms))
        if out is None:
            out = torch.empty((rows, N), device=self.device, dtype=torch.bfloat16)
        rc = lib.ft_tp_gemm_rs2(x.data_ptr(), w.data_ptr(), stage.ptr_array, out.data_ptr(),
                                residual.data_ptr() if residual is not None else None, M, N, K, x.stride(0),
                                w.stride(0), out.stride(0), residual.stride(0) if residual is not None else N,
                                int(w_is_kn), max_ctas, self.rank, self.world, ms,
                                self.counters(("rs", slot), M).data_ptr(), self.flags.ptr_array, slot, self.N_SLOTS,
                                0, self._epoch_ptr(slot), self.timeout_ms, self.device.index,
                                torch.cuda.current_stream().cuda_stream)
        _native.check(rc, "ft_tp_gemm_rs2")
        return out

    def check_status(self) -> None:
        code = _native.device_status(self.device.index)
        if code != 0:
            raise CommTimeout("a device-side wait ran out (status %d)" % code)
