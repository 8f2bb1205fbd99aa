"""Device runtime vocabulary of the reference's ``ferrotorch-gpu`` crate on top of ``torch.cuda``:
devices, transfers, the caching allocator's statistics, CUDA graphs with private pools, RNG
fork / join, and the memory guard (lib.rs:245-357: ``GpuDevice``, ``cuda`` / ``tensor_to_gpu`` /
``tensor_to_cpu``, ``alloc_zeros``, ``empty_cache`` / ``cached_bytes``, ``CapturedGraph`` /
``begin_capture`` / ``end_capture`` / ``make_graphed_callable`` / ``graph_pool_handle``,
``fork_rng`` / ``join_rng``).  The kernels themselves are in :mod:`ferrotorch_b200.ops`."""
from __future__ import annotations

import contextlib

import torch

from .utils.memory_guard import (MemoryBudgetExceeded, MemoryGuard, MemoryGuardBuilder, OomPolicy,  # noqa: F401
                                 PressureLevel)


class GpuError(RuntimeError):
    pass


def is_available() -> bool:
    return torch.cuda.is_available()


def _need():
    if not torch.cuda.is_available():
        raise GpuError("no CUDA device is available")


class GpuDevice:
    """One ordinal: its properties, default stream and memory figures (device.rs:40-117)."""

    def __init__(self, ordinal: int = 0):
        _need()
        if not 0 <= ordinal < torch.cuda.device_count():
            raise GpuError("device %d outside 0..%d" % (ordinal, torch.cuda.device_count() - 1))
        self.ordinal, self.device = ordinal, torch.device("cuda", ordinal)

    def name(self) -> str:
        return torch.cuda.get_device_name(self.ordinal)

    def compute_capability(self) -> tuple:
        return torch.cuda.get_device_capability(self.ordinal)

    def sm_count(self) -> int:
        return torch.cuda.get_device_properties(self.ordinal).multi_processor_count

    def memory_info(self) -> tuple:
        """``(free_bytes, total_bytes)`` as the driver reports them."""
        return tuple(int(v) for v in torch.cuda.mem_get_info(self.ordinal))

    def default_stream(self):
        return torch.cuda.default_stream(self.ordinal)

    def synchronize(self) -> None:
        torch.cuda.synchronize(self.ordinal)

    # ---- device.rs:60-117
    def stream(self):
        """The stream work is queued on from this thread (the fork made for a capture, when there is one)."""
        return getattr(self, "_stream", None) or torch.cuda.current_stream(self.ordinal)

    def context(self) -> int:
        """The device's primary context, identified by its ordinal (torch creates and owns it)."""
        torch.cuda.init()
        return self.ordinal

    def blas(self) -> int:
        """The cuBLAS handle bound to this thread's current stream on the device (library GEMMs only)."""
        with torch.cuda.device(self.ordinal):
            return torch.cuda.current_blas_handle()

    def fork_for_capture(self) -> "GpuDevice":
        """The same device with a stream of its own: graph capture is not allowed on the default stream."""
        fork = GpuDevice(self.ordinal)
        fork._stream = torch.cuda.Stream(self.ordinal)
        return fork


def get_cuda_device(ordinal: int = 0) -> GpuDevice:
    return GpuDevice(ordinal)


def cuda(tensor: torch.Tensor, ordinal: int = 0, non_blocking: bool = False) -> torch.Tensor:
    _need()
    return tensor.to(torch.device("cuda", ordinal), non_blocking=non_blocking)


cuda_default = tensor_to_gpu = cpu_to_gpu = cuda


def tensor_to_cpu(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.cpu()


gpu_to_cpu = tensor_to_cpu


def alloc_zeros(shape, dtype: torch.dtype = torch.float32, ordinal: int = 0) -> torch.Tensor:
    _need()
    return torch.zeros(tuple(shape), dtype=dtype, device=torch.device("cuda", ordinal))


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


empty_cache_all = empty_cache


def cached_bytes(ordinal: int = 0) -> int:
    """Bytes the caching allocator holds but no tensor uses (pool.rs ``cached_bytes``)."""
    if not torch.cuda.is_available():
        return 0
    return int(torch.cuda.memory_reserved(ordinal) - torch.cuda.memory_allocated(ordinal))


def round_len(nbytes: int) -> int:
    """The size class of the caching allocator (allocator.rs: 512-byte granules below 1 MiB,
    2 MiB granules from there on)."""
    if nbytes <= 0:
        return 512
    if nbytes < (1 << 20):
        return (nbytes + 511) // 512 * 512
    return (nbytes + (2 << 20) - 1) // (2 << 20) * (2 << 20)


# --------------------------------------------------------------------------- CUDA graphs
def graph_pool_handle():
    _need()
    return torch.cuda.graph_pool_handle()


class CapturedGraph:
    """A captured graph and its replay counter (graph.rs:97-500)."""

    def __init__(self, graph: "torch.cuda.CUDAGraph"):
        self.graph, self.num_replays = graph, 0

    def launch(self) -> None:
        self.graph.replay()
        self.num_replays += 1

    replay = launch

    def reset(self) -> None:
        self.graph.reset()

    # ---- graph.rs:477-515.  torch instantiates and uploads a graph when its capture ends and keeps the
    # capture's allocations in a pool that belongs to the graph, so these report rather than act.
    def upload(self) -> None:
        self._uploaded = True

    def is_uploaded(self) -> bool:
        return True

    def has_pool(self) -> bool:
        return True

    def pool(self):
        """The ``(device, id)`` handle of the memory pool that backs the capture's allocations."""
        return self.graph.pool()

    def pool_buffer_count(self) -> int:
        """Blocks currently held by the graph's private pool (0 when the allocator cannot say)."""
        try:
            snap = torch.cuda.memory_snapshot()
            handle = tuple(self.graph.pool())
            return sum(len(seg["blocks"]) for seg in snap if tuple(seg.get("segment_pool_id", ())) == handle)
        except Exception:  # noqa: BLE001 - statistics only
            return 0


@contextlib.contextmanager
def capture(pool=None, stream=None, capture_error_mode: str = "global"):
    """``with capture() as holder: ...`` records the block into a graph whose memory comes from a
    private pool (so replays cannot collide with the eager allocator); ``holder.captured`` is the
    :class:`CapturedGraph` afterwards (graph.rs ``capture_into_private_pool``)."""
    _need()
    g = torch.cuda.CUDAGraph()

    class Holder:
        captured: CapturedGraph | None = None

    h = Holder()
    with torch.cuda.graph(g, pool=pool, stream=stream, capture_error_mode=capture_error_mode):
        yield h
    h.captured = CapturedGraph(g)


def is_stream_capturing() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


def make_graphed_callable(fn, sample_args, num_warmup_iters: int = 3):
    """Capture ``fn`` (a module or function of tensors) into forward and backward graphs
    (graph.rs ``make_graphed_callable``)."""
    _need()
    return torch.cuda.make_graphed_callables(fn, tuple(sample_args), num_warmup_iters=num_warmup_iters)


# --------------------------------------------------------------------------- RNG
def fork_rng(devices=None):
    """Context manager: RNG state of the CPU and the given devices is restored on exit
    (rng.rs ``fork_rng`` / ``join_rng``)."""
    if devices is None:
        devices = list(range(torch.cuda.device_count())) if torch.cuda.is_available() else []
    return torch.random.fork_rng(devices=devices)


def cuda_rng_state(ordinal: int = 0) -> torch.Tensor:
    _need()
    return torch.cuda.get_rng_state(ordinal)


def set_cuda_rng_state(state: torch.Tensor, ordinal: int = 0) -> None:
    _need()
    torch.cuda.set_rng_state(state, ordinal)


# --------------------------------------------------------------------------- explicit begin / end capture, pools
import enum as _enum  # noqa: E402


class CaptureMode(str, _enum.Enum):
    """How strictly other threads' CUDA calls are policed during capture (graph.rs ``CaptureMode``)."""
    Global = "global"
    ThreadLocal = "thread_local"
    Relaxed = "relaxed"

    def __str__(self) -> str:
        return self.value

    def to_cuda(self) -> int:
        """The driver's ``cudaStreamCaptureMode`` value: global 0, thread-local 1, relaxed 2."""
        return {"global": 0, "thread_local": 1, "relaxed": 2}[self.value]


class CaptureStatus(_enum.Enum):
    NotCapturing = "none"
    Active = "active"
    Invalidated = "invalidated"

    def is_capturing(self) -> bool:
        return self is CaptureStatus.Active

    def is_invalidated(self) -> bool:
        return self is CaptureStatus.Invalidated


def capture_status() -> CaptureStatus:
    return CaptureStatus.Active if is_stream_capturing() else CaptureStatus.NotCapturing


class GraphPoolHandle:
    """A graph memory pool that several captures may share (graph.rs ``GraphPoolHandle``)."""

    def __init__(self, handle=None):
        self.handle = handle if handle is not None else graph_pool_handle()
        self._buffers: list = []
        self._sealed = False

    # ---- graph.rs ``CapturePool`` / ``PrivateMemPool``.  torch's graph pool *is* a private pool: blocks a
    # capture allocates stay reserved for the graphs that use the pool.  ``record_buffer`` additionally pins
    # tensors (graph inputs / outputs) for the pool's lifetime; sealing refuses further ones.
    @classmethod
    def with_private_pool(cls, ordinal: int = 0) -> "GraphPoolHandle":
        with torch.cuda.device(ordinal):
            return cls()

    def has_private_pool(self) -> bool:
        return True

    def record_buffer(self, tensor: torch.Tensor) -> None:
        if self._sealed:
            raise GpuError("CapturePool: the pool is sealed; buffers can only be recorded before the capture ends")
        self._buffers.append(tensor)

    def buffer_count(self) -> int:
        return len(self._buffers)

    def clear_buffers(self) -> None:
        self._buffers.clear()

    def seal(self) -> None:
        self._sealed = True

    def unseal(self) -> None:
        self._sealed = False

    def is_capture_pool_sealed(self) -> bool:
        return self._sealed

    def raw(self):
        """The allocator's ``(device, id)`` handle."""
        return self.handle

    def activate(self) -> "MemPoolScope":
        """A scope in which allocations come from this pool (see :class:`MemPoolScope`)."""
        return MemPoolScope(self)


CapturePool = PrivateMemPool = GraphPoolHandle
_live_pools: dict = {}


def capture_pool_for_handle(handle) -> GraphPoolHandle:
    key = id(handle) if not isinstance(handle, tuple) else handle
    return _live_pools.setdefault(key, GraphPoolHandle(handle))


def release_graph_pool_handle(pool: GraphPoolHandle) -> None:
    """Forget a pool; its memory returns to the allocator once the graphs that used it are gone."""
    for k, v in list(_live_pools.items()):
        if v is pool:
            del _live_pools[k]


class GraphCaptureGuard:
    """``begin_capture`` .. ``end_capture`` as an object: capture starts on construction, ``end()``
    (or leaving the ``with`` block) finishes it and yields the :class:`CapturedGraph`.  An
    exception inside the block still ends the capture, so the stream is never left capturing."""

    def __init__(self, pool: GraphPoolHandle | None = None, mode: CaptureMode = CaptureMode.Global, stream=None):
        _need()
        self._g = torch.cuda.CUDAGraph()
        self._cm = torch.cuda.graph(self._g, pool=pool.handle if pool is not None else None, stream=stream,
                                    capture_error_mode=str(mode))
        self._cm.__enter__()
        self.captured: CapturedGraph | None = None

    def end(self) -> CapturedGraph:
        if self.captured is None:
            self._cm.__exit__(None, None, None)
            self.captured = CapturedGraph(self._g)
        return self.captured

    finish = end

    # ---- graph.rs:776-835 constructors
    @classmethod
    def begin(cls, stream=None) -> "GraphCaptureGuard":
        return cls(stream=stream)

    @classmethod
    def begin_with_mode(cls, mode: CaptureMode, stream=None) -> "GraphCaptureGuard":
        return cls(mode=mode, stream=stream)

    @classmethod
    def begin_with_pool(cls, pool: GraphPoolHandle, stream=None) -> "GraphCaptureGuard":
        return cls(pool=pool, stream=stream)

    @classmethod
    def begin_with_pool_mode(cls, pool: GraphPoolHandle, mode: CaptureMode, stream=None) -> "GraphCaptureGuard":
        return cls(pool=pool, mode=mode, stream=stream)

    def status(self) -> CaptureStatus:
        return CaptureStatus.NotCapturing if self.captured is not None else capture_status()

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        if self.captured is None:
            self._cm.__exit__(et, ev, tb)
            if et is None:
                self.captured = CapturedGraph(self._g)
        return False


def begin_capture() -> GraphCaptureGuard:
    return GraphCaptureGuard()


def begin_capture_with_mode(mode: CaptureMode) -> GraphCaptureGuard:
    return GraphCaptureGuard(mode=mode)


def begin_capture_with_pool(pool: GraphPoolHandle) -> GraphCaptureGuard:
    return GraphCaptureGuard(pool)


def begin_capture_with_pool_mode(pool: GraphPoolHandle, mode: CaptureMode) -> GraphCaptureGuard:
    return GraphCaptureGuard(pool, mode)


def end_capture(guard: GraphCaptureGuard) -> CapturedGraph:
    return guard.end()


end_capture_with_pool = end_capture


def capture_into_private_pool(fn, *args, pool: GraphPoolHandle | None = None):
    """Run ``fn(*args)`` under capture with memory from ``pool`` (a fresh one by default);
    returns ``(captured graph, fn's outputs)`` -- the outputs are the static tensors replays fill."""
    g = GraphCaptureGuard(pool or GraphPoolHandle())
    with g:
        out = fn(*args)
    return g.captured, out


class MemPoolScope:
    """Allocations inside the block come from ``pool`` (``torch.cuda.use_mem_pool``)."""

    def __init__(self, pool=None):
        _need()
        self.pool = pool if pool is not None else torch.cuda.MemPool()
        self._cm = torch.cuda.use_mem_pool(self.pool)

    def __enter__(self):
        self._cm.__enter__()
        return self.pool

    def __exit__(self, *exc):
        return self._cm.__exit__(*exc)


# --------------------------------------------------------------------------- remaining type names of the GPU crate
GpuTensor = CudaBuffer = torch.Tensor          # device memory is a torch tensor on a CUDA device
GpuFloat = (torch.float32, torch.float64, torch.bfloat16, torch.float16)
GpuResult = object


def alloc_zeros_f32(n: int, ordinal: int = 0) -> torch.Tensor:
    return alloc_zeros((n,), torch.float32, ordinal)


def alloc_zeros_f64(n: int, ordinal: int = 0) -> torch.Tensor:
    return alloc_zeros((n,), torch.float64, ordinal)


def alloc_zeros_bf16(n: int, ordinal: int = 0) -> torch.Tensor:
    return alloc_zeros((n,), torch.bfloat16, ordinal)


def init_cuda_backend(ordinal: int = 0) -> GpuDevice:
    """Make the device current, create its context and load the kernel library; idempotent."""
    _need()
    torch.cuda.set_device(ordinal)
    torch.cuda.init()
    from . import _native

    _native.kernels()
    return get_cuda_device(ordinal)


class CudaAllocator:
    """Statistics and controls of the caching allocator that serves device tensors (torch's)."""

    def __init__(self, ordinal: int = 0):
        self.ordinal = ordinal

    def allocated_bytes(self) -> int:
        return torch.cuda.memory_allocated(self.ordinal) if is_available() else 0

    def reserved_bytes(self) -> int:
        return torch.cuda.memory_reserved(self.ordinal) if is_available() else 0

    def peak_bytes(self) -> int:
        return torch.cuda.max_memory_allocated(self.ordinal) if is_available() else 0

    def reset_peak_stats(self) -> None:
        if is_available():
            torch.cuda.reset_peak_memory_stats(self.ordinal)

    def empty_cache(self) -> None:
        empty_cache()

    @staticmethod
    def round_len(nbytes: int) -> int:
        return round_len(nbytes)

    # ---- the reference allocator's method names (allocator.rs:101-827) on torch's caching allocator
    memory_allocated = allocated_bytes
    memory_reserved = reserved_bytes
    max_memory_allocated = peak_bytes

    def device(self) -> "torch.device":
        return torch.device("cuda", self.ordinal)

    def cached_bytes(self) -> int:
        """Bytes the allocator holds but no tensor uses."""
        return max(0, self.reserved_bytes() - self.allocated_bytes())

    def cache_stats(self) -> dict:
        """Counters of the caching allocator (hits are allocations served without a driver call)."""
        st = torch.cuda.memory_stats(self.ordinal) if is_available() else {}
        allocs, driver = st.get("allocation.all.allocated", 0), st.get("segment.all.allocated", 0)
        return {"allocations": allocs, "driver_allocations": driver, "cache_hits": max(0, allocs - driver),
                "active_blocks": st.get("active.all.current", 0), "free_blocks": st.get("inactive_split.all.current", 0),
                "reserved_bytes": st.get("reserved_bytes.all.current", 0), "retries": st.get("num_alloc_retries", 0),
                "ooms": st.get("num_ooms", 0)}

    def block_count(self) -> int:
        return self.cache_stats()["active_blocks"]

    def free_block_count(self) -> int:
        return self.cache_stats()["free_blocks"]

    @staticmethod
    def driver_alloc_size(nbytes: int) -> int:
        """What one request costs at the driver: requests below 1 MiB come out of 2 MiB segments in
        512-byte blocks, larger ones are rounded to 2 MiB (``MIN_BLOCK_SIZE`` / ``SMALL_BUFFER`` /
        ``ROUND_LARGE`` of the reference's allocator, the same constants as torch's)."""
        if nbytes <= 0:
            return 0
        if nbytes < (1 << 20):
            return 2 << 20
        return round_len(nbytes)

    def alloc_zeros(self, shape, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        return alloc_zeros(shape, dtype, self.ordinal)

    def alloc_copy(self, data, dtype: torch.dtype | None = None) -> torch.Tensor:
        _need()
        return torch.as_tensor(data, dtype=dtype).to(self.device())

    @staticmethod
    def free(tensor: torch.Tensor) -> int:
        """Drop the tensor's storage (it returns to the cache); returns the bytes it held."""
        n = tensor.numel() * tensor.element_size()
        tensor.set_()
        return n

    @staticmethod
    def record_stream_on_block(tensor: torch.Tensor, stream) -> None:
        """Keep the block from being reused until the work queued on ``stream`` so far has finished."""
        if tensor.is_cuda:
            tensor.record_stream(stream)


# --------------------------------------------------------------------------- typed launcher names (``gpu_<op>_<dtype>``)
# The reference exports one launcher per op and dtype (ferrotorch-gpu/src/lib.rs: gpu_add,
# gpu_relu_bf16, gpu_matmul_bf16_bf16_nt, gpu_topk_f32 ...).  Device tensors carry their dtype here,
# so one function per op serves every suffix; ops that have a kernel of this framework go to it.
def _gpu_op_table() -> dict:
    F = torch.nn.functional

    def native(name):
        def call(*a, **kw):
            from .ops import functional as ops_f

            return getattr(ops_f, name)(*a, **kw)
        return call

    def _bf16_cuda(*ts):
        return all(isinstance(t, torch.Tensor) and t.is_cuda and t.dtype == torch.bfloat16 for t in ts)

    def matmul(a, b):
        # bf16 matrices on a GPU: this library's tcgen05 GEMM (b is read as stored, no transposed copy)
        if _bf16_cuda(a, b) and a.dim() == 2 and b.dim() == 2:
            from .ops import functional as ops_f

            return ops_f.gemm_nt(a, b.t())
        return torch.matmul(a, b)

    def matmul_nt(a, b):
        if _bf16_cuda(a, b) and a.dim() == 2 and b.dim() == 2:
            from .ops import functional as ops_f

            return ops_f.gemm_nt(a, b)
        return a @ b.transpose(-1, -2)

    def flash_attention(q, k, v, causal=False):
        # [batch, heads, seq, head_dim] in and out, as the reference's launcher takes them
        if _bf16_cuda(q, k, v) and q.dim() == 4 and q.shape[-1] in (64, 128) and q.shape[1] % k.shape[1] == 0:
            from .ops.attention import flash_attention as fa

            return fa(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal).transpose(1, 2)
        return F.scaled_dot_product_attention(q, k, v, is_causal=causal)

    def conv2d(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
        from .ops.conv import conv2d as own_conv2d    # falls back to the library for shapes it does not take

        return own_conv2d(x, w, bias, stride, padding, dilation, groups)

    def embedding(w, ids):
        if _bf16_cuda(w) and ids.is_cuda:
            from .ops import functional as ops_f

            return ops_f.embedding(ids, w)
        return F.embedding(ids, w)

    def max_pool2d(x, kernel_size, stride=None, padding=0):
        from .ops.pool import max_pool2d as own_pool

        return own_pool(x, kernel_size, stride, padding)

    def batch_norm_backward(x, grad_out, weight, running_mean, running_var, eps=1e-5, training=True):
        """(grad_input, grad_weight, grad_bias) of a [N, C, ...] batch norm; batch statistics in training,
        the running ones in evaluation (ferrotorch-gpu/src/group_norm.rs:1449)."""
        dims = [0] + list(range(2, x.dim()))
        shape = [1, -1] + [1] * (x.dim() - 2)
        if training:
            mean, var = x.mean(dims), x.var(dims, unbiased=False)
        else:
            mean, var = running_mean, running_var
        inv = torch.rsqrt(var + eps)
        xhat = (x - mean.view(shape)) * inv.view(shape)
        gw, gb = (grad_out * xhat).sum(dims), grad_out.sum(dims)
        gx = grad_out * (weight * inv).view(shape)
        if training:
            m = x.numel() // x.shape[1]
            gx = gx - ((weight * inv).view(shape) / m) * (gb.view(shape) + xhat * gw.view(shape))
        return gx, gw, gb

    def lrn_denominator(x, size, alpha=1e-4, beta=0.75, k=1.0):
        sq = F.pad(x.pow(2).unsqueeze(1), (0, 0) * (x.dim() - 2) + (size // 2, (size - 1) // 2))
        win = sq.unfold(2, size, 1).sum(-1).squeeze(1)
        return k + alpha / size * win

    def local_response_norm_backward(x, grad_out, denom, size, alpha=1e-4, beta=0.75):
        """Input gradient of ``x * denom^-beta`` with ``denom = k + alpha / size * window_sum(x^2)`` over the
        channel window (ferrotorch-gpu/src/group_norm.rs:1963): the direct term plus the window sum of
        ``grad * x * denom^(-beta-1)`` seen from every channel that has this one in its window."""
        t = grad_out * x * denom.pow(-beta - 1.0)
        tp = F.pad(t.unsqueeze(1), (0, 0) * (x.dim() - 2) + ((size - 1) // 2, size // 2))
        back = tp.unfold(2, size, 1).sum(-1).squeeze(1)
        return grad_out * denom.pow(-beta) - (2.0 * alpha * beta / size) * x * back

    def scatter_reduce_nd(x, dim, idx, src, reduce="sum", include_self=True):
        names = {0: "sum", 1: "prod", 2: "amax", 3: "amin", 4: "mean"}
        return x.scatter_reduce(dim, idx, src, names.get(reduce, reduce), include_self=include_self)

    def slice_write_indirect(src, dst, pos):
        """``dst[:, pos] = src`` with the position read on the device (no host read: usable inside a
        captured graph; ferrotorch-gpu/src/kernels.rs:31594)."""
        return dst.index_copy_(1, pos.reshape(1).long(), src.unsqueeze(1))

    def causal_mask_indirect(total_len, n_head, max_pos):
        """``[n_head, max_pos]``: 0 where the column is below the device-resident length, else -1e9
        (ferrotorch-gpu/src/kernels.rs:31670)."""
        col = torch.arange(max_pos, device=total_len.device)
        row = torch.where(col < total_len.reshape(1), 0.0, -1e9).to(torch.float32)
        return row.expand(n_head, max_pos).contiguous()

    return {
        "batch_norm_backward": batch_norm_backward, "local_response_norm_backward": local_response_norm_backward,
        "local_response_norm_denominator": lrn_denominator, "scatter_reduce_nd": scatter_reduce_nd,
        "slice_write_indirect": slice_write_indirect, "causal_mask_indirect": causal_mask_indirect,
        "add": torch.add, "sub": torch.sub, "mul": torch.mul, "neg": torch.neg, "relu": torch.relu, "gelu": F.gelu,
        "silu": F.silu, "softmax": lambda x, dim=-1: torch.softmax(x, dim), "dropout": F.dropout,
        "scale": lambda x, s: x * s, "add_scaled": lambda a, b, s: torch.add(a, b, alpha=s),
        "broadcast_add": torch.add, "broadcast_sub": torch.sub, "broadcast_mul": torch.mul,
        "div_rounding": lambda a, b, mode=None: torch.div(a, b, rounding_mode=mode), "broadcast_div_rounding":
        lambda a, b, mode=None: torch.div(a, b, rounding_mode=mode),
        "matmul": matmul, "matmul_nt": matmul_nt, "bmm": torch.bmm, "small_matmul": matmul,
        "small_bmm": torch.bmm, "matmul_bf16_bf16": matmul, "matmul_bf16_bf16_nt": native("gemm_nt"),
        "swiglu": native("swiglu"), "maxpool2d": max_pool2d,
        "matmul_bf16_bf16_strided_batched": torch.bmm, "matmul_f16_f16_strided_batched": torch.bmm,
        "matmul_bf16_bf16_strided_batched_nt": lambda a, b: torch.bmm(a, b.transpose(1, 2)),
        "broadcast_bmm_bf16_bf16": torch.matmul, "broadcast_bmm_f16_f16": torch.matmul,
        "layernorm": lambda x, w, b, eps=1e-5: F.layer_norm(x, x.shape[-1:], w, b, eps), "rmsnorm": native("rmsnorm"),
        "group_norm": lambda x, g, w=None, b=None, eps=1e-5: F.group_norm(x, g, w, b, eps),
        "local_response_norm": F.local_response_norm, "rope_half": native("rope_"), "fatrelu": lambda x, t: torch.where(x > t, x, torch.zeros_like(x)),
        "embed_lookup": embedding, "embedding_gather": embedding,
        "embedding_gather_bf16_to": lambda w, ids: F.embedding(ids, w).float(),
        "transpose_2d": lambda x: x.t().contiguous(), "permute_0213": lambda x: x.permute(0, 2, 1, 3).contiguous(),
        "transpose_to_heads": lambda x, h: x.reshape(x.shape[0], h, -1).transpose(0, 1).contiguous(),
        "transpose_from_heads": lambda x: x.transpose(0, 1).reshape(x.shape[1], -1).contiguous(),
        "repeat_kv": lambda x, n, dim=0: x.repeat_interleave(n, dim), "repeat_interleave": torch.repeat_interleave,
        "causal_mask": lambda s: s.masked_fill(torch.ones(s.shape[-2:], dtype=torch.bool, device=s.device).triu(1 + s.shape[-1] - s.shape[-2]), float("-inf")),
        "flash_attention": flash_attention,
        "conv2d": conv2d, "nearest_upsample2x": lambda x: F.interpolate(x, scale_factor=2, mode="nearest"),
        "flip": torch.flip, "roll": torch.roll, "histc": torch.histc, "searchsorted": torch.searchsorted,
        "topk": lambda x, k, largest=True: tuple(torch.topk(x, k, -1, largest)), "topk_nd": lambda x, k, dim=-1, largest=True: tuple(torch.topk(x, k, dim, largest)),
        "unique": torch.unique, "unique_consecutive": torch.unique_consecutive, "meshgrid": lambda *t: torch.meshgrid(*t, indexing="ij"),
        "gather_dim": lambda x, dim, idx: torch.gather(x, dim, idx), "scatter_dim": lambda x, dim, idx, src: x.scatter(dim, idx, src),
        "scatter_value_dim": lambda x, dim, idx, v: x.scatter(dim, idx, v), "scatter_add_dim": lambda x, dim, idx, src: x.scatter_add(dim, idx, src),
        "scatter_nd": lambda x, idx, src: x.index_put(tuple(idx.t()), src),
        "scatter_add_nd": lambda x, idx, src: x.index_put(tuple(idx.t()), src, accumulate=True),
        "scatter_value_nd": lambda x, idx, v: x.index_put(tuple(idx.t()), torch.as_tensor(v, dtype=x.dtype, device=x.device)),
        "scatter_add_segments": lambda src, index, dim_size: torch.zeros((dim_size,) + tuple(src.shape[1:]), dtype=src.dtype,
                                                                         device=src.device).index_add_(0, index, src),
        "repeat_interleave_backward": lambda g, n, dim=0: g.unflatten(dim, (-1, n)).sum(dim + 1),
        "broadcast_bool": torch.broadcast_to,
        "slice_read": lambda x, start, n, dim=0: x.narrow(dim, start, n).contiguous(),
        "slice_write": lambda dst, src, start, dim=0: dst.narrow(dim, start, src.shape[dim]).copy_(src),
        "block_reduce_max_abs": lambda x: x.abs().max(), "airy_ai": torch.special.airy_ai, "entr": torch.special.entr,
        "ndtr": torch.special.ndtr, "ndtri": torch.special.ndtri, "zeta": torch.special.zeta,
        "spherical_bessel_j0": torch.special.spherical_bessel_j0, "chebyshev_poly": torch.special.chebyshev_polynomial_t,
        "hermite_h_poly": torch.special.hermite_polynomial_h, "hermite_he_poly": torch.special.hermite_polynomial_he,
        "laguerre_poly": torch.special.laguerre_polynomial_l, "legendre_poly": torch.special.legendre_polynomial_p,
    }


_GPU_OPS: dict | None = None
_DTYPE_SUFFIX = {"f32": torch.float32, "f64": torch.float64, "bf16": torch.bfloat16, "f16": torch.float16}


def _resolve_gpu_op(name: str):
    """``gpu_<op>[_<dtype>][_into]`` -> callable; with a dtype suffix the first tensor argument is checked."""
    global _GPU_OPS
    if _GPU_OPS is None:
        _GPU_OPS = _gpu_op_table()
    base = name[4:]
    into = base.endswith("_into") or base.endswith("_into_on_stream")
    base = base.replace("_into_on_stream", "").replace("_into", "")
    want = None
    if base not in _GPU_OPS:
        for suf, dt in _DTYPE_SUFFIX.items():
            parts = base.split("_")
            if suf in parts:                                      # suffix (relu_bf16) or infix (matmul_f32_nt)
                parts.remove(suf)
                if "_".join(parts) in _GPU_OPS:
                    base, want = "_".join(parts), dt
                    break
        else:
            if base.endswith("_u16") and base[:-4] in _GPU_OPS:      # 16-bit payloads moved without arithmetic
                base = base[:-4]
            else:
                return None
    fn = _GPU_OPS[base]

    def call(*args, **kw):
        first = next((a for a in args if isinstance(a, torch.Tensor) and a.is_floating_point()), None)
        if want is not None and first is not None and first.dtype != want:
            raise GpuError("%s: expected %s tensors, got %s" % (name, want, first.dtype))
        if into:                                                  # trailing argument is the destination
            *ins, out = args
            out.copy_(fn(*ins, **kw))
            return out
        return fn(*args, **kw)

    call.__name__ = name
    return call


def __getattr__(name):
    """Typed launcher names resolve through the table above; memory-guard types are defined in
    ``utils.memory_guard``."""
    if name.startswith("gpu_") and name not in ("gpu_to_cpu",):
        fn = _resolve_gpu_op(name)
        if fn is not None:
            return fn
    table = {"MemoryGuardedDevice": "MemoryGuardedDevice", "MemoryWatchdog": "MemoryWatchdog", "MemoryStats": "MemoryStats",
             "MemoryReservation": "MemoryReservation", "MemoryHook": "MemoryHook",
             "MemoryPressureListener": "MemoryPressureListener", "MemoryGuard": "MemoryGuard",
             "MemoryGuardBuilder": "MemoryGuardBuilder", "PressureLevel": "PressureLevel", "OomPolicy": "OomPolicy"}
    if name in table:
        from .utils import memory_guard

        return getattr(memory_guard, table[name])
    if name in ("PhiloxGenerator", "PhiloxState", "CudaRngManager", "cuda_rng_manager", "fork_rng", "join_rng"):
        from .utils import philox

        return getattr(philox, name)
    if name == "CudaBackendImpl":
        return CudaBackendImpl
    raise AttributeError(name)


class CudaBackendImpl:
    """The reference's backend object (ferrotorch-gpu/src/backend_impl.rs:88: one method per typed
    kernel behind the core crate's dispatch trait) as a namespace over this module's launcher
    table: ``CudaBackendImpl().relu_bf16(x)`` is ``gpu_relu_bf16(x)``.  There is no second back-end
    to dispatch between here, so the object holds only the device ordinal it was made for."""

    def __init__(self, ordinal: int = 0):
        self.ordinal = ordinal

    def __getattr__(self, name):
        fn = _resolve_gpu_op("gpu_" + name)
        if fn is None:
            raise AttributeError("no launcher named gpu_%s" % name)
        return fn

    def default_device(self) -> "GpuDevice":
        return get_cuda_device(self.ordinal)

    def __repr__(self) -> str:
        return "CudaBackendImpl(ordinal=%d)" % self.ordinal
