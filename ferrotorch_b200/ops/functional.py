"""Differentiable front ends of the native sm_100a kernels.

Every op dispatches on the device of its input: CUDA tensors run the hand-written kernel
(and raise if the native library is missing -- no silent eager fallback on a GPU), CPU
tensors run the PyTorch restatement in :mod:`ferrotorch_b200.ops.reference`, which is also
the oracle the GPU tests compare against.

The GEMM front end :func:`gemm_nt` reads operand layout from strides: a logical ``[rows, K]``
operand may be K-major (``stride(-1) == 1``) or MN-major (``stride(0) == 1``).  ``x @ w.T``,
``dy @ w`` and ``dy.T @ x`` therefore all map onto the same tcgen05 kernel without a
transposed copy (the reference launches a transpose kernel before cuBLAS,
ferrotorch-core/src/grad_fns/linalg.rs:1440-1519).
"""
from __future__ import annotations

import torch

from .. import _native
from . import reference as ref

GEMM_OUT_F32, GEMM_ACCUMULATE, GEMM_BIAS, GEMM_BIAS_F32 = 1, 2, 4, 8
GEMM_RELU, GEMM_GELU, GEMM_SILU = 16, 32, 64
_ACT_FLAGS = {None: 0, "relu": GEMM_RELU, "gelu": GEMM_GELU, "silu": GEMM_SILU}

stats = {"gemm_native": 0, "gemm_library": 0, "gemm_small_m": 0}

_native.register_protos({
    "ft_gemm_small_m": (_native._i, [_native._vp] * 6 + [_native._i] * 3 + [_native._ll] * 4 + [_native._i] * 3 + [_native._vp]),
    "ft_gemm_small_m_workspace": (_native._ll, [_native._i, _native._i]),
})
_small_m_ws: dict = {}


def _small_m_workspace(n_floats: int, device) -> torch.Tensor:
    """fp32 workspace of the split-K small-batch GEMM for the current stream (one slice per piece
    of the contraction; contents do not matter between calls)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _small_m_ws.get(key)
    if buf is None or buf.numel() < n_floats:
        buf = torch.empty(n_floats, device=device, dtype=torch.float32)
        _small_m_ws[key] = buf
    return buf


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
                 residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
                 activation: str | None = None, ksplit: int = 0) -> torch.Tensor:
    """``x @ w.T (+ bias) (+ residual)`` for a small batch ``x [M <= 128, K]`` against ``w [N, K]``
    (both bf16, row-major): the decode-time GEMM.  The weight is the 128-row operand of the MMA and
    the contraction is split over the GPU when ``N / 256`` tiles would leave SMs idle."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    flags = _ACT_FLAGS[activation]
    bias_ptr = None
    if bias is not None:
        bias = bias.contiguous()
        flags |= GEMM_BIAS_F32 if bias.dtype == torch.float32 else GEMM_BIAS
        bias_ptr = bias.data_ptr()
    lib = _native.kernels()
    if activation is not None:
        ksplit = 1                      # the activation is applied by the single-pass epilogue only
    if residual is not None and ksplit == 1:
        raise ValueError("gemm_small_m: a residual needs the split path (ksplit != 1)")
    ws = None
    if ksplit != 1:
        ws = _small_m_workspace(int(lib.ft_gemm_small_m_workspace(M, N)), x.device)
    rc = lib.ft_gemm_small_m(x.data_ptr(), w.data_ptr(), out.data_ptr(), bias_ptr,
                             residual.data_ptr() if residual is not None else None,
                             ws.data_ptr() if ws is not None else None, M, N, K, x.stride(0), w.stride(0),
                             out.stride(0), residual.stride(0) if residual is not None else 0, flags, ksplit,
                             _dev(x), _stream())
    _native.check(rc, "ft_gemm_small_m")
    stats["gemm_small_m"] += 1
    return out

_NATIVE = True
_GEMM_CTA_LIMIT = 0


def set_gemm_cta_limit(n: int) -> int:
    """Limit the persistent grid of every GEMM launched from here on to ``n`` CTAs (0 = all SMs);
    returns the previous limit.  The data-parallel layer sets this while its bucket kernels share
    the GPU with the backward pass: a persistent GEMM whose grid does not fit next to them would
    run its left-over CTAs in a second round and take twice as long."""
    global _GEMM_CTA_LIMIT
    old, _GEMM_CTA_LIMIT = _GEMM_CTA_LIMIT, max(0, int(n))
    return old


def set_native(enabled: bool) -> bool:
    """Route every op of this module to its plain-PyTorch path (``False``) or back to the native
    kernels (``True``).  Used to measure a same-model PyTorch baseline; returns the old setting."""
    global _NATIVE
    old, _NATIVE = _NATIVE, bool(enabled)
    return old


def native_enabled() -> bool:
    return _NATIVE



def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dev(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _layout(t: torch.Tensor):
    """Return (mn_major, ld) of a 2-D operand, or None when neither stride is 1."""
    r, k = t.shape
    s0, s1 = t.stride()
    if s1 == 1 and (s0 >= k or r == 1):
        return 0, (s0 if r > 1 else max(s0, k))
    if s0 == 1 and (s1 >= r or k == 1):
        return 1, (s1 if k > 1 else max(s1, r))
    return None


def _gemm_ok(a: torch.Tensor, b: torch.Tensor, la, lb, N: int) -> bool:
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or la is None or lb is None:
        return False
    if N % 8 or la[1] % 8 or lb[1] % 8:
        return False
    return a.data_ptr() % 16 == 0 and b.data_ptr() % 16 == 0


def gemm_nt(a: torch.Tensor, b: torch.Tensor, *, bias: torch.Tensor | None = None,
            out: torch.Tensor | None = None, accumulate: bool = False,
            out_dtype: torch.dtype | None = None, activation: str | None = None,
            bn: int = 0, max_ctas: int = 0) -> torch.Tensor:
    """``out (+)= a @ b.T (+ bias)`` for logical ``a [M,K]``, ``b [N,K]`` (bf16 in, fp32 accumulate)."""
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2, "gemm_nt: contraction mismatch %s x %s" % (tuple(a.shape), tuple(b.shape))
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or a.dtype)
    if not a.is_cuda:
        r = a.float() @ b.float().t()
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            r = r + out.float()
        if activation:
            r = getattr(torch.nn.functional, activation)(r)
        out.copy_(r.to(out.dtype))
        return out
    la, lb = _layout(a), _layout(b)
    if la is None:
        a = a.contiguous(); la = _layout(a)
    if lb is None:
        b = b.contiguous(); lb = _layout(b)
    native_ok = (_gemm_ok(a, b, la, lb, N) and out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
                 and out.stride(0) % (8 if out.dtype == torch.bfloat16 else 4) == 0 and out.data_ptr() % 16 == 0)
    if not native_ok:
        # Unaligned / non-bf16 problems go to the library GEMM; counted, never silent.
        stats["gemm_library"] += 1
        r = torch.matmul(a, b.t()).float()
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            r = r + out.float()
        if activation:
            r = getattr(torch.nn.functional, activation)(r)
        out.copy_(r.to(out.dtype))
        return out
    if (M <= 128 and N >= 1024 and K >= 512 and not accumulate and out.dtype == torch.bfloat16 and la[0] == 0
            and lb[0] == 0 and bn == 0 and max_ctas == 0):
        # decode-sized batch against a large weight: the weight-stationary kernel
        return gemm_small_m(a, b, bias=bias, out=out, activation=activation)
    flags = _ACT_FLAGS[activation]
    if out.dtype == torch.float32:
        flags |= GEMM_OUT_F32
    if accumulate:
        flags |= GEMM_ACCUMULATE
    bias_ptr = None
    if bias is not None:
        bias = bias.contiguous()
        flags |= GEMM_BIAS_F32 if bias.dtype == torch.float32 else GEMM_BIAS
        assert bias.dtype in (torch.float32, torch.bfloat16)
        bias_ptr = bias.data_ptr()
    lib = _native.kernels()
    rc = lib.ft_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), bias_ptr, M, N, K, la[1], lb[1],
                          out.stride(0), la[0], lb[0], flags, bn, max_ctas or _GEMM_CTA_LIMIT, _dev(a), _stream())
    _native.check(rc, "ft_gemm_bf16")
    stats["gemm_native"] += 1
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        # the output is allocated in its final shape (not returned as a view) so that callers
        # may modify it in place
        y = torch.empty((*shp[:-1], w.shape[0]), device=x.device, dtype=x.dtype)
        gemm_nt(x2, w, bias=bias, out=y.view(-1, w.shape[0]))
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.in_shape = shp
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nt(dy2, w.t()).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                # gradient arena of the flat-parameter trainer: accumulate in the GEMM epilogue
                gemm_nt(dy2.t(), x2.t(), out=mg, accumulate=True)
                hook = getattr(w, "grad_ready_hook", None)
                if hook is not None:
                    hook(w)
            else:
                dw = gemm_nt(dy2.t(), x2.t())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T + bias`` with ``w [out, in]`` (ferrotorch-nn/src/linear.rs:166-211)."""
    if not _NATIVE or not x.is_cuda or x.dtype != torch.bfloat16:
        return torch.nn.functional.linear(x, w, bias)
    return _LinearFn.apply(x, w, bias)


# --------------------------------------------------------------------------- RMSNorm
_scratch: dict = {}


def _get_scratch(key, numel: int, device, dtype=torch.float32) -> torch.Tensor:
    """Per-(stream, purpose) scratch buffer, grown on demand and reused across calls."""
    k = (key, device, torch.cuda.current_stream(device).cuda_stream, dtype)
    buf = _scratch.get(k)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1), device=device, dtype=dtype)
        _scratch[k] = buf
    return buf


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        lib = _native.kernels()
        if residual is not None:
            r2 = residual.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
            xs = torch.empty_like(x2)
            rc = lib.ft_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), y.data_ptr(), xs.data_ptr(),
                                    rstd.data_ptr(), rows, H, eps, _dev(x), _stream())
        else:
            xs = x2
            rc = lib.ft_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), None,
                                    rstd.data_ptr(), rows, H, eps, _dev(x), _stream())
        _native.check(rc, "ft_rmsnorm_fwd")
        ctx.save_for_backward(xs, w, rstd)
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        if residual is not None:
            return y.view(x.shape), xs.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres=None):
        xs, w, rstd = ctx.saved_tensors
        rows, H = xs.shape
        dy2 = dy.reshape(rows, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres_ptr = None
        if dres is not None:
            dres = dres.reshape(rows, H)
            dres = dres if dres.is_contiguous() else dres.contiguous()
            dres_ptr = dres.data_ptr()
        dx = torch.empty_like(xs)
        lib = _native.kernels()
        dev = _dev(xs)
        need_dw = ctx.needs_input_grad[1]
        dw = None
        dw_ptr, scr_ptr, flags = None, None, 0
        if need_dw:
            nrows = lib.ft_rmsnorm_bwd_scratch_rows(rows, dev)
            scratch = _get_scratch("rmsnorm_dw", nrows * H, xs.device)
            scr_ptr = scratch.data_ptr()
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                dw_ptr, flags = mg.data_ptr(), (1 if mg.dtype == torch.float32 else 0) | 2
            else:
                dw = torch.empty_like(w)
                dw_ptr, flags = dw.data_ptr(), (1 if dw.dtype == torch.float32 else 0)
        rc = lib.ft_rmsnorm_bwd(dy2.data_ptr(), xs.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres_ptr,
                                dx.data_ptr(), dw_ptr, scr_ptr, rows, H, flags, dev, _stream())
        _native.check(rc, "ft_rmsnorm_bwd")
        if need_dw and dw is None:
            hook = getattr(w, "grad_ready_hook", None)
            if hook is not None:
                hook(w)
        dxv = dx.view(ctx.shape)
        return dxv, dw, None, (dxv if ctx.has_res else None)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5,
            residual: torch.Tensor | None = None):
    """RMSNorm; with ``residual`` returns ``(norm(x + residual), x + residual)`` from one kernel."""
    if not _NATIVE and x.is_cuda:
        # plain-PyTorch baseline path: torch's own fused RMSNorm
        if residual is not None:
            x = x + residual
        y = torch.nn.functional.rms_norm(x, (x.shape[-1],), weight.to(x.dtype), eps)
        return (y, x) if residual is not None else y
    if not _NATIVE or not x.is_cuda or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return ref.rmsnorm(x, weight, eps, residual)
    return _RMSNormFn.apply(x, weight, eps, residual)


# --------------------------------------------------------------------------- RoPE
def _rope_launch(x, cos, sin, positions, n_rot_heads, seq_len, pos_offset, interleaved, backward):
    T = x.numel() // (x.shape[-1] * x.shape[-2])
    D = x.shape[-1]
    ld = x.stride(-3) if x.dim() >= 3 else x.shape[-2] * D
    lib = _native.kernels()
    pos_ptr = None
    if positions is not None:
        positions = positions.to(torch.int32).contiguous()
        pos_ptr = positions.data_ptr()
    rc = lib.ft_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), pos_ptr, T, n_rot_heads, D, ld,
                     seq_len, pos_offset, int(interleaved), int(backward), _dev(x), _stream())
    _native.check(rc, "ft_rope")


class _RopeFn(torch.autograd.Function):
    """In-place rotation of the first ``n_rot_heads`` heads of ``x [..., T, H, D]``."""

    @staticmethod
    def forward(ctx, x, cos, sin, positions, n_rot_heads, seq_len, pos_offset, interleaved):
        ctx.mark_dirty(x)
        ctx.save_for_backward(cos, sin, positions if positions is not None else cos.new_empty(0))
        ctx.cfg = (positions is not None, n_rot_heads, seq_len, pos_offset, interleaved)
        _rope_launch(x, cos, sin, positions, n_rot_heads, seq_len, pos_offset, interleaved, False)
        return x

    @staticmethod
    def backward(ctx, dx):
        cos, sin, positions = ctx.saved_tensors
        has_pos, n_rot, seq_len, off, inter = ctx.cfg
        dx = dx.contiguous() if not dx.is_contiguous() else dx.clone()
        _rope_launch(dx, cos, sin, positions if has_pos else None, n_rot, seq_len, off, inter, True)
        return dx, None, None, None, None, None, None, None


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, *, positions: torch.Tensor | None = None,
          n_rot_heads: int | None = None, seq_len: int = 0, pos_offset: int = 0,
          interleaved: bool = False) -> torch.Tensor:
    """Rotary embedding on a token-major ``[..., T, H, D]`` tensor; rotates heads
    ``[0, n_rot_heads)`` (so a packed QKV buffer rotates q and k and leaves v).  Positions come
    from ``positions`` (int tensor ``[T]``) or ``(t % seq_len) + pos_offset``."""
    H = x.shape[-2]
    n_rot = H if n_rot_heads is None else n_rot_heads
    if not _NATIVE or not x.is_cuda or x.dtype != torch.bfloat16:
        T = x.numel() // (x.shape[-1] * H)
        if positions is None:
            positions = (torch.arange(T, device=x.device) % seq_len) + pos_offset
        xs = x.reshape(T, H, x.shape[-1])
        rot = ref.rope(xs[:, :n_rot], cos, sin, positions.long(), interleaved)
        return torch.cat([rot, xs[:, n_rot:]], dim=1).reshape(x.shape)
    assert x.stride(-1) == 1 and x.stride(-2) == x.shape[-1], "rope_: heads must be packed"
    return _RopeFn.apply(x, cos, sin, positions, n_rot, seq_len, pos_offset, interleaved)


# --------------------------------------------------------------------------- SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2)
        g2 = g2 if g2.stride(-1) == 1 else g2.contiguous()
        T, F = g2.shape[0], F2 // 2
        out = torch.empty((T, F), device=gu.device, dtype=gu.dtype)
        rc = _native.kernels().ft_swiglu_fwd(g2.data_ptr(), out.data_ptr(), T, F, g2.stride(0), act,
                                             _dev(gu), _stream())
        _native.check(rc, "ft_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.act = act
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        T, F = g2.shape[0], g2.shape[1] // 2
        dy2 = dy.reshape(T, F)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dgu = torch.empty((T, 2 * F), device=dy.device, dtype=dy.dtype)
        rc = _native.kernels().ft_swiglu_bwd(dy2.data_ptr(), g2.data_ptr(), dgu.data_ptr(), T, F,
                                             g2.stride(0), ctx.act, _dev(dy), _stream())
        _native.check(rc, "ft_swiglu_bwd")
        return dgu.view(ctx.shape), None


_ACT_ID = {"silu": 0, "relu": 1, "gelu": 2}


def swiglu(gu: torch.Tensor, activation: str = "silu", param: float | None = None) -> torch.Tensor:
    """``act(gate) * up`` for a packed ``[..., 2F]`` projection output.  ``"fatrelu"`` (ProSparse:
    the gate passes where it is >= ``param``, default 0.01, else 0 -- ferrotorch-llama/src/mlp.rs:60-71)
    runs as torch ops; silu / relu / gelu have the fused kernel."""
    if activation == "fatrelu":
        return ref.fatrelu_glu(gu, 0.01 if param is None else param)
    act = _ACT_ID[activation]
    if not _NATIVE or not gu.is_cuda or gu.dtype != torch.bfloat16 or (gu.shape[-1] // 2) % 8:
        return ref.swiglu(gu, act)
    return _SwiGLUFn.apply(gu, act)


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        T, (V, H) = flat.numel(), w.shape
        out = torch.empty((T, H), device=w.device, dtype=w.dtype)
        rc = _native.kernels().ft_embedding_fwd(flat.data_ptr(), w.data_ptr(), out.data_ptr(), T, H, V,
                                                _dev(w), _stream())
        _native.check(rc, "ft_embedding_fwd")
        ctx.save_for_backward(flat, w)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dy):
        flat, w = ctx.saved_tensors
        V, H = w.shape
        dy2 = dy.reshape(-1, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        mg = getattr(w, "main_grad", None)
        dw = None
        if mg is None or mg.dtype != torch.bfloat16:
            dw = torch.zeros_like(w)
            target = dw
        else:
            target = mg
        rc = _native.kernels().ft_embedding_bwd(flat.data_ptr(), dy2.data_ptr(), target.data_ptr(),
                                                flat.numel(), H, V, _dev(w), _stream())
        _native.check(rc, "ft_embedding_bwd")
        if dw is None:
            hook = getattr(w, "grad_ready_hook", None)
            if hook is not None:
                hook(w)
        elif mg is not None:
            mg.add_(dw)
            dw = None
        return None, dw


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Row gather ``weight[ids]`` (ferrotorch-gpu/src/bf16.rs:1065); the backward scatter-adds rows."""
    if not _NATIVE or not weight.is_cuda or weight.dtype != torch.bfloat16 or weight.shape[1] % 8:
        return torch.nn.functional.embedding(ids, weight)
    return _EmbeddingFn.apply(ids, weight)


# --------------------------------------------------------------------------- cross entropy
def cross_entropy_fwd_bwd_(logits: torch.Tensor, target: torch.Tensor, grad_scale: float,
                           ignore_index: int = -100, write_grad: bool = True) -> torch.Tensor:
    """Fused loss + gradient: returns per-row losses (fp32) and overwrites ``logits`` (bf16,
    ``[rows, V]``) with ``(softmax - onehot) * grad_scale``."""
    rows, V = logits.shape
    if not logits.is_cuda:
        loss = ref.cross_entropy(logits, target, ignore_index)
        if write_grad:
            p = torch.softmax(logits.float(), -1)
            valid = target != ignore_index
            oh = torch.zeros_like(p)
            oh[valid, target[valid]] = 1.0
            logits.copy_(((p - oh) * valid[:, None] * grad_scale).to(logits.dtype))
        return loss
    assert logits.dtype == torch.bfloat16 and logits.stride(-1) == 1
    target = target.to(torch.int64).contiguous()
    loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
    rc = _native.kernels().ft_cross_entropy(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), rows, V,
                                            logits.stride(0), float(grad_scale), ignore_index,
                                            int(write_grad), _dev(logits), _stream())
    _native.check(rc, "ft_cross_entropy")
    return loss


class _LinearCrossEntropyFn(torch.autograd.Function):
    """lm_head GEMM + softmax cross-entropy in row chunks: the ``[rows, vocab]`` logits never
    exist as a whole, and the backward GEMMs run in the forward pass on the in-place gradient."""

    @staticmethod
    def forward(ctx, h, w, target, ignore_index, chunk_rows, reduction_denominator):
        rows, H = h.shape
        V = w.shape[0]
        n_valid = reduction_denominator
        losses = torch.empty(rows, device=h.device, dtype=torch.float32)
        need_dh = h.requires_grad
        need_dw = w.requires_grad
        dh = torch.empty_like(h) if need_dh else None
        mg = getattr(w, "main_grad", None)
        dw = None
        if need_dw and mg is None:
            dw = torch.zeros_like(w)
        dw_target = mg if mg is not None else dw
        buf = torch.empty((min(chunk_rows, rows), V), device=h.device, dtype=h.dtype)
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            z = buf[: r1 - r0]
            gemm_nt(h[r0:r1], w, out=z)
            losses[r0:r1] = cross_entropy_fwd_bwd_(z, target[r0:r1], 1.0 / n_valid, ignore_index,
                                                   write_grad=need_dh or need_dw)
            if need_dh:
                gemm_nt(z, w.t(), out=dh[r0:r1])
            if need_dw:
                gemm_nt(z.t(), h[r0:r1].t(), out=dw_target, accumulate=True)
        ctx.save_for_backward(dh if dh is not None else h.new_empty(0))
        ctx.dw = dw
        ctx.used_main_grad = need_dw and mg is not None
        ctx.w = w if ctx.used_main_grad else None
        return losses.sum() / n_valid

    @staticmethod
    def backward(ctx, dloss):
        (dh,) = ctx.saved_tensors
        dh_out = dw_out = None
        if dh.numel():
            dh_out = dh * dloss.to(dh.dtype) if not _is_one(dloss) else dh
        if ctx.dw is not None:
            dw_out = ctx.dw * dloss.to(ctx.dw.dtype) if not _is_one(dloss) else ctx.dw
        if ctx.used_main_grad:
            hook = getattr(ctx.w, "grad_ready_hook", None)
            if hook is not None:
                hook(ctx.w)
        return dh_out, dw_out, None, None, None, None


def _is_one(t: torch.Tensor) -> bool:
    # the loss is normally the root of backward, so its incoming gradient is exactly 1;
    # checking on the host would synchronise, so only trust 0-dim CPU values
    return False if t.is_cuda else float(t) == 1.0


def linear_cross_entropy(h: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, *,
                         ignore_index: int = -100, chunk_rows: int = 4096,
                         num_valid: int | None = None) -> torch.Tensor:
    """Mean next-token cross-entropy of ``h @ weight.T`` against ``target`` without ever
    materialising the full logits.  ``num_valid`` (default: all rows) is the mean's denominator;
    pass the count of non-ignored targets when some are ignored."""
    h2 = h.reshape(-1, h.shape[-1])
    t2 = target.reshape(-1)
    n = num_valid if num_valid is not None else t2.numel()
    if not _NATIVE or not h.is_cuda or h.dtype != torch.bfloat16:
        z = torch.nn.functional.linear(h2, weight)
        return torch.nn.functional.cross_entropy(z.float(), t2, ignore_index=ignore_index, reduction="sum") / n
    return _LinearCrossEntropyFn.apply(h2.contiguous(), weight, t2, ignore_index, chunk_rows, n)


# --------------------------------------------------------------------------- flash attention
_native.register_protos({
    "ft_flash_attn_fwd": (_native._i, [_native._vp] * 5 + [_native._i] * 6 + [_native._ll] * 4 +
                          [_native._f, _native._i, _native._i, _native._i, _native._vp]),
})


def _tok_stride(t: torch.Tensor) -> int:
    """Token stride of a [B, S, H, D] tensor whose heads are packed (head stride == D)."""
    B, S, H, D = t.shape
    assert t.stride(3) == 1 and (H == 1 or t.stride(2) == D), "attention: heads must be packed"
    ld = t.stride(1) if S > 1 else max(t.stride(1), H * D)
    assert B == 1 or t.stride(0) == S * ld, "attention: batch stride must be seq * token stride"
    return ld


def flash_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
                   scale: float | None = None, causal_offset: int | None = None, return_lse: bool = True):
    """Forward only: ``q [B,Sq,Hq,D]``, ``k/v [B,Sk,Hkv,D]`` (may be slices of a packed QKV buffer).
    Returns ``(out [B,Sq,Hq,D], lse [B,Hq,Sq] fp32)``."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = scale if scale is not None else D ** -0.5
    off = (Sk - Sq) if causal_offset is None else causal_offset
    if not q.is_cuda:
        return ref.attention(q, k, v, causal, scale, off)
    out = torch.empty((B, Sq, Hq, D), device=q.device, dtype=q.dtype)
    lse = torch.empty((B, Hq, Sq), device=q.device, dtype=torch.float32) if return_lse else None
    rc = _native.kernels().ft_flash_attn_fwd(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr() if lse is not None else None,
        B, Sq, Sk, Hq, Hkv, D, _tok_stride(q), _tok_stride(k), _tok_stride(v), Hq * D, float(scale),
        int(causal), off, _dev(q), _stream())
    _native.check(rc, "ft_flash_attn_fwd")
    return out, lse
