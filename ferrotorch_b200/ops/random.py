"""Device-side random numbers and dropout on the Philox-4x32-10 stream of ``utils.philox``.

The reference draws uniform / normal numbers and dropout masks on the GPU from a Philox
generator whose state is (seed, counter, offset) (ferrotorch-gpu/src/rng.rs:94-300 state and
generator, :830 dropout, :998 uniform, :1460 normal).  Here ``csrc/rng.cu`` addresses the same
stream: output element ``i`` of a call that starts at counter ``c`` uses stream word ``4 c + i``, so

* :class:`DevicePhilox` produces, on the device, exactly the words / uniforms the host
  :class:`~ferrotorch_b200.utils.philox.PhiloxGenerator` produces for the same seed and position
  (normals agree to rounding of ``log`` / ``sincos``);
* :func:`dropout` keeps only ``(seed, counter)`` for the backward pass and regenerates the mask
  there; :func:`swiglu_dropout` does the same inside the SwiGLU kernel.

CPU tensors run the same arithmetic through the host generator.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _native
from ..utils.philox import PhiloxGenerator, philox_4x32_10
from . import functional as F

_i, _vp, _ll, _f = _native._i, _native._vp, _native._ll, _native._f
_u64 = ctypes.c_ulonglong
_native.register_protos({
    "ft_philox_fill": (_i, [_vp, _ll, _u64, _u64, _i, _i, _f, _f, _i, _vp]),
    "ft_philox_dropout": (_i, [_vp, _vp, _ll, _f, _u64, _u64, _i, _i, _vp]),
    "ft_swiglu_dropout": (_i, [_vp, _vp, _vp, _ll, _i, _ll, _f, _u64, _u64, _i, _i, _vp]),
    "ft_philox_words_host": (_i, [_vp, _ll, _u64, _u64]),
})

WORDS, UNIFORM, NORMAL = 0, 1, 2
_MASK64 = 2 ** 64 - 1


_fill_f32 = False        # False = not looked up yet, None = host library unavailable


def _host_fill():
    global _fill_f32
    if _fill_f32 is False:
        try:
            lib = _native.host()
            lib.ftp_fill_f32.argtypes = [_u64, _u64, _ll, _i, _f, _f, _vp, _i]
            lib.ftp_fill_f32.restype = _i
            _fill_f32 = lib.ftp_fill_f32
        except Exception:  # noqa: BLE001 - no compiler / library: the numpy path serves
            _fill_f32 = None
    return _fill_f32


def _host_words(n: int, seed: int, counter: int) -> np.ndarray:
    ctr = np.arange((n + 3) // 4, dtype=np.uint64) + np.uint64(counter & _MASK64)
    return philox_4x32_10(ctr, seed).reshape(-1)[:n]


def _host_u01(n: int, seed: int, counter: int) -> torch.Tensor:
    w = _host_words(n, seed, counter)
    return torch.from_numpy((w >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0))


def keep_mask(n: int, p: float, seed: int, counter: int) -> torch.Tensor:
    """The dropout keep-mask of ``n`` elements at ``(seed, counter)`` built on the host (bool)."""
    return _host_u01(n, seed, counter) >= np.float32(p)


class DevicePhilox:
    """Generator state ``(seed, counter)``; every draw consumes ``ceil(n / 4)`` counter values."""

    def __init__(self, seed: int = 0, device="cuda"):
        self.seed, self.counter, self.device = int(seed) & _MASK64, 0, torch.device(device)

    def manual_seed(self, seed: int) -> "DevicePhilox":
        self.seed, self.counter = int(seed) & _MASK64, 0
        return self

    def get_state(self) -> tuple[int, int]:
        return self.seed, self.counter

    def set_state(self, state: tuple[int, int]) -> None:
        self.seed, self.counter = int(state[0]) & _MASK64, int(state[1]) & _MASK64

    def reserve(self, n: int) -> int:
        """Claim the counter range for ``n`` outputs; returns its first counter."""
        c = self.counter
        self.counter = (c + (n + 3) // 4) & _MASK64
        return c

    def _fill(self, out: torch.Tensor, kind: int, a: float, b: float) -> torch.Tensor:
        n = out.numel()
        c = self.reserve(n)
        if not out.is_cuda:
            fill = _host_fill() if kind != WORDS else None
            if fill is not None:
                # the host library's threaded fill: same stream positions and the same word -> value
                # arithmetic as the device kernel
                buf = out if (out.dtype == torch.float32 and out.is_contiguous()) else torch.empty(n, dtype=torch.float32)
                if fill(c, self.seed, n, kind, float(a), float(b), buf.data_ptr(), torch.get_num_threads()) != 0:
                    raise RuntimeError("ftp_fill_f32 failed")
                if buf is not out:
                    out.copy_(buf.view(out.shape))
                return out
            if kind == WORDS:
                out.copy_(torch.from_numpy(_host_words(n, self.seed, c).astype(np.int64)).view(out.shape))
            elif kind == UNIFORM:
                out.copy_((a + (b - a) * _host_u01(n, self.seed, c)).view(out.shape))
            else:
                g = PhiloxGenerator(self.seed)
                g.counter = c
                out.copy_((a + b * torch.from_numpy(g.generate_normal(4 * ((n + 3) // 4))[:n])).view(out.shape))
            return out
        assert out.is_contiguous()
        rc = _native.kernels().ft_philox_fill(out.data_ptr(), n, self.seed, c, kind, int(out.dtype == torch.bfloat16),
                                              float(a), float(b), F._dev(out), F._stream())
        _native.check(rc, "ft_philox_fill")
        return out

    def words(self, n: int) -> torch.Tensor:
        """``n`` raw 32-bit words as int64 values in ``[0, 2^32)`` (int32 storage on the device side)."""
        if self.device.type != "cuda":
            return self._fill(torch.empty(n, dtype=torch.int64), WORDS, 0, 0)
        raw = self._fill(torch.empty(n, dtype=torch.int32, device=self.device), WORDS, 0, 0)
        return raw.to(torch.int64) & 0xFFFFFFFF

    def uniform(self, *shape, low: float = 0.0, high: float = 1.0, dtype=torch.float32) -> torch.Tensor:
        return self._fill(torch.empty(*shape, dtype=dtype, device=self.device), UNIFORM, low, high)

    def normal(self, *shape, mean: float = 0.0, std: float = 1.0, dtype=torch.float32) -> torch.Tensor:
        return self._fill(torch.empty(*shape, dtype=dtype, device=self.device), NORMAL, mean, std)


_default: dict = {}


def default_generator(device="cuda") -> DevicePhilox:
    device = torch.device(device)
    key = (device.type, device.index)
    if key not in _default:
        _default[key] = DevicePhilox(torch.initial_seed(), device)
    return _default[key]


def manual_seed(seed: int) -> None:
    """Reseed every default device generator of this module."""
    for g in _default.values():
        g.manual_seed(seed)


def _dropout_apply(x: torch.Tensor, p: float, seed: int, counter: int) -> torch.Tensor:
    x = x if x.is_contiguous() else x.contiguous()
    if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32):
        keep = keep_mask(x.numel(), p, seed, counter).view(x.shape).to(x.device)
        return torch.where(keep, x.float() * np.float32(1.0 / (1.0 - p)), torch.zeros((), device=x.device)).to(x.dtype)
    y = torch.empty_like(x)
    rc = _native.kernels().ft_philox_dropout(x.data_ptr(), y.data_ptr(), x.numel(), float(p), seed, counter,
                                             int(x.dtype == torch.float32), F._dev(x), F._stream())
    _native.check(rc, "ft_philox_dropout")
    return y


class _Dropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, p, seed, counter):
        ctx.cfg = (p, seed, counter)
        return _dropout_apply(x, p, seed, counter)

    @staticmethod
    def backward(ctx, gy):
        return _dropout_apply(gy, *ctx.cfg), None, None, None


def dropout(x: torch.Tensor, p: float = 0.5, training: bool = True, generator: DevicePhilox | None = None) -> torch.Tensor:
    """Inverted dropout.  The mask is a function of ``(seed, counter)`` of the generator at call
    time; backward regenerates it instead of storing it."""
    if not training or p <= 0.0:
        return x
    if p >= 1.0:
        return torch.zeros_like(x)
    g = generator or default_generator(x.device)
    return _Dropout.apply(x, float(p), g.seed, g.reserve(x.numel()))


class _SwigluDropout(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, p, seed, counter):
        rows, F2 = gu.shape
        Fd = F2 // 2
        ctx.cfg = (p, seed, counter)
        ctx.save_for_backward(gu)
        if not gu.is_cuda:
            act = torch.nn.functional.silu(gu[:, :Fd].float()) * gu[:, Fd:].float()
            keep = keep_mask(rows * Fd, p, seed, counter).view(rows, Fd)
            return torch.where(keep, act * np.float32(1.0 / (1.0 - p)), torch.zeros(())).to(gu.dtype)
        y = torch.empty((rows, Fd), device=gu.device, dtype=gu.dtype)
        rc = _native.kernels().ft_swiglu_dropout(gu.data_ptr(), y.data_ptr(), None, rows, Fd, gu.stride(0), float(p), seed,
                                                 counter, 0, F._dev(gu), F._stream())
        _native.check(rc, "ft_swiglu_dropout")
        return y

    @staticmethod
    def backward(ctx, gy):
        (gu,) = ctx.saved_tensors
        p, seed, counter = ctx.cfg
        rows, F2 = gu.shape
        Fd = F2 // 2
        gy = gy if gy.is_contiguous() else gy.contiguous()
        if not gu.is_cuda:
            keep = keep_mask(rows * Fd, p, seed, counter).view(rows, Fd)
            d = torch.where(keep, gy.float() * np.float32(1.0 / (1.0 - p)), torch.zeros(()))
            g, u = gu[:, :Fd].float(), gu[:, Fd:].float()
            s = torch.sigmoid(g)
            return torch.cat([d * u * s * (1 + g * (1 - s)), d * g * s], 1).to(gu.dtype), None, None, None
        dgu = torch.empty_like(gu)
        rc = _native.kernels().ft_swiglu_dropout(gu.data_ptr(), gy.data_ptr(), dgu.data_ptr(), rows, Fd, gu.stride(0),
                                                 float(p), seed, counter, 1, F._dev(gu), F._stream())
        _native.check(rc, "ft_swiglu_dropout")
        return dgu, None, None, None


def swiglu_dropout(gu: torch.Tensor, p: float, training: bool = True, generator: DevicePhilox | None = None) -> torch.Tensor:
    """``dropout(silu(gate) * up)`` for ``gu = [gate | up]`` (last dim ``2 F``, bf16 on the GPU) in one
    kernel, forward and backward; with ``p == 0`` or in eval mode this is :func:`functional.swiglu`."""
    if not training or p <= 0.0:
        return F.swiglu(gu)
    shp = gu.shape
    g2 = gu.reshape(-1, shp[-1])
    g2 = g2 if g2.is_contiguous() else g2.contiguous()
    g = generator or default_generator(gu.device)
    out = _SwigluDropout.apply(g2, float(p), g.seed, g.reserve(g2.shape[0] * (shp[-1] // 2)))
    return out.view(*shp[:-1], shp[-1] // 2)
