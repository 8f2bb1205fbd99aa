"""Loader and builder for the native libraries of ferrotorch_b200.

Two shared objects are built in-tree (``ferrotorch_b200/_C``):

* ``libft_kernels.so`` -- every hand-written sm_100a CUDA kernel plus its ``extern "C"``
  launcher (``csrc/*.cu``), compiled with
  ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``libft_host.so`` -- the host-only C++ runtime (TCP store + ring collectives, GGUF
  reader, TensorBoard record writer, JIT source cache; ``csrc/host/*.cpp``).

The libraries are plain C ABI and are bound with :mod:`ctypes`: the launchers take raw
device pointers and a ``cudaStream_t`` so the same entry points serve PyTorch tensors,
CUDA-graph capture and callers that are not Python at all.

On a machine with a GPU the kernels library must load; an op whose kernel is missing
raises instead of silently running an eager fallback (the reference has the same
no-silent-fallback policy, ferrotorch-gpu/src/kernels.rs:1-6).
"""
from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
OUT = _PKG / "_C"
KERNELS_SO = OUT / "libft_kernels.so"
HOST_SO = OUT / "libft_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]

_lock = threading.Lock()
_kernels = None
_host = None


def _nvcc() -> str | None:
    for cand in (os.environ.get("FT_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` into ``_C/libft_kernels.so`` (no-op when up to date)."""
    srcs = sorted(CSRC.glob("*.cu"))
    deps = srcs + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not force and KERNELS_SO.exists() and KERNELS_SO.stat().st_mtime >= _newest(deps):
        return KERNELS_SO
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build libft_kernels.so")
    OUT.mkdir(exist_ok=True)
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    hdr_m = _newest(sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")))

    def compile_one(src: Path) -> Path:
        obj = objdir / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            _run(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = KERNELS_SO.with_suffix(".so.tmp%d" % os.getpid())
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"])
    os.replace(tmp, KERNELS_SO)
    return KERNELS_SO


def build_host(force: bool = False) -> Path:
    """Compile ``csrc/host/*.cpp`` into ``_C/libft_host.so`` (no-op when up to date)."""
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    deps = srcs + sorted((CSRC / "host").glob("*.h"))
    if not srcs:
        return HOST_SO
    if not force and HOST_SO.exists() and HOST_SO.stat().st_mtime >= _newest(deps):
        return HOST_SO
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("g++ not found; cannot build libft_host.so")
    OUT.mkdir(exist_ok=True)
    tmp = HOST_SO.with_suffix(".so.tmp%d" % os.getpid())
    _run([cxx, *CXX_FLAGS, "-shared", "-o", str(tmp), *map(str, srcs), "-I", str(CSRC / "host")])
    os.replace(tmp, HOST_SO)
    return HOST_SO


def build(force: bool = False, verbose: bool = False) -> None:
    build_host(force)
    build_kernels(force, verbose)


# --------------------------------------------------------------------------- ctypes prototypes
_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_KERNEL_PROTOS = {
    "ft_launch_count": (_ll, []),
    "ft_last_error": (ctypes.c_char_p, []),
    "ft_read_device_status": (_i, [_i]),
    "ft_abi_version": (_i, []),
    "ft_count_external_launch": (None, [_i]),
    "ft_gemm_bf16": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _i, _vp]),
    "ft_rmsnorm_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp]),
    "ft_rmsnorm_bwd_scratch_rows": (_i, [_i, _i]),
    "ft_rmsnorm_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "ft_rope": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _i, _i, _i, _i, _vp]),
    "ft_swiglu_fwd": (_i, [_vp, _vp, _ll, _i, _ll, _i, _i, _vp]),
    "ft_swiglu_bwd": (_i, [_vp, _vp, _vp, _ll, _i, _ll, _i, _i, _vp]),
    "ft_embedding_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "ft_embedding_bwd": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "ft_adamw_flat": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _i, _vp, _f, _f, _f, _f, _f, _i, _i, _i, _vp]),
    "ft_sgd_flat": (_i, [_vp, _vp, _vp, _vp, _ll, _i, _vp, _f, _f, _f, _f, _i, _i, _i, _vp]),
    "ft_grad_norm_scratch": (_i, [_i]),
    "ft_grad_norm": (_i, [_vp, _ll, _i, _vp, _vp, _f, _vp, _i, _vp]),
    "ft_cross_entropy": (_i, [_vp, _vp, _vp, _i, _i, _ll, _f, _ll, _i, _i, _vp]),
}


def _bind(lib: ctypes.CDLL, protos: dict) -> None:
    for name, (res, args) in protos.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue  # optional symbol (older build); callers check with hasattr
        fn.restype = res
        fn.argtypes = args


def register_protos(protos: dict) -> None:
    """Let other modules of the package declare the entry points they use."""
    _KERNEL_PROTOS.update(protos)
    if _kernels is not None:
        _bind(_kernels, protos)


def kernels(required: bool = True) -> ctypes.CDLL | None:
    """Return the kernels library, building it first when a compiler is available."""
    global _kernels
    if _kernels is not None:
        return _kernels
    with _lock:
        if _kernels is not None:
            return _kernels
        try:
            if os.environ.get("FT_NO_AUTOBUILD") != "1" and _nvcc() is not None:
                build_kernels()
            if not KERNELS_SO.exists():
                raise RuntimeError("%s does not exist (run `python -c 'import __graft_entry__ as g; g.build()'`)" % KERNELS_SO)
            lib = ctypes.CDLL(str(KERNELS_SO), mode=ctypes.RTLD_GLOBAL)
            _bind(lib, _KERNEL_PROTOS)
            _kernels = lib
        except Exception:
            if required:
                raise
            return None
    return _kernels


def host(required: bool = True) -> ctypes.CDLL | None:
    """Return the host runtime library (TCP collectives, GGUF, ...)."""
    global _host
    if _host is not None:
        return _host
    with _lock:
        if _host is not None:
            return _host
        try:
            if os.environ.get("FT_NO_AUTOBUILD") != "1":
                build_host()
            lib = ctypes.CDLL(str(HOST_SO))
            _host = lib
        except Exception:
            if required:
                raise
            return None
    return _host


class NativeError(RuntimeError):
    """A native entry point returned an error code."""


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = _kernels.ft_last_error() if _kernels is not None else b""
        raise NativeError("%s failed (code %d): %s" % (what or "native call", rc, (msg or b"").decode(errors="replace")))


def launch_count() -> int:
    """Kernels launched by libft_kernels.so since it was loaded."""
    lib = kernels(required=False)
    return int(lib.ft_launch_count()) if lib is not None else 0


def device_status(device: int = 0) -> int:
    """Read-and-clear the device status word (non-zero = a bounded wait ran out)."""
    return int(kernels().ft_read_device_status(device))


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(KERNELS_SO, HOST_SO)
