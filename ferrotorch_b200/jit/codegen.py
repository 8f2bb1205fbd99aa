"""Fused-elementwise code generation: a fused program -> CUDA C -> sm_100a cubin (NVRTC).

The reference emits sm_52 PTX text for a chain of f32 ops and launches it 1-D with 256 threads,
one element per thread (ferrotorch-jit/src/fusion.rs ``generate_ptx_named``; fusion_gpu.rs:79-269;
codegen_gpu.rs).  Here a fused *DAG* of the same op set becomes one kernel that

* loads every external input once with 128-bit vectors (8 bf16 / fp16 or 4 fp32 elements per
  thread and step), grid-stride, fp32 math, one vector store;
* broadcasts scalar inputs and row vectors (``[N]`` against ``[..., N]``);
* is compiled by NVRTC for ``sm_100a`` and cached by (program, dtypes, broadcast kinds, vector
  width); launched through the driver API on the current torch stream.

``eval_elementwise`` / ``run_program_torch`` are the CPU (and oracle) path of the same programs.
"""
from __future__ import annotations

import hashlib
import math

import torch

from .. import _native

_UNARY_C = {
    "neg": "-({a})", "relu": "fmaxf({a}, 0.f)", "sigmoid": "__fdividef(1.f, 1.f + __expf(-({a})))",
    # tanh as 1 - 2 / (1 + e^2x): absolute error about 1e-7, a fraction of the cost of tanhf
    "tanh": "(1.f - __fdividef(2.f, 1.f + __expf(2.f * ({a}))))",
    "gelu": "0.5f * ({a}) * (1.f + erff(({a}) * 0.70710678118654752f))", "silu": "__fdividef({a}, 1.f + __expf(-({a})))",
    "sqrt": "sqrtf({a})", "abs": "fabsf({a})", "exp": "__expf({a})", "log": "__logf({a})",
}
_BINARY_C = {"add": "({a}) + ({b})", "sub": "({a}) - ({b})", "mul": "({a}) * ({b})", "div": "({a}) / ({b})"}
_SCALAR_C = {"add_c": "({a}) + {c}", "mul_c": "({a}) * {c}", "pow_c": "powf({a}, {c})", "rsub_c": "{c} - ({a})",
             "rdiv_c": "{c} / ({a})"}
_CTYPE = {torch.float32: "float", torch.bfloat16: "__nv_bfloat16", torch.float16: "__half"}


def eval_elementwise(op: str, xs, c=None):
    a = xs[0]
    if op in _BINARY_C:
        return {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}[op](a, xs[1])
    if op == "add_c":
        return a + c
    if op == "mul_c":
        return a * c
    if op == "pow_c":
        return a ** c
    if op == "rsub_c":
        return c - a
    if op == "rdiv_c":
        return c / a
    return {"neg": torch.neg, "relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
            "gelu": torch.nn.functional.gelu, "silu": torch.nn.functional.silu, "sqrt": torch.sqrt, "abs": torch.abs,
            "exp": torch.exp, "log": torch.log}[op](a)


def run_program_torch(program, inputs):
    """Reference execution of a fused program with torch ops (fp32 math, like the kernel)."""
    dt = inputs[0].dtype if inputs else torch.float32
    regs = []
    for ins in program:
        xs = [regs[i] if kind == "r" else inputs[i].float() for kind, i in ins["src"]]
        regs.append(eval_elementwise(ins["op"], xs, ins.get("c")))
    return regs[-1].to(dt)


def _cfloat(c) -> str:
    c = float(c)
    if math.isinf(c):
        return "INFINITY" if c > 0 else "-INFINITY"
    return repr(c) + "f" if "." in repr(c) or "e" in repr(c) or "n" in repr(c) else repr(c) + ".f"


def generate_source(program, in_dtypes, in_kinds, out_dtype, vec: int, name: str = "fused_kernel") -> str:
    """CUDA C for one fused program.  ``in_kinds[i]``: "full" | "scalar" | "row"."""
    args = ", ".join("const %s* __restrict__ x%d" % (_CTYPE[d], i) for i, d in enumerate(in_dtypes))
    lines = ["#include <cuda_bf16.h>", "#include <cuda_fp16.h>",
             "__device__ __forceinline__ float ld(const float* p, long long i) { return p[i]; }",
             "__device__ __forceinline__ float ld(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }",
             "__device__ __forceinline__ float ld(const __half* p, long long i) { return __half2float(p[i]); }",
             "__device__ __forceinline__ void st(float* p, long long i, float v) { p[i] = v; }",
             "__device__ __forceinline__ void st(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }",
             "__device__ __forceinline__ void st(__half* p, long long i, float v) { p[i] = __float2half(v); }",
             "template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T v[V]; };",
             'extern "C" __global__ void __launch_bounds__(256) %s(%s%s%s* __restrict__ out, long long n, long long row) {'
             % (name, args, ", " if args else "", _CTYPE[out_dtype]),
             "  constexpr int V = %d;" % vec,
             "  const long long nv = n / V;",
             "  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {"]
    for k, (d, kind) in enumerate(zip(in_dtypes, in_kinds)):
        ct = _CTYPE[d]
        if kind == "full":
            lines.append("    const Vec<%s, V> a%d = reinterpret_cast<const Vec<%s, V>*>(x%d)[i];" % (ct, k, ct, k))
        elif kind == "scalar":
            lines.append("    const float s%d = ld(x%d, 0);" % (k, k))
    lines.append("    Vec<%s, V> o;" % _CTYPE[out_dtype])
    lines.append("#pragma unroll")
    lines.append("    for (int j = 0; j < V; ++j) {")
    for k, kind in enumerate(in_kinds):
        if kind == "full":
            lines.append("      const float e%d = ld(a%d.v, j);" % (k, k))
        elif kind == "scalar":
            lines.append("      const float e%d = s%d;" % (k, k))
        else:
            lines.append("      const float e%d = ld(x%d, (i * V + j) %% row);" % (k, k))
    for r, ins in enumerate(program):
        ops = ["r%d" % i if kind == "r" else "e%d" % i for kind, i in ins["src"]]
        op = ins["op"]
        if op in _UNARY_C:
            expr = _UNARY_C[op].format(a=ops[0])
        elif op in _BINARY_C:
            expr = _BINARY_C[op].format(a=ops[0], b=ops[1])
        else:
            expr = _SCALAR_C[op].format(a=ops[0], c=_cfloat(ins["c"]))
        lines.append("      const float r%d = %s;" % (r, expr))
    lines.append("      st(o.v, j, r%d);" % (len(program) - 1))
    lines.append("    }")
    lines.append("    reinterpret_cast<Vec<%s, V>*>(out)[i] = o;" % _CTYPE[out_dtype])
    lines.append("  }")
    lines.append("}")
    return "\n".join(lines)


_cache: dict[str, object] = {}
compile_count = 0


def compile_cubin(source: str, name: str) -> bytes:
    """NVRTC -> sm_100a cubin.  Needs no GPU."""
    from cuda.bindings import nvrtc

    import os

    inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    err, prog = nvrtc.nvrtcCreateProgram(source.encode(), (name + ".cu").encode(), 0, [], [])
    opts = [b"--gpu-architecture=sm_100a", b"--std=c++17", b"-lineinfo", ("-I" + inc).encode()]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if err != nvrtc.nvrtcResult.NVRTC_SUCCESS:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC failed:\n%s\n%s" % (log.decode(errors="replace"), source))
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * n
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    nvrtc.nvrtcDestroyProgram(prog)
    return cubin


class CompiledKernel:
    def __init__(self, cubin: bytes, name: str):
        from cuda.bindings import driver

        err, self.module = driver.cuModuleLoadData(cubin)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError("cuModuleLoadData failed: %s" % err)
        err, self.fn = driver.cuModuleGetFunction(self.module, name.encode())
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError("cuModuleGetFunction failed: %s" % err)

    n_inputs: int | None = None        # set by the generator that built the kernel, when it knows

    def num_inputs(self) -> int | None:
        return self.n_inputs

    @staticmethod
    def output_len(*inputs: torch.Tensor) -> int:
        """Elements of the output for these operands: the broadcast of their shapes."""
        n = 1
        for d in torch.broadcast_shapes(*[t.shape for t in inputs]):
            n *= int(d)
        return n

    def execute(self, inputs, out: torch.Tensor | None = None, block: int = 256) -> torch.Tensor:
        """Launch over contiguous device operands of the output's shape (one row of ``row = 1`` columns)."""
        shape = torch.broadcast_shapes(*[t.shape for t in inputs])
        xs = [t.expand(shape).contiguous() for t in inputs]
        out = out if out is not None else torch.empty(shape, dtype=xs[0].dtype, device=xs[0].device)
        n = out.numel()
        self.launch([t.data_ptr() for t in xs] + [out.data_ptr()], n, 1, max(1, (n + block - 1) // block), block,
                    torch.cuda.current_stream(out.device).cuda_stream)
        return out

    def launch(self, ptrs, n: int, row: int, grid: int, block: int, stream: int) -> None:
        import ctypes

        from cuda.bindings import driver

        vals = tuple(ptrs) + (n, row)
        types = tuple([ctypes.c_void_p] * len(ptrs) + [ctypes.c_longlong, ctypes.c_longlong])
        (err,) = driver.cuLaunchKernel(self.fn, grid, 1, 1, block, 1, 1, 0, stream, (vals, types), 0)
        if err != driver.CUresult.CUDA_SUCCESS:
            raise RuntimeError("cuLaunchKernel failed: %s" % err)
        _native.kernels().ft_count_external_launch(1)


def _kind(t: torch.Tensor, out_shape) -> str | None:
    if t.numel() == 1:
        return "scalar"
    if tuple(t.shape) == tuple(out_shape) and t.is_contiguous():
        return "full"
    if t.dim() == 1 and len(out_shape) >= 1 and t.shape[0] == out_shape[-1] and t.is_contiguous():
        return "row"
    return None


def run_fused(program, inputs, out_shape, block: int = 256) -> torch.Tensor:
    """Execute a fused program: generated kernel on CUDA tensors, torch ops elsewhere."""
    global compile_count
    out_dtype = next((t.dtype for t in inputs if t.numel() > 1), inputs[0].dtype if inputs else torch.float32)
    on_gpu = all(t.is_cuda for t in inputs) and inputs and out_dtype in _CTYPE
    kinds = [_kind(t, out_shape) for t in inputs] if on_gpu else None
    if not on_gpu or any(k is None for k in kinds) or any(t.dtype not in _CTYPE for t in inputs):
        shaped = [t for t in inputs]
        return run_program_torch(program, shaped).expand(out_shape).contiguous() if inputs else None
    out = torch.empty(out_shape, device=inputs[0].device, dtype=out_dtype)
    n = out.numel()
    if n == 0:
        return out
    width = 16 // max(t.element_size() for t in list(inputs) + [out])
    aligned = all(t.data_ptr() % 16 == 0 for t in inputs if t.numel() > 1) and out.data_ptr() % 16 == 0
    vec = width if (n % width == 0 and aligned) else 1
    key = hashlib.sha1(repr((program, [str(t.dtype) for t in inputs], kinds, str(out_dtype), vec)).encode()).hexdigest()
    kern = _cache.get(key)
    if kern is None:
        name = "fused_" + key[:12]
        src = generate_source(program, [t.dtype for t in inputs], kinds, out_dtype, vec, name)
        kern = CompiledKernel(compile_cubin(src, name), name)
        _cache[key] = kern
        compile_count += 1
    nv = n // vec
    grid = max(1, min((nv + block - 1) // block, 148 * 8))
    row = out_shape[-1] if len(out_shape) else 1
    kern.launch([t.data_ptr() for t in inputs] + [out.data_ptr()], n, row, grid, block,
                torch.cuda.current_stream().cuda_stream)
    return out
