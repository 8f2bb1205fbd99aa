"""Execution back-ends for an optimised IR graph and the loop-level IR under the code generator
(ferrotorch-jit/src/codegen.rs: ``Codegen`` / ``InterpreterBackend`` / ``NativeBackend`` /
``InductorBackend``; codegen_ir.rs: ``Expr`` / ``LoopIR``; interpreter.rs; fusion.rs:
``FusedOp`` / ``FusedChain`` / ``ReductionKind``; memory_plan.rs).

* :func:`interpret` / :func:`interpret_multi` walk the graph node by node.
* :class:`NativeBackend` resolves every node to a closure once, so a call is a flat list of
  Python calls without any dispatch on op names.
* :class:`InductorBackend` lowers every fused elementwise group to :class:`LoopIR` and from there
  to source text: CUDA C for sm_100a (``InductorTarget.GpuCuda``; compiled by NVRTC the first
  time the group runs on a device) or Python over torch scalars-as-tensors
  (``InductorTarget.CpuTorch``; what the CPU tests execute).  Reductions over the last axis have
  their own generator (:func:`generate_reduction_source`).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

import torch

from . import codegen
from .ir import IrGraph, plan_memory
from .module import CompileConfig, JitError, TracedModule, _call_node, _interpret, compile as _compile
from . import module as _module


# --------------------------------------------------------------------------- interpreter
def interpret_multi(graph: IrGraph, inputs) -> list:
    """All outputs of the graph, in ``graph.outputs`` order."""
    env = _interpret(graph, list(inputs))
    return [env[i] for i in graph.outputs]


def interpret(graph: IrGraph, inputs):
    """The single output of a single-output graph."""
    outs = interpret_multi(graph, inputs)
    if len(outs) != 1:
        raise JitError("interpret: the graph has %d outputs; use interpret_multi" % len(outs))
    return outs[0]


def interpret_multi_with_captures(graph: IrGraph, inputs, capture_ids) -> tuple:
    """Outputs plus the values of the listed intermediate nodes (used by the AOT backward split)."""
    env = _interpret(graph, list(inputs))
    return [env[i] for i in graph.outputs], [env[i] for i in capture_ids]


def is_fusion_enabled() -> bool:
    return _module._fusion_enabled


def compile_with_config(fn, example_inputs, config: CompileConfig):
    return _compile(fn, example_inputs, config)


def estimate_numel_for_inputs(shapes) -> int:
    """Element count of the broadcast of ``shapes`` (what one fused launch has to cover)."""
    out = torch.broadcast_shapes(*[tuple(s) for s in shapes]) if shapes else ()
    n = 1
    for d in out:
        n *= int(d)
    return n


@dataclass
class MemoryPlan:
    slot_of: dict
    n_slots: int
    peak_bytes: int

    naive_bytes: int = 0

    @classmethod
    def of(cls, graph: IrGraph) -> "MemoryPlan":
        naive = 0
        for i in graph.order:
            n = graph.nodes[i]
            if n.op not in ("input", "const") and n.shape is not None:
                numel = 1
                for d in n.shape:
                    numel *= int(d)
                naive += numel * torch.empty(0, dtype=n.dtype or torch.float32).element_size()
        return cls(**plan_memory(graph), naive_bytes=naive)

    def reuse_count(self) -> int:
        return len(self.slot_of) - self.n_slots

    def savings_percent(self) -> float:
        """How much smaller the planned peak is than one buffer per intermediate value, in percent."""
        return 100.0 * (1.0 - self.peak_bytes / self.naive_bytes) if self.naive_bytes else 0.0


# --------------------------------------------------------------------------- loop IR
class UnaryOpKind(enum.Enum):
    Neg = "neg"; Relu = "relu"; Sigmoid = "sigmoid"; Tanh = "tanh"; Gelu = "gelu"; Silu = "silu"  # noqa: E702
    Sqrt = "sqrt"; Abs = "abs"; Exp = "exp"; Log = "log"  # noqa: E702


class BinOpKind(enum.Enum):
    Add = "add"; Sub = "sub"; Mul = "mul"; Div = "div"; Pow = "pow"  # noqa: E702


@dataclass(frozen=True)
class Expr:
    """``kind``: "load" (input ``index``), "const" (``value``), "unary" (``op``, one arg), "binary" (``op``, two args)."""
    kind: str
    op: object = None
    args: tuple = ()
    index: int = -1
    value: float = 0.0

    @staticmethod
    def load(index: int) -> "Expr":
        return Expr("load", index=index)

    @staticmethod
    def const(value: float) -> "Expr":
        return Expr("const", value=float(value))

    @staticmethod
    def unary(op: UnaryOpKind, a: "Expr") -> "Expr":
        return Expr("unary", op, (a,))

    @staticmethod
    def binary(op: BinOpKind, a: "Expr", b: "Expr") -> "Expr":
        return Expr("binary", op, (a, b))

    # the reference's constructor names (ferrotorch-jit/src/codegen_ir.rs ``impl Expr``)
    @staticmethod
    def var(index: int) -> "Expr":
        return Expr.load(index)

    @staticmethod
    def constant(value: float) -> "Expr":
        return Expr.const(value)

    @staticmethod
    def int(value) -> "Expr":
        return Expr.const(float(value))

    @staticmethod
    def bin(op, a: "Expr", b: "Expr") -> "Expr":
        return Expr.binary(op if isinstance(op, BinOpKind) else BinOpKind(op), a, b)

    @staticmethod
    def call(fn, a: "Expr") -> "Expr":
        """A unary function by kind or by name (``"exp"``, ``"relu"`` ...)."""
        return Expr.unary(fn if isinstance(fn, UnaryOpKind) else UnaryOpKind(fn), a)

    @staticmethod
    def sum(terms) -> "Expr":
        terms = list(terms)
        out = terms[0] if terms else Expr.const(0.0)
        for t in terms[1:]:
            out = Expr.binary(BinOpKind.Add, out, t)
        return out

    @staticmethod
    def prod(terms) -> "Expr":
        terms = list(terms)
        out = terms[0] if terms else Expr.const(1.0)
        for t in terms[1:]:
            out = Expr.binary(BinOpKind.Mul, out, t)
        return out

    def depth(self) -> int:
        return 1 + max((a.depth() for a in self.args), default=0)

    def loads(self) -> set:
        return {self.index} if self.kind == "load" else set().union(*[a.loads() for a in self.args]) if self.args else set()


@dataclass
class LoopIR:
    """One parallel loop ``for i in range(numel): out[i] = body`` over ``n_inputs`` operands."""
    n_inputs: int
    body: Expr

    @classmethod
    def from_program(cls, program, n_inputs: int) -> "LoopIR":
        """Lower a fused program (the IR node's register machine) to one expression tree."""
        regs: list[Expr] = []
        for ins in program:
            src = [Expr.load(i) if kind == "x" else regs[i] for kind, i in ins["src"]]
            op, c = ins["op"], ins.get("c")
            if op in ("add", "sub", "mul", "div"):
                e = Expr.binary(BinOpKind(op), src[0], src[1])
            elif op == "add_c":
                e = Expr.binary(BinOpKind.Add, src[0], Expr.const(c))
            elif op == "mul_c":
                e = Expr.binary(BinOpKind.Mul, src[0], Expr.const(c))
            elif op == "pow_c":
                e = Expr.binary(BinOpKind.Pow, src[0], Expr.const(c))
            elif op == "rsub_c":
                e = Expr.binary(BinOpKind.Sub, Expr.const(c), src[0])
            elif op == "rdiv_c":
                e = Expr.binary(BinOpKind.Div, Expr.const(c), src[0])
            else:
                e = Expr.unary(UnaryOpKind(op), src[0])
            regs.append(e)
        return cls(n_inputs, regs[-1])


_PY_UNARY = {"neg": "(-{a})", "relu": "torch.relu({a})", "sigmoid": "torch.sigmoid({a})", "tanh": "torch.tanh({a})",
             "gelu": "torch.nn.functional.gelu({a})", "silu": "torch.nn.functional.silu({a})", "sqrt": "torch.sqrt({a})",
             "abs": "torch.abs({a})", "exp": "torch.exp({a})", "log": "torch.log({a})"}
_BIN_SYM = {"add": "+", "sub": "-", "mul": "*", "div": "/"}


class CpuCodegen:
    """LoopIR -> Python source over torch tensors (the loop is the tensor op)."""

    def expr(self, e: Expr) -> str:
        if e.kind == "load":
            return "x%d" % e.index
        if e.kind == "const":
            return repr(e.value)
        if e.kind == "unary":
            return _PY_UNARY[e.op.value].format(a=self.expr(e.args[0]))
        a, b = self.expr(e.args[0]), self.expr(e.args[1])
        return "(%s ** %s)" % (a, b) if e.op is BinOpKind.Pow else "(%s %s %s)" % (a, _BIN_SYM[e.op.value], b)

    def generate(self, ir: LoopIR, name: str = "fused") -> str:
        args = ", ".join("x%d" % i for i in range(ir.n_inputs))
        return "def %s(%s):\n    return %s\n" % (name, args, self.expr(ir.body))

    def compile(self, ir: LoopIR, name: str = "fused"):
        scope = {"torch": torch}
        exec(self.generate(ir, name), scope)  # noqa: S102 - source generated here from a closed op set
        return scope[name]


class GpuCodegen:
    """LoopIR -> CUDA C for sm_100a: fp32 math, one element per thread and grid-stride step.  The
    vectorised, broadcast-aware kernels that actually run come from ``codegen.generate_source``;
    this generator is the plain form of the same loop, kept for inspection and as a second oracle."""

    _UNARY = codegen._UNARY_C

    def expr(self, e: Expr) -> str:
        if e.kind == "load":
            return "v%d" % e.index
        if e.kind == "const":
            return codegen._cfloat(e.value)
        if e.kind == "unary":
            return "(" + self._UNARY[e.op.value].format(a=self.expr(e.args[0])) + ")"
        a, b = self.expr(e.args[0]), self.expr(e.args[1])
        return "powf(%s, %s)" % (a, b) if e.op is BinOpKind.Pow else "(%s %s %s)" % (a, _BIN_SYM[e.op.value], b)

    def generate(self, ir: LoopIR, name: str = "fused_loop") -> str:
        params = ", ".join("const float* __restrict__ x%d" % i for i in range(ir.n_inputs))
        loads = "".join("    const float v%d = x%d[i];\n" % (i, i) for i in sorted(ir.body.loads()))
        return ('extern "C" __global__ void %s(%s%sfloat* __restrict__ out, long long n) {\n'
                "  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {\n"
                "%s    out[i] = %s;\n  }\n}\n") % (name, params, ", " if params else "", loads, self.expr(ir.body))


# --------------------------------------------------------------------------- fused chains, reductions
class FusedOp(enum.Enum):
    """The unary / scalar ops a fused chain may hold (fusion.rs:112)."""
    Neg = "neg"; Relu = "relu"; Sigmoid = "sigmoid"; Tanh = "tanh"; Gelu = "gelu"; Silu = "silu"  # noqa: E702
    Sqrt = "sqrt"; Abs = "abs"; Exp = "exp"; Log = "log"  # noqa: E702
    AddScalar = "add_c"; MulScalar = "mul_c"; PowScalar = "pow_c"  # noqa: E702


@dataclass
class FusedChain:
    """A straight chain of unary / scalar ops applied to one tensor in one kernel."""
    ops: list = field(default_factory=list)     # FusedOp or (FusedOp, scalar)

    def push(self, op: FusedOp, scalar: float | None = None) -> "FusedChain":
        needs = op.value.endswith("_c")
        if needs != (scalar is not None):
            raise JitError("FusedChain: %s %s a scalar" % (op.name, "needs" if needs else "does not take"))
        self.ops.append((op, scalar) if needs else op)
        return self

    def __len__(self) -> int:
        return len(self.ops)

    def _plain(self) -> list:
        return [(o[0].value, o[1]) if isinstance(o, tuple) else o.value for o in self.ops]

    def program(self) -> list:
        return [{"op": (o if isinstance(o, str) else o[0]), "src": [("x", 0)] if k == 0 else [("r", k - 1)],
                 "c": None if isinstance(o, str) else o[1]} for k, o in enumerate(self._plain())]

    def loop_ir(self) -> LoopIR:
        return LoopIR.from_program(self.program(), 1)

    def execute(self, x: torch.Tensor) -> torch.Tensor:
        return _module.apply_fused(self._plain(), x)

    def generate_source(self, dtype: torch.dtype = torch.float32, vec: int = 4) -> str:
        return codegen.generate_source(self.program(), [dtype], ["full"], dtype, vec)

    # the reference's names (fusion.rs ``impl FusedChain``).  Its device code is PTX text and its host code
    # Rust text; here both generators emit what this package compiles: CUDA C for sm_100a and a Python
    # function over torch ops.
    def len(self) -> int:
        return len(self.ops)

    def is_empty(self) -> bool:
        return not self.ops

    def execute_cpu(self, x: torch.Tensor) -> torch.Tensor:
        return CpuCodegen().compile(self.loop_ir(), "fused_chain")(x.detach().cpu())

    def generate_ptx(self) -> str:
        return self.generate_source(torch.float32)

    def generate_ptx_named(self, name: str) -> str:
        return GpuCodegen().generate(self.loop_ir(), name)

    def generate_ptx_f64_named(self, name: str) -> str:
        return GpuCodegen().generate(self.loop_ir(), name).replace("float", "double")

    def generate_rust(self) -> str:
        return CpuCodegen().generate(self.loop_ir(), "fused_chain")


CpuCodegen.generate_rust_source = CpuCodegen.generate        # the host generator's output (Python over torch ops here)
GpuCodegen.generate_ptx_source = GpuCodegen.generate         # the device generator's output (CUDA C for sm_100a here)


class ReductionKind(enum.Enum):
    Sum = "sum"; Mean = "mean"; Max = "max"; Min = "min"; Prod = "prod"  # noqa: E702


_RED = {ReductionKind.Sum: ("0.f", "a + b"), ReductionKind.Mean: ("0.f", "a + b"), ReductionKind.Prod: ("1.f", "a * b"),
        ReductionKind.Max: ("__int_as_float(0xff800000)", "fmaxf(a, b)"),
        ReductionKind.Min: ("__int_as_float(0x7f800000)", "fminf(a, b)")}


def generate_reduction_source(kind: ReductionKind, pre: FusedChain | None = None, name: str = "fused_reduce") -> str:
    """CUDA C for ``out[row] = reduce(pre(x[row, :]))`` over the last axis: one warp per row,
    lanes stride the row, a shuffle tree combines them (the reference's
    ``generate_reduction_ptx`` emits the block-per-row PTX equivalent, fusion.rs)."""
    init, comb = _RED[kind]
    body = GpuCodegen().expr(pre.loop_ir().body) if pre is not None and len(pre) else "v0"
    return ('extern "C" __global__ void %s(const float* __restrict__ x, float* __restrict__ out, long long rows, int cols) {\n'
            "  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;\n"
            "  const int lane = threadIdx.x & 31;\n"
            "  if (row >= rows) return;\n"
            "  float acc = %s;\n"
            "  for (int c = lane; c < cols; c += 32) {\n"
            "    const float v0 = x[row * cols + c];\n"
            "    const float a = acc, b = %s;\n"
            "    acc = %s;\n  }\n"
            "  for (int s = 16; s > 0; s >>= 1) {\n"
            "    const float a = acc, b = __shfl_xor_sync(0xffffffffu, acc, s);\n"
            "    acc = %s;\n  }\n"
            "  if (lane == 0) out[row] = acc%s;\n}\n") % (name, init, body, comb, comb,
                                                       " / (float)cols" if kind is ReductionKind.Mean else "")


def reduce_reference(kind: ReductionKind, x: torch.Tensor, pre: FusedChain | None = None) -> torch.Tensor:
    """What the generated reduction computes, with torch ops."""
    if pre is not None and len(pre):
        x = codegen.run_program_torch(pre.program(), [x])
    return {ReductionKind.Sum: lambda t: t.sum(-1), ReductionKind.Mean: lambda t: t.mean(-1),
            ReductionKind.Prod: lambda t: t.prod(-1), ReductionKind.Max: lambda t: t.amax(-1),
            ReductionKind.Min: lambda t: t.amin(-1)}[kind](x)


# --------------------------------------------------------------------------- graph back-ends
class CompiledGraph:
    """A graph bound to a way of running it: ``execute(inputs) -> list of outputs``."""

    def __init__(self, graph: IrGraph, steps, backend: str, sources: dict | None = None):
        self.graph, self._steps, self.backend, self.sources = graph, steps, backend, sources or {}

    def execute(self, inputs) -> list:
        env: dict = {}
        for node_id, fn in self._steps:
            env[node_id] = fn(env, inputs)
        return [env[i] for i in self.graph.outputs]

    def __call__(self, inputs) -> list:
        return self.execute(inputs)

    def num_inputs(self) -> int:
        return self.graph.count("input")

    def output_shape(self):
        n = self.graph.nodes[self.graph.outputs[0]]
        return tuple(n.shape) if n.shape is not None else None


class Codegen:
    """Back-end protocol: ``compile(graph) -> CompiledGraph``."""
    name = "abstract"

    def compile(self, graph: IrGraph) -> CompiledGraph:
        raise NotImplementedError


class InterpreterBackend(Codegen):
    name = "interpreter"

    def compile(self, graph: IrGraph) -> CompiledGraph:
        class _Whole(CompiledGraph):
            def execute(self, inputs):
                return interpret_multi(self.graph, inputs)

        return _Whole(graph, [], self.name)


def _node_closure(graph: IrGraph, n, fused_runner):
    ins = tuple(n.inputs)
    if n.op == "input":
        idx = n.attrs["index"]
        return lambda env, inputs: inputs[idx]
    if n.op == "const":
        val = n.attrs["value"]
        return lambda env, inputs: val
    if n.op == "call":
        return lambda env, inputs: _call_node(n, env)
    if n.op == "fused_elementwise":
        return fused_runner(n)
    if n.op in ("fused_linear_act", "fused_attention"):
        return lambda env, inputs: _interpret_one(graph, n, env)
    if n.op in _module.ELEMENTWISE:
        op, c = n.op, n.attrs.get("c")
        return lambda env, inputs: codegen.eval_elementwise(op, [env[j] for j in ins], c)
    raise JitError("unknown IR op %s" % n.op)


def _interpret_one(graph: IrGraph, n, env):
    """Evaluate one node with the interpreter's semantics given its inputs in ``env``."""
    seeded = IrGraph()                                          # the inputs enter as constants
    for j in n.inputs:
        seeded.nodes[j] = type(n)(j, "const", [], {"value": env[j]})
        seeded.order.append(j)
    seeded.nodes[n.id] = n
    seeded.order.append(n.id)
    return _interpret(seeded, [])[n.id]


class NativeBackend(Codegen):
    """Every node resolved to a closure ahead of time; fused groups run the generated kernels on
    CUDA tensors and the torch program elsewhere (``codegen.run_fused`` decides)."""
    name = "native"

    def compile(self, graph: IrGraph) -> CompiledGraph:
        def fused(n):
            ins, prog, shape = tuple(n.inputs), n.attrs["program"], n.shape

            def run(env, inputs):
                xs = [env[j] for j in ins]
                return codegen.run_fused(prog, xs, tuple(shape) if shape is not None
                                         else tuple(torch.broadcast_shapes(*[t.shape for t in xs])))
            return run

        return CompiledGraph(graph, [(i, _node_closure(graph, graph.nodes[i], fused)) for i in graph.order], self.name)


class InductorTarget(enum.Enum):
    CpuTorch = "cpu"
    GpuCuda = "cuda"


class InductorCompileStatus(enum.Enum):
    Compiled = "compiled"            # every fused group went through LoopIR -> source
    Partial = "partial"              # some groups were left to the native runner
    Interpreted = "interpreted"      # nothing to generate

    def is_compiled(self) -> bool:
        return self is InductorCompileStatus.Compiled

    def is_fallback(self) -> bool:
        return self is not InductorCompileStatus.Compiled


@dataclass
class InductorCompileOutcome:
    """What ``InductorBackend.compile_with_status`` returns: the runnable graph and how much of it went
    through generated source (codegen.rs ``InductorCompileStatus::{Compiled, Fallback}``)."""
    status: InductorCompileStatus
    graph: "CompiledGraph"
    reason: str = ""

    def is_compiled(self) -> bool:
        return self.status.is_compiled()

    def is_fallback(self) -> bool:
        return self.status.is_fallback()

    def compiled_graph(self) -> "CompiledGraph":
        return self.graph

    into_compiled_graph = compiled_graph


class InductorBackend(Codegen):
    """Fused groups -> :class:`LoopIR` -> source for the target; the rest of the graph as in
    :class:`NativeBackend`.  ``sources`` of the result maps node id -> generated text."""
    name = "inductor"

    def __init__(self, target: InductorTarget = InductorTarget.CpuTorch):
        self.target, self.status = target, InductorCompileStatus.Interpreted

    def compile(self, graph: IrGraph) -> CompiledGraph:
        sources, done, total = {}, 0, 0

        def fused(n):
            nonlocal done, total
            total += 1
            ins, prog, shape = tuple(n.inputs), n.attrs["program"], n.shape
            ir = LoopIR.from_program(prog, len(ins))
            if self.target is InductorTarget.CpuTorch:
                sources[n.id] = CpuCodegen().generate(ir, "fused_%d" % n.id)
                fn = CpuCodegen().compile(ir, "fused_%d" % n.id)
                done += 1
                return lambda env, inputs: fn(*[env[j] for j in ins])
            sources[n.id] = GpuCodegen().generate(ir, "fused_%d" % n.id)
            done += 1

            def run(env, inputs):                                # the vectorised kernel of the same program
                xs = [env[j] for j in ins]
                return codegen.run_fused(prog, xs, tuple(shape) if shape is not None
                                         else tuple(torch.broadcast_shapes(*[t.shape for t in xs])))
            return run

        steps = [(i, _node_closure(graph, graph.nodes[i], fused)) for i in graph.order]
        self.status = (InductorCompileStatus.Interpreted if total == 0 else
                       InductorCompileStatus.Compiled if done == total else InductorCompileStatus.Partial)
        return CompiledGraph(graph, steps, self.name, sources)

    def with_block_size(self, block_size: int) -> "InductorBackend":
        self.block_size = int(block_size)
        return self

    def compile_with_status(self, graph: IrGraph) -> "InductorCompileOutcome":
        compiled = self.compile(graph)
        reason = {InductorCompileStatus.Compiled: "", InductorCompileStatus.Partial: "some fused groups run through the native runner",
                  InductorCompileStatus.Interpreted: "the graph has no fused group to generate code for"}[self.status]
        return InductorCompileOutcome(self.status, compiled, reason)

    def generate(self, graph: IrGraph) -> dict:
        """Generated source per fused node, without keeping the runnable graph."""
        return dict(self.compile(graph).sources)


def compile_loop_ir_kernel(ir: LoopIR, name: str = "fused_loop"):
    """LoopIR -> (source, cubin bytes) for sm_100a through NVRTC (codegen_jit.rs ``compile_loop_ir_kernel``)."""
    src = GpuCodegen().generate(ir, name)
    return src, codegen.compile_cubin(src, name)


# --------------------------------------------------------------------------- remaining names of the reference's JIT
from . import advanced as _adv  # noqa: E402

AotCompiledModule = _adv.AotModule
TraceResult = _adv.SegmentedModule            # what ``trace_with_breaks`` returns
JitCompiledKernel = codegen.CompiledKernel


def export_with_dynamic_shapes(module, example_inputs, dynamic_dims: dict):
    """``export`` with ``{input index: {dim index: name}}`` naming the dimensions that may vary."""
    specs = []
    for i, t in enumerate(example_inputs):
        names = dynamic_dims.get(i, {})
        specs.append(_adv.InputSpec([_adv.DimSpec.dynamic(names[d]) if d in names else _adv.DimSpec.static(int(s))
                                     for d, s in enumerate(t.shape)]))
    return _adv.export(module, example_inputs, specs)


def estimate_matmul_dims(shapes) -> tuple:
    """``(M, N, K)`` of ``a @ b`` for operand shapes ``[..., M, K]`` and ``[..., K, N]`` (batch folded into M)."""
    a, b = tuple(shapes[0]), tuple(shapes[1])
    if len(a) < 2 or len(b) < 2 or a[-1] != b[-2]:
        raise JitError("estimate_matmul_dims: %s @ %s" % (a, b))
    m = a[-2]
    for d in a[:-2]:
        m *= d
    return int(m), int(b[-1]), int(a[-1])


class FusionGroupKind(enum.Enum):
    Elementwise = "fused_elementwise"
    LinearActivation = "fused_linear_act"
    Attention = "fused_attention"


@dataclass
class FusionGroup:
    """One fused node of an optimised graph: its kind, the node id, how many primitive ops it absorbed."""
    kind: FusionGroupKind
    node_id: int
    n_ops: int

    @classmethod
    def of(cls, graph: IrGraph) -> list:
        out = []
        for i in graph.order:
            n = graph.nodes[i]
            if n.op in (k.value for k in FusionGroupKind):
                out.append(cls(FusionGroupKind(n.op), i, len(n.attrs.get("program", ())) or 2))
        return out


@dataclass(frozen=True)
class AutotuneKey:
    """What a tuning result is valid for: the graph's op sequence and the input signature."""
    ops: tuple
    signature: tuple

    @classmethod
    def of(cls, module: TracedModule) -> "AutotuneKey":
        return cls(tuple(module.graph.ops()), tuple(module.guard))

    @classmethod
    def from_graph(cls, graph: IrGraph, inputs=()) -> "AutotuneKey":
        return cls(tuple(graph.ops()) + (graph.fingerprint(),), tuple((tuple(t.shape), t.dtype) for t in inputs))


@dataclass
class AutotuneCandidate:
    block_size: int
    ms: float = float("nan")

    @property
    def name(self) -> str:
        return "block_size=%d" % self.block_size


@dataclass
class AutotuneResult:
    key: AutotuneKey
    best: AutotuneCandidate
    candidates: list

    def winner_name(self) -> str:
        return self.best.name

    def winner_time(self) -> float:
        """Seconds per call of the winner (NaN when nothing was timed)."""
        return self.best.ms * 1e-3

    def winner_compiled(self):
        """Block-size tuning changes the module in place; there is no separate compiled object."""
        return None

    def all_timings(self) -> list:
        return [(c.name, c.ms * 1e-3) for c in self.candidates]


@dataclass
class BackendTuneResult:
    """What ``Autotuner.tune(graph, inputs)`` found: the winning back-end, its median time in seconds,
    every ``(name, median)`` that was timed (only the winner's on a cache hit), the winner's compiled
    graph, and the candidates that could not compile the graph (autotune.rs ``AutotuneResult``)."""
    winner: str
    median_s: float
    all_timings: list
    compiled: "CompiledGraph"
    from_cache: bool = False
    failed: dict = field(default_factory=dict)

    def winner_name(self) -> str:
        return self.winner

    def winner_time(self) -> float:
        return self.median_s

    def winner_compiled(self) -> "CompiledGraph":
        return self.compiled


def autotune(module: TracedModule, inputs, candidates=(128, 256, 512), iters: int = 5, cache: dict | None = None) -> AutotuneResult:
    """Time every candidate block size (CUDA events; on the CPU nothing is timed and the module's
    current block size stands) and keep the best; ``cache`` (key -> result) skips repeated tuning."""
    key = AutotuneKey.of(module)
    if cache is not None and key in cache:
        module.cfg.block_size = cache[key].best.block_size
        return cache[key]
    cands = []
    if torch.cuda.is_available() and any(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs):
        for b in candidates:
            module.cfg.block_size = b
            module(*inputs)
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                module(*inputs)
            e.record()
            torch.cuda.synchronize()
            cands.append(AutotuneCandidate(b, s.elapsed_time(e) / iters))
        best = min(cands, key=lambda c: c.ms)
    else:
        best = AutotuneCandidate(module.cfg.block_size)
        cands = [best]
    module.cfg.block_size = best.block_size
    res = AutotuneResult(key, best, cands)
    if cache is not None:
        cache[key] = res
    return res


def generate_reduction_ptx(kind: ReductionKind, pre: FusedChain | None = None, name: str = "fused_reduce") -> str:
    """The reference emits PTX text here; this build's generated kernels are CUDA C compiled for
    sm_100a by NVRTC, so this returns that source (:func:`generate_reduction_source`)."""
    return generate_reduction_source(kind, pre, name)


def generate_reduction_rust(kind: ReductionKind, pre: FusedChain | None = None, name: str = "fused_reduce") -> str:
    """Host-side counterpart of :func:`generate_reduction_ptx`: Python source over torch ops."""
    body = CpuCodegen().expr(pre.loop_ir().body) if pre is not None and len(pre) else "x0"
    red = {"sum": "sum(-1)", "mean": "mean(-1)", "prod": "prod(-1)", "max": "amax(-1)", "min": "amin(-1)"}[kind.value]
    return "def %s(x0):\n    return (%s).%s\n" % (name, body, red)


# --------------------------------------------------------------------------- op classification and lowering entry points
# (ferrotorch-jit/src/codegen_ir.rs:300-400, 840; dag_fusion.rs:105, 392; codegen_jit.rs:325; fusion_gpu.rs:79)
_REDUCTIONS = ("sum", "mean", "prod", "max", "min", "amax", "amin")


def _op_name(op) -> str:
    return str(getattr(op, "op", getattr(op, "value", op)))


def is_unary_elementwise(op) -> bool:
    from .ir import SCALAR, UNARY

    return _op_name(op) in UNARY or _op_name(op) in SCALAR


def is_binary_elementwise(op) -> bool:
    from .ir import BINARY

    return _op_name(op) in BINARY


def is_elementwise(op) -> bool:
    return is_unary_elementwise(op) or is_binary_elementwise(op)


def is_reduction(op) -> bool:
    return _op_name(op) in _REDUCTIONS


def ir_op_to_unary(op):
    """The :class:`UnaryOpKind` of an IR op name, or ``None``."""
    try:
        return UnaryOpKind(_op_name(op))
    except ValueError:
        return None


def ir_op_to_binary(op):
    try:
        return BinOpKind(_op_name(op))
    except ValueError:
        return None


def apply_op_expr(op, a: Expr, c: float | None = None) -> Expr:
    """The expression of a unary IR op (or a scalar op with constant ``c``) applied to ``a``."""
    name = _op_name(op)
    return LoopIR.from_program([{"op": name, "src": [("x", 0)], "c": c}], 1).body if a.kind == "load" and a.index == 0 else \
        _substitute(LoopIR.from_program([{"op": name, "src": [("x", 0)], "c": c}], 1).body, {0: a})


def apply_binary_op_expr(op, a: Expr, b: Expr) -> Expr:
    kind = ir_op_to_binary(op)
    if kind is None:
        raise JitError("apply_binary_op_expr: %r is not a binary elementwise op" % _op_name(op))
    return Expr.binary(kind, a, b)


def _substitute(e: Expr, env: dict) -> Expr:
    if e.kind == "load":
        return env.get(e.index, e)
    if not e.args:
        return e
    return Expr(e.kind, e.op, tuple(_substitute(x, env) for x in e.args), e.index, e.value)


@dataclass
class MatmulLoops:
    """The triple loop nest of ``out[m, n] = sum_k a[m, k] * b[k, n]`` as data, plus a runnable form."""
    m: int
    k: int
    n: int
    a_name: str = "a"
    b_name: str = "b"
    out_name: str = "out"

    def source(self) -> str:
        return ("for i in range(%d):\n    for j in range(%d):\n        acc = 0.0\n        for p in range(%d):\n"
                "            acc += %s[i * %d + p] * %s[p * %d + j]\n        %s[i * %d + j] = acc\n"
                % (self.m, self.n, self.k, self.a_name, self.k, self.b_name, self.n, self.out_name, self.n))

    def flops(self) -> int:
        return 2 * self.m * self.k * self.n

    def run(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        if tuple(a.shape) != (self.m, self.k) or tuple(b.shape) != (self.k, self.n):
            raise JitError("lower_matmul: operands %s @ %s do not match the lowered %dx%dx%d"
                           % (tuple(a.shape), tuple(b.shape), self.m, self.k, self.n))
        return a @ b


def lower_matmul(m: int, k: int, n: int, a_name: str = "a", b_name: str = "b", out_name: str = "out") -> MatmulLoops:
    return MatmulLoops(int(m), int(k), int(n), a_name, b_name, out_name)


def lower_to_loops(ops, n_inputs: int = 1) -> list:
    """A chain of IR ops (names, or ``(name, constant)`` pairs, applied in order to input 0; a binary op takes
    the running value and the next unused input) as loop IR: one fused :class:`LoopIR` for the elementwise
    run, ended by a ``("reduce", kind)`` marker when the chain closes with a reduction."""
    program, used = [], 1
    tail = None
    for k, o in enumerate(ops):
        name, c = (o, None) if isinstance(o, str) else (o[0], o[1])
        if is_reduction(name):
            if k != len(list(ops)) - 1:
                raise JitError("lower_to_loops: a reduction may only end the chain")
            tail = ("reduce", name)
            break
        src = [("x", 0)] if not program else [("r", len(program) - 1)]
        if is_binary_elementwise(name):
            if used >= n_inputs:
                raise JitError("lower_to_loops: %r needs another input (have %d)" % (name, n_inputs))
            src.append(("x", used))
            used += 1
        elif not is_unary_elementwise(name):
            raise JitError("lower_to_loops: %r is neither elementwise nor a reduction" % name)
        program.append({"op": name, "src": src, "c": c})
    loops = [LoopIR.from_program(program, n_inputs)] if program else []
    return loops + ([tail] if tail else [])


def jit_supports(loops) -> bool:
    """Whether the code generators take every construct in ``loops`` (elementwise expression trees over the
    documented unary / binary kinds; reductions by the kinds of :class:`ReductionKind`)."""
    def ok(e: Expr) -> bool:
        if e.kind in ("load", "const"):
            return True
        if e.kind == "unary":
            return isinstance(e.op, UnaryOpKind) and all(ok(a) for a in e.args)
        if e.kind == "binary":
            return isinstance(e.op, BinOpKind) and all(ok(a) for a in e.args)
        return False

    for item in loops:
        if isinstance(item, LoopIR):
            if not ok(item.body):
                return False
        elif isinstance(item, tuple) and item and item[0] == "reduce":
            if item[1] not in ("sum", "mean", "max", "min", "prod"):
                return False
        elif not isinstance(item, MatmulLoops):
            return False
    return True


def find_fusion_groups(graph: IrGraph) -> list:
    """The fused nodes of a graph, in topological order.  On a graph that has not been through the fusion
    passes yet, a copy is optimised first (the original is left as it is)."""
    groups = FusionGroup.of(graph)
    if groups or not any(is_elementwise(graph.nodes[i].op) for i in graph.order):
        return groups
    import copy

    from .ir import fuse_elementwise, pattern_fuse

    g2 = copy.deepcopy(graph)
    fuse_elementwise(g2)
    pattern_fuse(g2)
    return FusionGroup.of(g2)


def fuse_dag(groups, graph: IrGraph) -> list:
    """One list of loop IR per group: a fused loop for an elementwise group, a :class:`MatmulLoops` for a
    fused linear layer, nothing for groups without a loop form (attention)."""
    out = []
    for grp in groups:
        n = graph.nodes.get(grp.node_id)
        if n is None:
            out.append([])
        elif n.op == "fused_elementwise":
            out.append([LoopIR.from_program(n.attrs["program"], len(n.inputs))])
        elif n.op == "fused_linear_act" and n.shape is not None and graph.nodes[n.inputs[0]].shape is not None:
            k = graph.nodes[n.inputs[0]].shape[-1]
            rows = 1
            for d in n.shape[:-1]:
                rows *= d
            out.append([lower_matmul(rows, k, n.shape[-1])])
        else:
            out.append([])
    return out


def apply_fused_gpu(ops, x: torch.Tensor) -> torch.Tensor:
    """A chain of unary / scalar ops on a CUDA tensor in one generated kernel; the caller makes sure the
    tensor is on a CUDA device (``apply_fused`` checks and forwards here)."""
    if not x.is_cuda:
        raise JitError("apply_fused_gpu: the input is on %s, not on a CUDA device" % x.device)
    return _module.apply_fused(ops, x)
