"""The rest of the JIT surface: symbolic shapes with guards, segment-level graph breaks, AOT autograd
(a compiled forward and a compiled backward graph) and exported programs.

Reference: ferrotorch-jit/src/symbolic.rs (``ShapeSignature``, ``Guard``, ``compile_symbolic``),
graph_break.rs (``trace_with_breaks``, ``SegmentedModule``), aot_autograd.rs
(``decompose_forward_backward``, ``compile_aot``), export.rs (``DimSpec``, ``InputSpec``,
``ExportedProgram``, ``export``).  All of it sits on the IR, passes and generated kernels of
``jit.ir`` / ``jit.codegen`` / ``jit.module``.
"""
from __future__ import annotations

import io
import json
import struct
from dataclasses import dataclass, field

import torch
from torch import nn

from .ir import IrGraph, optimize
from .module import CompileConfig, JitError, TracedModule, _interpret, compile as _compile, lower_fx, trace


# --------------------------------------------------------------------------- symbolic shapes
@dataclass(frozen=True)
class SymbolicDim:
    input_index: int
    dim: int
    min: int = 1
    max: int | None = None


class ShapeSignature:
    """Which dimensions of which inputs may vary between calls (symbolic.rs:92-180)."""

    def __init__(self):
        self.dims: list[SymbolicDim] = []

    def symbolic_dim(self, input_index: int, dim: int) -> "ShapeSignature":
        return self.symbolic_dim_with_range(input_index, dim, 1, None)

    def symbolic_dim_with_range(self, input_index: int, dim: int, lo: int, hi: int | None) -> "ShapeSignature":
        if lo < 0 or (hi is not None and hi < lo):
            raise ValueError("symbolic_dim_with_range: need 0 <= min <= max")
        self.dims = [d for d in self.dims if (d.input_index, d.dim) != (input_index, dim)]
        self.dims.append(SymbolicDim(input_index, dim, lo, hi))
        return self

    def symbolic_dims_for(self, input_index: int) -> list[SymbolicDim]:
        return [d for d in self.dims if d.input_index == input_index]

    def is_symbolic(self, input_index: int, dim: int) -> bool:
        return any((d.input_index, d.dim) == (input_index, dim) for d in self.dims)


class Guard:
    """Checks a call's input shapes against the traced ones: fixed dimensions must match exactly,
    symbolic ones must lie in their range (symbolic.rs:183-290)."""

    def __init__(self, trace_shapes, signature: ShapeSignature):
        self.trace_shapes = [tuple(s) for s in trace_shapes]
        self.signature = signature
        for d in signature.dims:
            if d.input_index >= len(self.trace_shapes) or not -len(self.trace_shapes[d.input_index]) <= d.dim < len(self.trace_shapes[d.input_index]):
                raise ValueError("ShapeSignature names dimension %d of input %d, which the traced inputs do not have"
                                 % (d.dim, d.input_index))

    def check(self, input_shapes) -> None:
        shapes = [tuple(s) for s in input_shapes]
        if len(shapes) != len(self.trace_shapes):
            raise JitError("guard: %d inputs, traced with %d" % (len(shapes), len(self.trace_shapes)))
        for i, (got, want) in enumerate(zip(shapes, self.trace_shapes)):
            if len(got) != len(want):
                raise JitError("guard: input %d has rank %d, traced with rank %d" % (i, len(got), len(want)))
            sym = {d.dim % len(want): d for d in self.signature.symbolic_dims_for(i)}
            for k, (a, b) in enumerate(zip(got, want)):
                if k in sym:
                    d = sym[k]
                    if a < d.min or (d.max is not None and a > d.max):
                        raise JitError("guard: input %d dim %d = %d outside [%d, %s]" % (i, k, a, d.min, d.max))
                elif a != b:
                    raise JitError("guard: input %d dim %d = %d, traced with %d (not symbolic)" % (i, k, a, b))


def patch_reshape_for_symbolic_dims(g: IrGraph, trace_shapes, signature: ShapeSignature) -> int:
    """Shape arguments baked into ``reshape`` / ``view`` calls at trace time would pin a symbolic
    dimension to its traced size.  Where exactly one entry of such a shape equals the traced size
    of a symbolic dimension, that size occurs once in the reshaped tensor's own traced shape too
    (so the match is not a coincidence of equal sizes) and no entry is already -1, the entry becomes
    -1.  Shapes written as ``x.shape[0]`` in the traced code need no patch: fx keeps them dynamic.
    Returns the number of calls patched (symbolic.rs:341)."""
    sizes = {trace_shapes[d.input_index][d.dim] for d in signature.dims}
    patched = 0
    for n in g.nodes.values():
        if n.op != "call" or n.attrs.get("target") not in ("reshape", "view", torch.reshape):
            continue
        args = list(n.attrs["args"])
        shape = list(args[1]) if len(args) == 2 and isinstance(args[1], (tuple, list)) else args[1:]
        if not shape or not all(isinstance(v, int) for v in shape) or -1 in shape:
            continue
        hits = [k for k, v in enumerate(shape) if v in sizes]
        src = g.nodes[n.inputs[0]].shape if n.inputs else None
        if len(hits) == 1 and src is not None and list(src).count(shape[hits[0]]) == 1:
            shape[hits[0]] = -1
            n.attrs["args"] = (args[0], tuple(shape)) if len(args) == 2 and isinstance(args[1], (tuple, list)) else (args[0], *shape)
            patched += 1
    return patched


class SymbolicTracedModule(nn.Module):
    def __init__(self, traced: TracedModule, guard: Guard):
        super().__init__()
        self.traced, self.guard_ = traced, guard

    def inner(self) -> TracedModule:
        return self.traced

    def guard(self) -> Guard:
        return self.guard_

    def forward_symbolic(self, *inputs):
        tens = [t for t in inputs if isinstance(t, torch.Tensor)]
        self.guard_.check([t.shape for t in tens])
        env = _interpret(self.traced.graph, inputs, block=self.traced.cfg.block_size)
        outs = [env[i] for i in self.traced.graph.outputs]
        return torch.utils._pytree.tree_unflatten(outs, self.traced.graph.output_spec)

    forward = forward_symbolic


def compile_symbolic(fn, example_inputs, signature: ShapeSignature, config: CompileConfig | None = None) -> SymbolicTracedModule:
    """``compile`` whose result accepts other sizes in the dimensions ``signature`` names; the fused
    kernels take their extent from the call's inputs instead of the traced shape."""
    cfg = config or CompileConfig(fallback_to_eager=False)
    traced = _compile(fn, example_inputs, cfg)
    if not isinstance(traced, TracedModule):
        raise JitError("compile_symbolic: the callable could not be traced (%s)" % getattr(traced, "reason", "?"))
    shapes = [tuple(t.shape) for t in example_inputs if isinstance(t, torch.Tensor)]
    guard = Guard(shapes, signature)
    patch_reshape_for_symbolic_dims(traced.graph, shapes, signature)
    for n in traced.graph.nodes.values():
        if n.op == "fused_elementwise":
            n.shape = None                      # broadcast extent is computed per call
    return SymbolicTracedModule(traced, guard)


# --------------------------------------------------------------------------- graph breaks
@dataclass
class GraphSegment:
    """A run of stages that traced (``compiled`` is the :class:`TracedModule`) or one stage that did
    not (``eager`` is the original callable; ``reason`` says why) -- graph_break.rs:109-130."""
    compiled: nn.Module | None = None
    eager: object | None = None
    reason: str = ""

    def is_compiled(self) -> bool:
        return self.compiled is not None

    def __call__(self, x):
        return self.compiled(x) if self.compiled is not None else self.eager(x)


class SegmentedModule(nn.Module):
    def __init__(self, segments: list[GraphSegment]):
        super().__init__()
        self.segs = list(segments)
        self.compiled_modules = nn.ModuleList(s.compiled for s in self.segs if s.compiled is not None)

    def forward(self, x):
        for s in self.segs:
            x = s(x)
        return x

    def segment_count(self) -> int:
        return len(self.segs)

    def segments(self) -> list[GraphSegment]:
        return self.segs

    def is_fully_compiled(self) -> bool:
        return all(s.is_compiled() for s in self.segs)


def trace_with_breaks(stages, example_input: torch.Tensor, config: CompileConfig | None = None) -> SegmentedModule:
    """Compile a pipeline of single-input stages (an ``nn.Sequential`` or a list of callables) piece
    by piece: neighbouring stages that trace are compiled together as one graph, a stage that does
    not trace (data-dependent control flow, unsupported Python) stays eager between them
    (graph_break.rs:242).  The reference splits one function at the untraceable operation; here
    the split points are the stage boundaries the caller provides."""
    cfg = config or CompileConfig(fallback_to_eager=False)
    stages = list(stages.children()) if isinstance(stages, nn.Sequential) else list(stages)
    segments: list[GraphSegment] = []
    run: list = []
    x = example_input

    def flush(inp):
        if not run:
            return
        fn = nn.Sequential(*run) if all(isinstance(s, nn.Module) for s in run) else _Chain(list(run))
        segments.append(GraphSegment(compiled=_compile(fn, (inp,), CompileConfig(cfg.optimization, False, cfg.block_size))))
        run.clear()

    run_input = x
    for st in stages:
        try:
            trace(st if isinstance(st, nn.Module) else _Chain([st]), (x,))
            ok, why = True, ""
        except JitError as e:
            ok, why = False, str(e)
        if ok:
            if not run:
                run_input = x
            run.append(st)
        else:
            flush(run_input)
            segments.append(GraphSegment(eager=st, reason=why))
        with torch.no_grad():
            x = st(x)
    flush(run_input)
    return SegmentedModule(segments)


class _Chain(nn.Module):
    def __init__(self, fns):
        super().__init__()
        self.fns = fns
        self.mods = nn.ModuleList(f for f in fns if isinstance(f, nn.Module))

    def forward(self, x):
        for f in self.fns:
            x = f(x)
        return x


# --------------------------------------------------------------------------- AOT autograd
@dataclass
class AotGraphPair:
    """The forward graph and the graph that maps ``(parameters, inputs, output gradients)`` to the
    gradients of the parameters and inputs (aot_autograd.rs:39-90).  The backward graph recomputes
    the forward's intermediates instead of receiving them, so the pair shares no saved tensors."""
    forward: IrGraph
    backward: IrGraph
    n_params: int
    n_inputs: int
    stats: dict = field(default_factory=dict)


def decompose_forward_backward(fn, example_inputs, config: CompileConfig | None = None):
    """Trace ``fn`` (module or function) to its forward graph and, through ATen-level tracing of
    ``torch.autograd.grad``, to a backward graph; both go through the same optimisation passes, so
    the elementwise chains of the backward are fused kernels too.  Returns
    ``(pair, param_names, functional)``."""
    from torch.fx.experimental.proxy_tensor import make_fx

    cfg = config or CompileConfig()
    example_inputs = tuple(example_inputs)
    mod = fn if isinstance(fn, nn.Module) else None
    names = [n for n, _ in mod.named_parameters()] if mod is not None else []
    params = [p.detach() for _, p in mod.named_parameters()] if mod is not None else []

    def functional(*flat):
        ps, xs = flat[:len(names)], flat[len(names):]
        if mod is None:
            return fn(*xs)
        return torch.func.functional_call(mod, dict(zip(names, ps)), tuple(xs))

    with torch.no_grad():
        out = functional(*params, *example_inputs)
    if not isinstance(out, torch.Tensor):
        raise JitError("compile_aot: the callable must return one tensor")
    diff = [i for i, t in enumerate((*params, *example_inputs)) if t.is_floating_point()]

    def bwd(*flat_and_grad):
        *flat, g = flat_and_grad
        leaves = [t.detach().requires_grad_(i in diff) for i, t in enumerate(flat)]
        y = functional(*leaves)
        grads = torch.autograd.grad(y, [leaves[i] for i in diff], g, allow_unused=True)
        return tuple(torch.zeros_like(leaves[i]) if gr is None else gr for i, gr in zip(diff, grads))

    fwd_graph = lower_fx(make_fx(functional)(*params, *example_inputs), (*params, *example_inputs))
    bwd_args = (*params, *example_inputs, torch.ones_like(out))
    bwd_graph = lower_fx(make_fx(bwd)(*bwd_args), bwd_args)
    stats = {"forward": optimize(fwd_graph, cfg.optimization), "backward": optimize(bwd_graph, cfg.optimization)}
    pair = AotGraphPair(fwd_graph, bwd_graph, len(names), len(example_inputs), stats)
    pair.diff = diff
    return pair, names, functional


class _AotFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pair, block, *flat):
        ctx.pair, ctx.block = pair, block
        ctx.save_for_backward(*flat)
        env = _interpret(pair.forward, flat, block=block)
        return env[pair.forward.outputs[0]]

    @staticmethod
    def backward(ctx, g):
        pair, flat = ctx.pair, ctx.saved_tensors
        env = _interpret(pair.backward, (*flat, g.contiguous()), block=ctx.block)
        got = {i: env[o] for i, o in zip(pair.diff, pair.backward.outputs)}
        return (None, None, *[got.get(i) for i in range(len(flat))])


class AotModule(nn.Module):
    """Runs the compiled forward graph and, in ``backward()``, the compiled backward graph."""

    def __init__(self, pair: AotGraphPair, module: nn.Module | None, names: list[str], cfg: CompileConfig):
        super().__init__()
        self.pair, self.module, self.names, self.cfg = pair, module, names, cfg

    def forward(self, *inputs):
        ps = [dict(self.module.named_parameters())[n] for n in self.names] if self.module is not None else []
        return _AotFn.apply(self.pair, self.cfg.block_size, *ps, *inputs)

    # ---- the two directions by hand (aot_autograd.rs ``AotCompiledModule``): here the backward graph takes the
    # forward's *inputs* and recomputes what it needs, so the "saved tensors" are the parameters and inputs
    def forward_graph(self) -> IrGraph:
        return self.pair.forward

    def backward_graph(self) -> IrGraph:
        return self.pair.backward

    def _flat(self, inputs) -> list:
        ps = [dict(self.module.named_parameters())[n].detach() for n in self.names] if self.module is not None else []
        return [*ps, *[t.detach() for t in inputs]]

    def forward_with_ctx(self, *inputs):
        """``(output, context)``; hand the context to :meth:`backward` with the output's gradient."""
        flat = self._flat(inputs)
        env = _interpret(self.pair.forward, flat, block=self.cfg.block_size)
        return env[self.pair.forward.outputs[0]], flat

    def saved_tensors(self, ctx) -> list:
        return list(ctx)

    def saved_tensor_indices(self) -> list:
        """Positions, among ``parameters + inputs``, of the tensors the backward graph reads: all of them."""
        return list(range(self.pair.n_params + self.pair.n_inputs))

    def backward(self, ctx, grad_output: torch.Tensor) -> list:
        """Gradients in the order ``parameters + inputs`` (``None`` where none is defined)."""
        env = _interpret(self.pair.backward, (*ctx, grad_output.contiguous()), block=self.cfg.block_size)
        got = {i: env[o] for i, o in zip(self.pair.diff, self.pair.backward.outputs)}
        return [got.get(i) for i in range(len(ctx))]


def compile_aot(fn, example_inputs, config: CompileConfig | None = None) -> AotModule:
    """``compile`` for training: both directions run from graphs built ahead of time
    (aot_autograd.rs:465).  Shapes are those of ``example_inputs``."""
    cfg = config or CompileConfig()
    pair, names, _ = decompose_forward_backward(fn, example_inputs, cfg)
    return AotModule(pair, fn if isinstance(fn, nn.Module) else None, names, cfg)


# --------------------------------------------------------------------------- export
@dataclass(frozen=True)
class DimSpec:
    """One dimension of an exported program's input: a fixed size, or a named dynamic one with an
    optional range (export.rs:50-95)."""
    size: int | None = None
    name: str | None = None
    min: int = 1
    max: int | None = None

    @classmethod
    def static(cls, size: int) -> "DimSpec":
        return cls(size=size)

    @classmethod
    def dynamic(cls, name: str) -> "DimSpec":
        return cls(name=name)

    @classmethod
    def dynamic_range(cls, name: str, lo: int, hi: int) -> "DimSpec":
        if lo < 0 or hi < lo:
            raise ValueError("dynamic_range: need 0 <= min <= max")
        return cls(name=name, min=lo, max=hi)

    def is_dynamic(self) -> bool:
        return self.name is not None


@dataclass
class InputSpec:
    shape: list

    @classmethod
    def all_static(cls, shape) -> "InputSpec":
        return cls([DimSpec.static(int(s)) for s in shape])

    def has_dynamic_dims(self) -> bool:
        return any(d.is_dynamic() for d in self.shape)

    def rank(self) -> int:
        return len(self.shape)


@dataclass
class ExportedProgramMetadata:
    input_specs: list
    input_dtypes: list
    output_shape: list
    ir_ops: list


_EP_MAGIC = b"FTEP1\n"


class ExportedProgram:
    """A traced module frozen with its weights: runs without the Python class that defined it,
    checks its inputs against the declared specs, and round-trips through bytes or a file
    (export.rs:145-660).  The graph and weights travel in ``torch.export``'s archive; the metadata
    (input specs, dtypes, output shape, the IR's op list) as JSON in front of it."""

    def __init__(self, program, meta: ExportedProgramMetadata):
        self.program, self.meta = program, meta
        self._module = program.module()
        self.ir_graph = None

    # -- running
    def check_inputs(self, *inputs) -> None:
        if len(inputs) != len(self.meta.input_specs):
            raise JitError("exported program takes %d inputs, got %d" % (len(self.meta.input_specs), len(inputs)))
        names: dict[str, int] = {}
        for i, (t, spec, dt) in enumerate(zip(inputs, self.meta.input_specs, self.meta.input_dtypes)):
            if t.dim() != spec.rank():
                raise JitError("input %d: rank %d, exported with rank %d" % (i, t.dim(), spec.rank()))
            if str(t.dtype) != dt:
                raise JitError("input %d: dtype %s, exported with %s" % (i, t.dtype, dt))
            for k, (n, d) in enumerate(zip(t.shape, spec.shape)):
                if not d.is_dynamic():
                    if n != d.size:
                        raise JitError("input %d dim %d = %d, exported as %d" % (i, k, n, d.size))
                    continue
                if n < d.min or (d.max is not None and n > d.max):
                    raise JitError("input %d dim %d (%s) = %d outside [%d, %s]" % (i, k, d.name, n, d.min, d.max))
                if names.setdefault(d.name, n) != n:
                    raise JitError("dynamic dimension %r is %d in one place and %d in another" % (d.name, names[d.name], n))

    def run(self, *inputs):
        return self._module(*inputs)

    def run_with_guards(self, *inputs):
        self.check_inputs(*inputs)
        return self._module(*inputs)

    __call__ = run_with_guards

    # -- metadata
    def to_json(self) -> str:
        m = self.meta
        return json.dumps({"input_specs": [[{"size": d.size, "name": d.name, "min": d.min, "max": d.max} for d in s.shape]
                                           for s in m.input_specs],
                           "input_dtypes": m.input_dtypes, "output_shape": m.output_shape, "ir_ops": m.ir_ops})

    @staticmethod
    def parse_json_metadata(text: str) -> ExportedProgramMetadata:
        try:
            d = json.loads(text)
            specs = [InputSpec([DimSpec(**e) for e in s]) for s in d["input_specs"]]
            return ExportedProgramMetadata(specs, list(d["input_dtypes"]), list(d["output_shape"]), list(d["ir_ops"]))
        except (ValueError, KeyError, TypeError) as e:
            raise JitError("exported program: bad metadata (%s)" % e)

    # -- bytes and files
    def serialize(self) -> bytes:
        buf = io.BytesIO()
        torch.export.save(self.program, buf)
        meta = self.to_json().encode()
        return _EP_MAGIC + struct.pack("<Q", len(meta)) + meta + buf.getvalue()

    @classmethod
    def deserialize(cls, data: bytes) -> "ExportedProgram":
        if not data.startswith(_EP_MAGIC) or len(data) < len(_EP_MAGIC) + 8:
            raise JitError("not an exported program (bad magic)")
        off = len(_EP_MAGIC)
        (n,) = struct.unpack_from("<Q", data, off)
        if n > len(data) - off - 8:
            raise JitError("exported program: metadata length %d exceeds the data" % n)
        meta = cls.parse_json_metadata(data[off + 8:off + 8 + n].decode())
        return cls(torch.export.load(io.BytesIO(data[off + 8 + n:])), meta)

    def save(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.serialize())

    @classmethod
    def load(cls, path: str) -> "ExportedProgram":
        with open(path, "rb") as f:
            return cls.deserialize(f.read())


def export(module: nn.Module, example_inputs, input_specs: list[InputSpec] | None = None) -> ExportedProgram:
    """Freeze ``module`` for the given example inputs; ``input_specs`` (one per input) names the
    dimensions that may vary (export.rs:663)."""
    example_inputs = tuple(example_inputs)
    specs = input_specs or [InputSpec.all_static(t.shape) for t in example_inputs]
    if len(specs) != len(example_inputs):
        raise JitError("export: %d specs for %d inputs" % (len(specs), len(example_inputs)))
    dims: dict[str, object] = {}
    dynamic = []
    for t, s in zip(example_inputs, specs):
        if s.rank() != t.dim():
            raise JitError("export: a spec of rank %d for an input of rank %d" % (s.rank(), t.dim()))
        entry = {}
        for k, d in enumerate(s.shape):
            if d.is_dynamic():
                if d.name not in dims:
                    dims[d.name] = torch.export.Dim(d.name, min=max(d.min, 1) if d.min > 1 else None, max=d.max)
                entry[k] = dims[d.name]
            elif d.size != t.shape[k]:
                raise JitError("export: spec says %d for a dimension of size %d" % (d.size, t.shape[k]))
        dynamic.append(entry or None)
    try:
        ir_graph = trace(module, example_inputs)
        ir_ops = ir_graph.ops()
    except JitError:
        ir_graph, ir_ops = None, []
    program = torch.export.export(module, example_inputs, dynamic_shapes=tuple(dynamic) if dims else None)
    with torch.no_grad():
        out = module(*example_inputs)
    meta = ExportedProgramMetadata(list(specs), [str(t.dtype) for t in example_inputs],
                                   list(out.shape) if isinstance(out, torch.Tensor) else [], ir_ops)
    ep = ExportedProgram(program, meta)
    ep.ir_graph = ir_graph          # kept in memory only (ONNX export uses it); a loaded program has none
    return ep
