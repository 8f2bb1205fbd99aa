"""ONNX export of a traced graph with a hand-written protobuf encoder, plus a small decoder and
reference evaluator so an exported file can be checked without any ONNX package.

The reference does the same (ferrotorch-serialize/src/onnx_export.rs:68-1182: ``ProtobufWriter``,
``encode_*`` builders, ``map_ir_op``, SiLU / GELU decomposed for opset 17, ``OnnxDimSpec`` for
dynamic axes, ``ir_graph_to_onnx``, ``export_onnx``, ``export_ir_graph_to_onnx``).  ``torch.onnx``
needs the ``onnxscript`` package, which is not part of every install; this path needs nothing.

Supported graph content: the IR's elementwise ops, ``nn.Linear`` (MatMul + Add), ``matmul``,
``softmax``, transposes of the last two axes, ``reshape`` / ``view`` / ``flatten``.  Anything else
raises :class:`OnnxExportError` naming the node.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass, field

import torch
from torch import nn

ONNX_FLOAT, ONNX_UINT8, ONNX_INT8, ONNX_INT32, ONNX_INT64, ONNX_BOOL, ONNX_FLOAT16, ONNX_DOUBLE, ONNX_BFLOAT16 = 1, 2, 3, 6, 7, 9, 10, 11, 16
_DTYPE = {torch.float32: ONNX_FLOAT, torch.float64: ONNX_DOUBLE, torch.float16: ONNX_FLOAT16, torch.bfloat16: ONNX_BFLOAT16,
          torch.int64: ONNX_INT64, torch.int32: ONNX_INT32, torch.int8: ONNX_INT8, torch.uint8: ONNX_UINT8, torch.bool: ONNX_BOOL}
_DTYPE_INV = {v: k for k, v in _DTYPE.items()}


class OnnxExportError(ValueError):
    pass


@dataclass
class OnnxExportConfig:
    opset_version: int = 17
    model_name: str = "ferrotorch_b200_model"
    producer_name: str = "ferrotorch_b200"
    producer_version: str = "0.1.0"
    input_names: list | None = None
    output_names: list | None = None
    dynamic_axes: dict = field(default_factory=dict)     # input / output name -> {axis: symbol}


# --------------------------------------------------------------------------- protobuf wire format
class ProtobufWriter:
    """Varints, tags and length-delimited fields: all the wire format ONNX needs."""

    def __init__(self):
        self.buf = bytearray()

    @staticmethod
    def varint(n: int) -> bytes:
        if n < 0:
            n += 1 << 64                      # negative int64 values are ten-byte two's-complement varints
        out = bytearray()
        while True:
            b = n & 0x7F
            n >>= 7
            out.append(b | (0x80 if n else 0))
            if not n:
                return bytes(out)

    def _tag(self, fieldno: int, wire: int) -> None:
        self.buf += self.varint((fieldno << 3) | wire)

    def int(self, fieldno: int, value: int) -> "ProtobufWriter":
        self._tag(fieldno, 0)
        self.buf += self.varint(int(value))
        return self

    def float(self, fieldno: int, value: float) -> "ProtobufWriter":
        self._tag(fieldno, 5)
        self.buf += struct.pack("<f", value)
        return self

    def bytes(self, fieldno: int, data) -> "ProtobufWriter":
        data = data.encode() if isinstance(data, str) else bytes(data)
        self._tag(fieldno, 2)
        self.buf += self.varint(len(data)) + data
        return self

    string = bytes

    def message(self, fieldno: int, sub: "ProtobufWriter") -> "ProtobufWriter":
        return self.bytes(fieldno, sub.buf)

    def packed_ints(self, fieldno: int, values) -> "ProtobufWriter":
        return self.bytes(fieldno, b"".join(self.varint(int(v)) for v in values))

    def finish(self) -> bytes:
        return bytes(self.buf)


def read_message(data: bytes) -> list[tuple[int, int, object]]:
    """Decode one message level into ``(field, wire type, value)`` triples; nested messages stay
    bytes (call again on them)."""
    out, i, n = [], 0, len(data)

    def varint():
        nonlocal i
        shift = v = 0
        while True:
            if i >= n:
                raise OnnxExportError("protobuf: truncated varint")
            b = data[i]
            i += 1
            v |= (b & 0x7F) << shift
            if not b & 0x80:
                return v
            shift += 7
            if shift > 63:
                raise OnnxExportError("protobuf: varint longer than 10 bytes")

    while i < n:
        key = varint()
        f, w = key >> 3, key & 7
        if w == 0:
            out.append((f, w, varint()))
        elif w == 2:
            ln = varint()
            if i + ln > n:
                raise OnnxExportError("protobuf: length-delimited field overruns the buffer")
            out.append((f, w, data[i:i + ln]))
            i += ln
        elif w == 5:
            out.append((f, w, struct.unpack_from("<f", data, i)[0]))
            i += 4
        elif w == 1:
            out.append((f, w, struct.unpack_from("<d", data, i)[0]))
            i += 8
        else:
            raise OnnxExportError("protobuf: unsupported wire type %d" % w)
    return out


# --------------------------------------------------------------------------- ONNX message builders
def encode_tensor(name: str, t: torch.Tensor) -> ProtobufWriter:
    if t.dtype not in _DTYPE:
        raise OnnxExportError("tensor %s: dtype %s has no ONNX counterpart" % (name, t.dtype))
    w = ProtobufWriter()
    for d in t.shape:
        w.int(1, d)
    w.int(2, _DTYPE[t.dtype]).string(8, name)
    c = t.detach().cpu().contiguous()
    raw = c.reshape(-1).view(torch.uint8).numpy().tobytes() if c.numel() else b""
    return w.bytes(9, raw)


def encode_value_info(name: str, dtype: torch.dtype, shape, dynamic: dict | None = None) -> ProtobufWriter:
    shp = ProtobufWriter()
    for axis, d in enumerate(shape):
        dim = ProtobufWriter()
        if dynamic and axis in dynamic:
            dim.string(2, dynamic[axis])          # dim_param
        else:
            dim.int(1, d)                         # dim_value
        shp.message(1, dim)
    tensor_type = ProtobufWriter().int(1, _DTYPE[dtype]).message(2, shp)
    return ProtobufWriter().string(1, name).message(2, ProtobufWriter().message(1, tensor_type))


def encode_dim_param(param: str) -> ProtobufWriter:
    """A ``TensorShapeProto.Dimension`` that is symbolic: ``dim_param = param`` (onnx_export.rs:337)."""
    return ProtobufWriter().string(2, param)


def encode_shape_with_dynamic(dims) -> ProtobufWriter:
    """A ``TensorShapeProto`` from a list whose entries are integers (static extents) or strings (names of
    dynamic dimensions)."""
    shp = ProtobufWriter()
    for d in dims:
        shp.message(1, encode_dim_param(d) if isinstance(d, str) else ProtobufWriter().int(1, int(d)))
    return shp


def encode_value_info_dynamic(name: str, elem_type, dims) -> ProtobufWriter:
    """A ``ValueInfoProto`` whose shape mixes static and named dynamic dimensions; ``elem_type`` is an ONNX element
    type number or a torch dtype."""
    et = _DTYPE[elem_type] if isinstance(elem_type, torch.dtype) else int(elem_type)
    tensor_type = ProtobufWriter().int(1, et).message(2, encode_shape_with_dynamic(dims))
    return ProtobufWriter().string(1, name).message(2, ProtobufWriter().message(1, tensor_type))


def encode_attribute(name: str, value) -> ProtobufWriter:
    a = ProtobufWriter().string(1, name)
    if isinstance(value, bool) or isinstance(value, int):
        return a.int(3, int(value)).int(20, 2)                     # INT
    if isinstance(value, float):
        return a.float(2, value).int(20, 1)                        # FLOAT
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        for v in value:
            a.int(8, v)
        return a.int(20, 7)                                        # INTS
    if isinstance(value, torch.Tensor):
        return a.message(5, encode_tensor("", value)).int(20, 4)   # TENSOR
    raise OnnxExportError("attribute %s: unsupported value %r" % (name, value))


def encode_node(op_type: str, inputs, outputs, name: str = "", **attrs) -> ProtobufWriter:
    n = ProtobufWriter()
    for i in inputs:
        n.string(1, i)
    for o in outputs:
        n.string(2, o)
    n.string(3, name or outputs[0]).string(4, op_type)
    for k, v in attrs.items():
        n.message(5, encode_attribute(k, v))
    return n


# --------------------------------------------------------------------------- IR -> ONNX
_SIMPLE_UNARY = {"neg": "Neg", "relu": "Relu", "sigmoid": "Sigmoid", "tanh": "Tanh", "sqrt": "Sqrt", "abs": "Abs",
                 "exp": "Exp", "log": "Log"}
_SIMPLE_BINARY = {"add": "Add", "sub": "Sub", "mul": "Mul", "div": "Div"}


class _Builder:
    def __init__(self, cfg: OnnxExportConfig):
        self.cfg = cfg
        self.nodes: list[ProtobufWriter] = []
        self.inits: list[ProtobufWriter] = []
        self._n = 0

    def fresh(self, hint: str = "t") -> str:
        self._n += 1
        return "%s_%d" % (hint, self._n)

    def const(self, value: torch.Tensor, hint: str = "c") -> str:
        name = self.fresh(hint)
        self.inits.append(encode_tensor(name, value))
        return name

    def scalar(self, v: float, dtype: torch.dtype) -> str:
        return self.const(torch.tensor(v, dtype=dtype), "s")

    def node(self, op: str, inputs, out: str | None = None, **attrs) -> str:
        out = out or self.fresh(op.lower())
        self.nodes.append(encode_node(op, inputs, [out], **attrs))
        return out


def _emit(b: _Builder, n, names: dict, out: str) -> None:
    """Append the ONNX nodes of IR node ``n``; its result must be called ``out``."""
    ins = [names[i] for i in n.inputs]
    dt = n.dtype or torch.float32
    op = n.op
    if op in _SIMPLE_UNARY:
        b.node(_SIMPLE_UNARY[op], ins, out)
    elif op in _SIMPLE_BINARY:
        b.node(_SIMPLE_BINARY[op], ins, out)
    elif op == "silu":                                   # x * sigmoid(x): no Silu operator before opset 22
        b.node("Mul", [ins[0], b.node("Sigmoid", ins)], out)
    elif op == "gelu":                                   # 0.5 x (1 + erf(x / sqrt 2)): no Gelu before opset 20
        e = b.node("Erf", [b.node("Mul", [ins[0], b.scalar(1.0 / math.sqrt(2.0), dt)])])
        half = b.node("Mul", [ins[0], b.scalar(0.5, dt)])
        b.node("Mul", [half, b.node("Add", [e, b.scalar(1.0, dt)])], out)
    elif op in ("add_c", "mul_c", "pow_c", "rsub_c", "rdiv_c"):
        c = b.scalar(float(n.attrs["c"]), dt)
        kind, args = {"add_c": ("Add", [ins[0], c]), "mul_c": ("Mul", [ins[0], c]), "pow_c": ("Pow", [ins[0], c]),
                      "rsub_c": ("Sub", [c, ins[0]]), "rdiv_c": ("Div", [c, ins[0]])}[op]
        b.node(kind, args, out)
    elif op == "call":
        _emit_call(b, n, names, out)
    else:
        raise OnnxExportError("node %d: IR op %r cannot be exported (export the un-optimised trace)" % (n.id, op))


def _emit_call(b: _Builder, n, names: dict, out: str) -> None:
    tgt, kind, args, kwargs = n.attrs["target"], n.attrs.get("kind"), n.attrs["args"], n.attrs["kwargs"]
    ins = [names[i] for i in n.inputs]

    def plain(a):
        return a if not hasattr(a, "id") else None

    if kind == "linear" and n.shape is not None and len(n.shape) == 2:
        # a matrix times a weight: one Gemm with the weight as stored (transB), as the reference emits
        w = [ins[0], b.const(tgt.weight.detach(), "weight")] + ([b.const(tgt.bias.detach(), "bias")] if tgt.bias is not None else [])
        b.node("Gemm", w, out, transB=1)
    elif kind == "linear":
        w = b.const(tgt.weight.detach().t().contiguous(), "weight")
        y = b.node("MatMul", [ins[0], w], None if tgt.bias is not None else out)
        if tgt.bias is not None:
            b.node("Add", [y, b.const(tgt.bias.detach(), "bias")], out)
    elif kind == "matmul":
        b.node("MatMul", ins[:2], out)
    elif kind == "softmax":
        dim = kwargs.get("dim", plain(args[1]) if len(args) > 1 else -1)
        b.node("Softmax", ins[:1], out, axis=int(dim))
    elif kind == "transpose_last":
        rank = len(n.shape)
        perm = list(range(rank))
        perm[-1], perm[-2] = perm[-2], perm[-1]
        b.node("Transpose", ins[:1], out, perm=perm)
    elif tgt in ("reshape", "view", torch.reshape, "flatten", torch.flatten) or isinstance(tgt, nn.Flatten):
        b.node("Reshape", [ins[0], b.const(torch.tensor(list(n.shape), dtype=torch.int64), "shape")], out)
    elif isinstance(tgt, nn.Dropout) or tgt in (nn.functional.dropout, "contiguous", "detach") or isinstance(tgt, nn.Identity):
        b.node("Identity", ins[:1], out)
    elif _emit_structural(b, n, tgt, args, kwargs, ins, out):
        pass
    else:
        raise OnnxExportError("node %d: call to %r has no ONNX mapping" % (n.id, getattr(tgt, "__name__", tgt)))


def _axes(v, rank: int) -> list[int]:
    v = [v] if isinstance(v, int) else list(v)
    return [a % rank for a in v]


def _emit_structural(b: _Builder, n, tgt, args, kwargs, ins, out) -> bool:
    """Reductions, log-softmax, squeeze / unsqueeze, concatenation, general transposes and the
    layers of a convolutional network (the operator list of the reference's exporter,
    ferrotorch-serialize/src/onnx_export.rs:528-716, plus Conv / pooling / batch norm).  Returns
    False when ``tgt`` is none of them."""
    plain = [a for a in args if not hasattr(a, "id")]
    first = args[0] if args else None
    in_rank = len(first.shape) if hasattr(first, "shape") and first.shape is not None else None
    i64 = lambda v: b.const(torch.tensor(list(v), dtype=torch.int64), "axes")  # noqa: E731
    red = {torch.sum: "ReduceSum", "sum": "ReduceSum", torch.mean: "ReduceMean", "mean": "ReduceMean", torch.prod: "ReduceProd",
           "prod": "ReduceProd"}
    if tgt in red:
        dim = kwargs.get("dim", plain[0] if plain else None)
        keep = int(bool(kwargs.get("keepdim", plain[1] if len(plain) > 1 else False)))
        op = red[tgt]
        if dim is None:
            b.node(op, ins[:1], out, keepdims=0)
        elif op == "ReduceSum":                                   # axes are an input since opset 13
            b.node(op, [ins[0], i64(_axes(dim, in_rank))], out, keepdims=keep)
        else:                                                     # ... and an attribute until opset 18
            b.node(op, ins[:1], out, axes=_axes(dim, in_rank), keepdims=keep)
        return True
    if tgt in (torch.log_softmax, nn.functional.log_softmax, "log_softmax") or isinstance(tgt, nn.LogSoftmax):
        dim = tgt.dim if isinstance(tgt, nn.LogSoftmax) else kwargs.get("dim", plain[0] if plain else -1)
        b.node("LogSoftmax", ins[:1], out, axis=int(dim))
        return True
    if tgt in (torch.squeeze, "squeeze", torch.unsqueeze, "unsqueeze"):
        dim = kwargs.get("dim", plain[0] if plain else None)
        if tgt in (torch.squeeze, "squeeze"):
            b.node("Squeeze", ins[:1] if dim is None else [ins[0], i64(_axes(dim, in_rank))], out)
        else:
            b.node("Unsqueeze", [ins[0], i64([dim % (in_rank + 1)])], out)
        return True
    if tgt in (torch.cat, torch.concat):
        dim = kwargs.get("dim", args[1] if len(args) > 1 else 0)
        b.node("Concat", ins, out, axis=int(dim) % len(n.shape))
        return True
    if tgt in ("permute", torch.permute):
        perm = plain[0] if len(plain) == 1 and isinstance(plain[0], (list, tuple)) else plain
        b.node("Transpose", ins[:1], out, perm=_axes(perm, in_rank))
        return True
    if tgt in ("transpose", torch.transpose, "t"):
        perm = list(range(in_rank))
        a0, a1 = (0, 1) if tgt == "t" else (plain[0] % in_rank, plain[1] % in_rank)
        perm[a0], perm[a1] = perm[a1], perm[a0]
        b.node("Transpose", ins[:1], out, perm=perm)
        return True
    if isinstance(tgt, nn.Conv2d):
        if isinstance(tgt.padding, str) or tgt.padding_mode != "zeros":
            raise OnnxExportError("Conv2d with padding %r / mode %r cannot be exported" % (tgt.padding, tgt.padding_mode))
        w = [ins[0], b.const(tgt.weight.detach(), "weight")] + ([b.const(tgt.bias.detach(), "bias")] if tgt.bias is not None else [])
        b.node("Conv", w, out, kernel_shape=list(tgt.kernel_size), strides=list(tgt.stride), pads=list(tgt.padding) * 2,
               dilations=list(tgt.dilation), group=int(tgt.groups))
        return True
    if isinstance(tgt, nn.BatchNorm2d):
        if tgt.training or tgt.running_mean is None:
            raise OnnxExportError("BatchNorm2d is exported in eval mode with running statistics")
        ones, zeros = torch.ones_like(tgt.running_mean), torch.zeros_like(tgt.running_mean)
        b.node("BatchNormalization", [ins[0], b.const((tgt.weight if tgt.weight is not None else ones).detach(), "scale"),
                                      b.const((tgt.bias if tgt.bias is not None else zeros).detach(), "bias"),
                                      b.const(tgt.running_mean.detach(), "mean"), b.const(tgt.running_var.detach(), "var")],
               out, epsilon=float(tgt.eps))
        return True
    if isinstance(tgt, (nn.MaxPool2d, nn.AvgPool2d)):
        pair = lambda v: [v, v] if isinstance(v, int) else list(v)  # noqa: E731
        k, st, pd = pair(tgt.kernel_size), pair(tgt.stride or tgt.kernel_size), pair(tgt.padding)
        extra = {"ceil_mode": int(tgt.ceil_mode)}
        if isinstance(tgt, nn.AvgPool2d):
            extra["count_include_pad"] = int(tgt.count_include_pad)
        elif pair(tgt.dilation) != [1, 1]:
            extra["dilations"] = pair(tgt.dilation)
        b.node("MaxPool" if isinstance(tgt, nn.MaxPool2d) else "AveragePool", ins[:1], out, kernel_shape=k, strides=st, pads=pd * 2, **extra)
        return True
    if isinstance(tgt, nn.AdaptiveAvgPool2d) and tgt.output_size in (1, (1, 1)):
        b.node("GlobalAveragePool", ins[:1], out)
        return True
    return False


def ir_graph_to_onnx(graph, config: OnnxExportConfig | None = None) -> bytes:
    """Serialise an :class:`~ferrotorch_b200.jit.ir.IrGraph` (as ``jit.trace`` returns it) to the
    bytes of an ONNX ``ModelProto``."""
    cfg = config or OnnxExportConfig()
    b = _Builder(cfg)
    names: dict[int, str] = {}
    inputs, n_in = [], 0
    out_names = {}
    for k, oid in enumerate(graph.outputs):
        out_names[oid] = (cfg.output_names[k] if cfg.output_names and k < len(cfg.output_names) else "output_%d" % k)
    for i in graph.order:
        n = graph.nodes[i]
        if n.op == "input":
            nm = cfg.input_names[n_in] if cfg.input_names and n_in < len(cfg.input_names) else "input_%d" % n_in
            n_in += 1
            names[i] = nm
            inputs.append(encode_value_info(nm, n.dtype, n.shape, cfg.dynamic_axes.get(nm)))
        elif n.op == "const":
            names[i] = b.const(n.attrs["value"].detach(), "const")
        else:
            names[i] = out_names.get(i) or b.fresh("n%d" % i)
            _emit(b, n, names, names[i])
    g = ProtobufWriter()
    for nd in b.nodes:
        g.message(1, nd)
    g.string(2, cfg.model_name)
    for t in b.inits:
        g.message(5, t)
    for vi in inputs:
        g.message(11, vi)
    for oid, nm in out_names.items():
        n = graph.nodes[oid]
        if n.op in ("input", "const"):                       # an output that is an input / constant: route it through Identity
            g.message(1, encode_node("Identity", [names[oid]], [nm]))
        g.message(12, encode_value_info(nm, n.dtype, n.shape, cfg.dynamic_axes.get(nm)))
    model = ProtobufWriter().int(1, 8).string(2, cfg.producer_name).string(3, cfg.producer_version)
    model.message(7, g).message(8, ProtobufWriter().string(1, "").int(2, cfg.opset_version))
    return model.finish()


def export_ir_graph_to_onnx(graph, path: str, config: OnnxExportConfig | None = None) -> None:
    data = ir_graph_to_onnx(graph, config)
    with open(path, "wb") as f:
        f.write(data)


def export_onnx(model, example_inputs, path: str, config: OnnxExportConfig | None = None) -> None:
    """Trace ``model`` on ``example_inputs`` and write the ONNX file."""
    from ..jit.module import trace

    was_training = getattr(model, "training", False)
    if isinstance(model, nn.Module):
        model.eval()
    try:
        export_ir_graph_to_onnx(trace(model, tuple(example_inputs)), path, config)
    finally:
        if isinstance(model, nn.Module) and was_training:
            model.train()


def export_from_program(program, path: str, config: OnnxExportConfig | None = None) -> None:
    """Export what :func:`ferrotorch_b200.jit.export` froze; its dynamic dimensions become
    ``dim_param`` entries of the ONNX inputs."""
    from ..jit.module import trace

    cfg = config or OnnxExportConfig()
    names = cfg.input_names or ["input_%d" % i for i in range(len(program.meta.input_specs))]
    dyn = dict(cfg.dynamic_axes)
    for nm, spec in zip(names, program.meta.input_specs):
        axes = {k: d.name for k, d in enumerate(spec.shape) if d.is_dynamic()}
        if axes:
            dyn.setdefault(nm, axes)
    cfg = OnnxExportConfig(cfg.opset_version, cfg.model_name, cfg.producer_name, cfg.producer_version, names,
                           cfg.output_names, dyn)
    graph = getattr(program, "ir_graph", None)
    if graph is None:
        raise OnnxExportError("export_from_program: this program carries no IR graph (it was loaded from bytes); "
                              "export the module it came from with export_onnx")
    export_ir_graph_to_onnx(graph, path, cfg)


# --------------------------------------------------------------------------- reading back
@dataclass
class OnnxNode:
    op_type: str
    inputs: list
    outputs: list
    attrs: dict


@dataclass
class OnnxModel:
    ir_version: int
    producer_name: str
    opset_version: int
    graph_name: str
    nodes: list
    initializers: dict
    inputs: list            # (name, dtype, shape) with a str for symbolic dimensions
    outputs: list


def _decode_tensor(data: bytes):
    dims, dt, name, raw = [], ONNX_FLOAT, "", b""
    for f, _, v in read_message(data):
        if f == 1:
            dims.append(v)
        elif f == 2:
            dt = v
        elif f == 8:
            name = v.decode()
        elif f == 9:
            raw = v
    dtype = _DTYPE_INV[dt]
    t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype) if raw else torch.empty(0, dtype=dtype)
    return name, t.reshape(dims)


def _decode_value_info(data: bytes):
    name, dtype, shape = "", torch.float32, []
    for f, _, v in read_message(data):
        if f == 1:
            name = v.decode()
        elif f == 2:
            for f2, _, tt in read_message(v):
                if f2 != 1:
                    continue
                for f3, _, x in read_message(tt):
                    if f3 == 1:
                        dtype = _DTYPE_INV[x]
                    elif f3 == 2:
                        for _, _, dim in read_message(x):
                            d = read_message(dim)
                            shape.append(d[0][2].decode() if d and d[0][0] == 2 else (d[0][2] if d else 0))
    return name, dtype, shape


def _decode_node(data: bytes) -> OnnxNode:
    n = OnnxNode("", [], [], {})
    for f, _, v in read_message(data):
        if f == 1:
            n.inputs.append(v.decode())
        elif f == 2:
            n.outputs.append(v.decode())
        elif f == 4:
            n.op_type = v.decode()
        elif f == 5:
            name, val, ints = "", None, []
            for fa, _, x in read_message(v):
                if fa == 1:
                    name = x.decode()
                elif fa == 2:
                    val = x
                elif fa == 3:
                    val = x - (1 << 64) if x >= 1 << 63 else x
                elif fa == 5:
                    val = _decode_tensor(x)[1]
                elif fa == 8:
                    ints.append(x - (1 << 64) if x >= 1 << 63 else x)
            n.attrs[name] = ints if ints else val
    return n


def load_onnx(data) -> OnnxModel:
    """Parse the subset of ``ModelProto`` this module writes (bytes or a path)."""
    if isinstance(data, str):
        with open(data, "rb") as f:
            data = f.read()
    m = OnnxModel(0, "", 0, "", [], {}, [], [])
    for f, _, v in read_message(data):
        if f == 1:
            m.ir_version = v
        elif f == 2:
            m.producer_name = v.decode()
        elif f == 8:
            for f2, _, x in read_message(v):
                if f2 == 2:
                    m.opset_version = x
        elif f == 7:
            for f2, _, x in read_message(v):
                if f2 == 1:
                    m.nodes.append(_decode_node(x))
                elif f2 == 2:
                    m.graph_name = x.decode()
                elif f2 == 5:
                    name, t = _decode_tensor(x)
                    m.initializers[name] = t
                elif f2 == 11:
                    m.inputs.append(_decode_value_info(x))
                elif f2 == 12:
                    m.outputs.append(_decode_value_info(x))
    if not m.nodes and not m.outputs:
        raise OnnxExportError("not an ONNX model this module can read")
    return m


_EVAL = {
    "Neg": torch.neg, "Relu": torch.relu, "Sigmoid": torch.sigmoid, "Tanh": torch.tanh, "Sqrt": torch.sqrt, "Abs": torch.abs,
    "Exp": torch.exp, "Log": torch.log, "Erf": torch.erf, "Add": torch.add, "Sub": torch.sub, "Mul": torch.mul,
    "Div": torch.div, "Pow": torch.pow, "MatMul": torch.matmul, "Identity": lambda x: x,
}


def _ints(v) -> list[int]:
    return [int(v)] if isinstance(v, int) else [int(x) for x in v]


def run_onnx(model: OnnxModel, *inputs: torch.Tensor) -> list[torch.Tensor]:
    """Evaluate the model with torch operators, following the ONNX operator definitions: a
    reference run for checking an export where no ONNX runtime is installed."""
    if len(inputs) != len(model.inputs):
        raise OnnxExportError("the model takes %d inputs, got %d" % (len(model.inputs), len(inputs)))
    env = dict(model.initializers)
    for (name, dtype, shape), t in zip(model.inputs, inputs):
        if t.dtype != dtype or len(shape) != t.dim() or any(isinstance(d, int) and d != s for d, s in zip(shape, t.shape)):
            raise OnnxExportError("input %s: expected %s %s, got %s %s" % (name, dtype, shape, t.dtype, tuple(t.shape)))
        env[name] = t
    for n in model.nodes:
        xs = [env[i] for i in n.inputs]
        if n.op_type in _EVAL:
            y = _EVAL[n.op_type](*xs)
        elif n.op_type == "Softmax":
            y = torch.softmax(xs[0], dim=n.attrs.get("axis", -1))
        elif n.op_type == "Transpose":
            y = xs[0].permute(*n.attrs["perm"])
        elif n.op_type == "Reshape":
            y = xs[0].reshape([int(v) for v in xs[1].tolist()])
        elif n.op_type in ("ReduceSum", "ReduceMean", "ReduceProd"):
            axes = [int(v) for v in xs[1].tolist()] if len(xs) > 1 else n.attrs.get("axes")
            axes = ([axes] if isinstance(axes, int) else axes) or list(range(xs[0].dim()))
            keep = bool(n.attrs.get("keepdims", 1))
            if n.op_type == "ReduceProd":
                y = xs[0]
                for a in sorted(axes, reverse=True):
                    y = y.prod(a, keepdim=keep)
            else:
                y = (torch.sum if n.op_type == "ReduceSum" else torch.mean)(xs[0], dim=axes, keepdim=keep)
        elif n.op_type == "LogSoftmax":
            y = torch.log_softmax(xs[0], dim=n.attrs.get("axis", -1))
        elif n.op_type == "Squeeze":
            y = xs[0].squeeze() if len(xs) == 1 else xs[0].squeeze(tuple(int(v) for v in xs[1].tolist()))
        elif n.op_type == "Unsqueeze":
            y = xs[0]
            for a in sorted(int(v) for v in xs[1].tolist()):
                y = y.unsqueeze(a)
        elif n.op_type == "Concat":
            y = torch.cat(xs, dim=n.attrs["axis"])
        elif n.op_type == "Gemm":
            a_, b_ = (xs[0].t() if n.attrs.get("transA") else xs[0]), (xs[1].t() if n.attrs.get("transB") else xs[1])
            y = float(n.attrs.get("alpha", 1.0)) * (a_ @ b_)
            if len(xs) > 2:
                y = y + float(n.attrs.get("beta", 1.0)) * xs[2]
        elif n.op_type == "Conv":
            pads = _ints(n.attrs.get("pads", [0, 0, 0, 0]))
            if pads[:2] != pads[2:]:
                raise OnnxExportError("reference evaluator: asymmetric Conv padding")
            y = nn.functional.conv2d(xs[0], xs[1], xs[2] if len(xs) > 2 else None, _ints(n.attrs.get("strides", [1, 1])), pads[:2],
                                     _ints(n.attrs.get("dilations", [1, 1])), int(n.attrs.get("group", 1)))
        elif n.op_type == "BatchNormalization":
            y = nn.functional.batch_norm(xs[0], xs[3], xs[4], xs[1], xs[2], False, 0.0, float(n.attrs.get("epsilon", 1e-5)))
        elif n.op_type in ("MaxPool", "AveragePool"):
            k, st, pads = _ints(n.attrs["kernel_shape"]), _ints(n.attrs.get("strides", [1, 1])), _ints(n.attrs.get("pads", [0, 0, 0, 0]))
            ceil = bool(n.attrs.get("ceil_mode", 0))
            if n.op_type == "MaxPool":
                y = nn.functional.max_pool2d(xs[0], k, st, pads[:2], _ints(n.attrs.get("dilations", [1, 1])), ceil)
            else:
                y = nn.functional.avg_pool2d(xs[0], k, st, pads[:2], ceil, bool(n.attrs.get("count_include_pad", 0)))
        elif n.op_type == "GlobalAveragePool":
            y = xs[0].mean((2, 3), keepdim=True)
        else:
            raise OnnxExportError("reference evaluator: operator %s is not implemented" % n.op_type)
        env[n.outputs[0]] = y
    return [env[name] for name, _, _ in model.outputs]
