"""Graph IR of the JIT and its optimisation passes.

Mirrors the reference's ``IrGraph`` / ``IrOpKind`` (ferrotorch-jit/src/graph.rs:37-172, including
``FusedElementwise{ops}``, ``FusedLinearActivation{activation}`` and ``FusedAttention``) and its
pass pipeline ``constant_fold -> dead_code_eliminate -> fuse_elementwise -> pattern_fuse ->
plan_memory`` (optimize.rs:61, 230, 352, 405, 523; memory_plan.rs).  The fusible op set is the
reference's ``FusedOp`` list (fusion.rs:112-135) plus broadcasting binary inputs.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

import torch

UNARY = ("neg", "relu", "sigmoid", "tanh", "gelu", "silu", "sqrt", "abs", "exp", "log")
BINARY = ("add", "sub", "mul", "div")
SCALAR = ("add_c", "mul_c", "pow_c", "rsub_c", "rdiv_c")  # c on the right: x+c, x*c, x**c, c-x, c/x
ELEMENTWISE = UNARY + BINARY + SCALAR


@dataclass
class Node:
    id: int
    op: str                      # input | const | call | fused_elementwise | fused_linear_act | fused_attention | <elementwise>
    inputs: list[int] = field(default_factory=list)
    attrs: dict = field(default_factory=dict)
    shape: tuple | None = None
    dtype: torch.dtype | None = None


_FUNCTION_HOMES = ("torch", "torch.nn.functional", "operator", "_operator", "torch.linalg", "torch.special", "math")


def _function_reference(fn) -> str | None:
    """``"module:name"`` for a function of torch / operator / math that can be found again by that name."""
    import importlib

    name, mod = getattr(fn, "__name__", None), getattr(fn, "__module__", None)
    if not callable(fn) or name is None:
        return None
    for home in ((mod,) if mod in _FUNCTION_HOMES else ()) + _FUNCTION_HOMES:
        try:
            if getattr(importlib.import_module(home), name, None) is fn:
                return "%s:%s" % (home, name)
        except ImportError:
            continue
    return None


def _resolve_function(ref: str):
    import importlib

    home, name = ref.split(":", 1)
    if home not in _FUNCTION_HOMES:
        raise ValueError("serialised graph names a function outside the allowed modules: %r" % ref)
    return getattr(importlib.import_module(home), name)


class IrGraph:
    def __init__(self):
        self.nodes: dict[int, Node] = {}
        self.order: list[int] = []
        self.outputs: list[int] = []
        self.output_spec = None      # how to rebuild the python return value
        self._next = 0

    def add(self, op: str, inputs=(), **attrs) -> Node:
        n = Node(self._next, op, list(inputs), attrs)
        self._next += 1
        self.nodes[n.id] = n
        self.order.append(n.id)
        return n

    # ---- builder and query calls under the reference's names (ferrotorch-jit/src/graph.rs ``impl IrGraph``).
    # A node here produces exactly one value and the value carries the node's id, so node ids and
    # value ids coincide.
    def add_input(self, shape, dtype: torch.dtype = torch.float32) -> int:
        n = self.add("input", index=sum(1 for i in self.order if self.nodes[i].op == "input"))
        n.shape, n.dtype = tuple(shape), dtype
        return n.id

    add_input_with_dtype = add_input

    def add_constant(self, data, shape=None, dtype: torch.dtype = torch.float32) -> int:
        t = torch.as_tensor(data, dtype=dtype)
        if shape is not None:
            t = t.reshape(tuple(shape))
        n = self.add("const", value=t)
        n.shape, n.dtype = tuple(t.shape), dtype
        return n.id

    add_constant_with_dtype = add_constant

    def add_node(self, op: str, inputs, output_shapes=None, output_dtypes=None, **attrs):
        """Returns ``(node id, [value ids])``; one output per node, so the list has one entry."""
        for i in inputs:
            if i not in self.nodes:
                raise KeyError("add_node(%r): input value %r does not exist" % (op, i))
        if output_shapes is not None and len(output_shapes) != 1:
            raise ValueError("a node produces one value; got %d output shapes" % len(output_shapes))
        if output_dtypes is not None and output_shapes is not None and len(output_dtypes) != len(output_shapes):
            raise ValueError("one dtype per output shape")
        n = self.add(op, inputs, **attrs)
        n.shape = tuple(output_shapes[0]) if output_shapes else None
        n.dtype = output_dtypes[0] if output_dtypes else torch.float32
        return n.id, [n.id]

    add_node_with_dtype = add_node

    def set_outputs(self, values) -> None:
        values = list(values)
        for v in values:
            if v not in self.nodes:
                raise KeyError("set_outputs: value %r does not exist" % (v,))
        self.outputs = values

    def node_count(self) -> int:
        return len(self.order)

    value_count = node_count

    def alloc_node_id(self) -> int:
        i, self._next = self._next, self._next + 1
        return i

    alloc_value_id = alloc_node_id

    def is_constant(self, value_id: int) -> bool:
        return value_id in self.nodes and self.nodes[value_id].op == "const"

    def remove_node(self, node_id: int) -> None:
        """Remove one node and its value; nodes that become dead upstream stay (iterate to a fixed
        point, or run :func:`dead_code_eliminate`).  A node that still has users cannot go."""
        if node_id not in self.nodes:
            raise KeyError(node_id)
        users = [i for i in self.order if node_id in self.nodes[i].inputs]
        if users or node_id in self.outputs:
            raise ValueError("node %d is still used by %s" % (node_id, users or "the graph outputs"))
        del self.nodes[node_id]
        self.order.remove(node_id)

    def topological_order(self) -> list[int]:
        """Node ids such that every node comes after the producers of its inputs (Kahn's algorithm;
        ties in insertion order).  Raises on a cycle."""
        pending = {i: len(set(self.nodes[i].inputs)) for i in self.order}
        users = self.users()
        ready = [i for i in self.order if pending[i] == 0]
        out = []
        while ready:
            i = ready.pop(0)
            out.append(i)
            for u in dict.fromkeys(users[i]):
                pending[u] -= 1
                if pending[u] == 0:
                    ready.append(u)
        if len(out) != len(self.order):
            raise ValueError("the graph has a cycle")
        return out

    def fingerprint(self) -> int:
        """A 64-bit digest of the structure (ops, wiring, shapes, dtypes, scalar attributes, outputs);
        equal for graphs built the same way in any process, which is what an autotune cache keys on."""
        import hashlib

        h = hashlib.blake2b(digest_size=8)
        pos = {i: k for k, i in enumerate(self.order)}

        def canon(v):
            if isinstance(v, (int, float, str, bool, type(None))):
                return v
            if isinstance(v, (list, tuple)):
                return tuple(canon(x) for x in v)
            if isinstance(v, dict):
                return tuple(sorted((str(k), canon(x)) for k, x in v.items()))
            if isinstance(v, Node):
                return ("node", pos.get(v.id, -1))
            if isinstance(v, torch.Tensor):
                return ("tensor", tuple(v.shape), str(v.dtype))
            return ("object", _function_reference(v) or type(v).__name__)

        for i in self.order:
            n = self.nodes[i]
            h.update(repr((n.op, [pos[j] for j in n.inputs], n.shape, str(n.dtype), canon(n.attrs))).encode())
        h.update(repr([pos[o] for o in self.outputs]).encode())
        return int.from_bytes(h.digest(), "little")

    def users(self) -> dict[int, list[int]]:
        u: dict[int, list[int]] = {i: [] for i in self.nodes}
        for i in self.order:
            for j in self.nodes[i].inputs:
                u[j].append(i)
        return u

    def count(self, op: str) -> int:
        return sum(1 for i in self.order if self.nodes[i].op == op)

    def ops(self) -> list[str]:
        return [self.nodes[i].op for i in self.order]

    # ---- serialisation (the reference has a binary IR format; structure only, constants and
    # opaque call targets are referenced by name)
    def to_json(self, strict: bool = False) -> str:
        """``strict``: raise on a value that cannot be found again in another process (a Python object
        that is neither a tensor, a node, plain data nor a named torch / operator function) instead of
        writing a placeholder."""
        def enc(v):
            if isinstance(v, torch.Tensor):
                return {"__tensor__": list(v.shape), "dtype": str(v.dtype)}
            if isinstance(v, Node):
                return {"__node__": v.id}
            if isinstance(v, (int, float, str, bool, type(None))):
                return v
            if isinstance(v, (list, tuple)):
                return [enc(x) for x in v]
            if isinstance(v, dict):
                return {str(k): enc(x) for k, x in v.items()}
            if isinstance(v, torch.dtype):
                return {"__dtype__": str(v)}
            ref = _function_reference(v)
            if ref is not None:
                return {"__fn__": ref}
            if strict:
                raise ValueError("%s object %r" % (type(v).__name__, getattr(v, "__name__", v)))
            return {"__opaque__": getattr(v, "__name__", type(v).__name__)}

        rows = []
        for n in (self.nodes[i] for i in self.order):
            try:
                attrs = enc(n.attrs)
            except ValueError as e:
                raise ValueError("cannot serialise a graph that calls opaque objects: node %d (%s): %s" % (n.id, n.op, e)) from None
            rows.append({"id": n.id, "op": n.op, "inputs": n.inputs, "attrs": attrs,
                         "shape": list(n.shape) if n.shape is not None else None, "dtype": str(n.dtype) if n.dtype is not None else None})
        return json.dumps({"nodes": rows, "outputs": self.outputs})

    @classmethod
    def from_json(cls, text: str, constants: dict | None = None) -> "IrGraph":
        """Rebuild the structure written by :meth:`to_json`.  Tensor constants and opaque call
        targets were saved by name / shape only: pass them back in ``constants`` (node id ->
        attrs to merge); nodes without an entry keep the placeholder dictionaries."""
        d = json.loads(text)
        g = cls()

        def dec(v):
            if isinstance(v, dict):
                if "__fn__" in v:
                    return _resolve_function(v["__fn__"])
                if "__node__" in v:
                    return g.nodes[v["__node__"]]                   # producers come before their users
                if "__dtype__" in v:
                    return getattr(torch, v["__dtype__"].split(".")[-1])
                return {k: dec(x) for k, x in v.items()}
            if isinstance(v, list):
                return tuple(dec(x) for x in v)
            return v

        for nd in d["nodes"]:
            dt = getattr(torch, nd["dtype"].split(".")[-1]) if nd["dtype"] else None
            n = Node(nd["id"], nd["op"], list(nd["inputs"]), dec(nd["attrs"]),
                     tuple(nd["shape"]) if nd["shape"] is not None else None, dt)
            if constants and n.id in constants:
                n.attrs.update(constants[n.id])
            g.nodes[n.id] = n
            g.order.append(n.id)
            g._next = max(g._next, n.id + 1)
        g.outputs = list(d["outputs"])
        return g


    # ---- binary form (the reference's ``IrGraph::serialize`` / ``deserialize``, ferrotorch-jit/src/serialize.rs):
    # ``FTIR``, a version word, the length of the structure, the structure as JSON, then every tensor
    # constant in the state-dict byte layout.  Graphs that still call opaque Python objects cannot be
    # written: their targets do not exist in another process.
    _MAGIC = b"FTIR"

    def serialize(self) -> bytes:
        import struct

        from ..serialize.state import dumps_state_dict

        consts = {}
        for i in self.order:
            for k, v in self.nodes[i].attrs.items():
                if isinstance(v, torch.Tensor):
                    consts["%d.%s" % (i, k)] = v.detach().contiguous()
        js = self.to_json(strict=True).encode()
        return self._MAGIC + struct.pack("<IQ", 1, len(js)) + js + dumps_state_dict(consts)

    @classmethod
    def deserialize(cls, data: bytes) -> "IrGraph":
        import struct

        from ..serialize.state import loads_state_dict

        if len(data) < 16 or data[:4] != cls._MAGIC:
            raise ValueError("not a serialised IR graph (bad magic)")
        version, n = struct.unpack("<IQ", data[4:16])
        if version != 1:
            raise ValueError("IR graph format version %d is not supported" % version)
        if 16 + n > len(data):
            raise ValueError("serialised IR graph is truncated")
        consts: dict = {}
        for name, t in loads_state_dict(bytes(data[16 + n:])).items():
            nid, key = name.split(".", 1)
            consts.setdefault(int(nid), {})[key] = t.clone()
        return cls.from_json(data[16:16 + n].decode(), consts)


# --------------------------------------------------------------------------- passes
def constant_fold(g: IrGraph) -> int:
    """Evaluate elementwise nodes whose inputs are all constants."""
    from .codegen import eval_elementwise

    folded = 0
    for i in list(g.order):
        n = g.nodes[i]
        if n.op in ELEMENTWISE and n.inputs and all(g.nodes[j].op == "const" for j in n.inputs):
            val = eval_elementwise(n.op, [g.nodes[j].attrs["value"] for j in n.inputs], n.attrs.get("c"))
            n.op, n.inputs, n.attrs = "const", [], {"value": val}
            folded += 1
    return folded


def dead_code_eliminate(g: IrGraph) -> int:
    live, stack = set(), list(g.outputs)
    while stack:
        i = stack.pop()
        if i not in live:
            live.add(i)
            stack.extend(g.nodes[i].inputs)
    dead = [i for i in g.order if i not in live and g.nodes[i].op != "input"]
    for i in dead:
        del g.nodes[i]
    g.order = [i for i in g.order if i in g.nodes]
    return len(dead)


def fuse_elementwise(g: IrGraph) -> int:
    """Merge connected elementwise nodes into ``fused_elementwise`` nodes.  A producer joins its
    consumer's group when the consumer is its only user and both produce the same shape."""
    users = g.users()
    group_of: dict[int, int] = {}
    groups: dict[int, list[int]] = {}
    for i in g.order:
        n = g.nodes[i]
        if n.op not in ELEMENTWISE or n.shape is None:
            continue
        gid = None
        for j in n.inputs:
            p = g.nodes[j]
            if j in group_of and len(users[j]) == 1 and j not in g.outputs and p.shape == n.shape:
                if gid is None:
                    gid = group_of[j]
                elif group_of[j] != gid:          # merge two groups feeding one node
                    old = group_of[j]
                    for k in groups.pop(old):
                        group_of[k] = gid
                        groups[gid].append(k)
        if gid is None:
            gid = i
            groups[gid] = []
        groups[gid].append(i)
        group_of[i] = gid
    made = 0
    for gid, members in groups.items():
        if len(members) < 2:
            continue
        members = [i for i in g.order if i in set(members)]
        mset, ext, program = set(members), [], []
        reg = {}
        for i in members:
            n = g.nodes[i]
            srcs = []
            for j in n.inputs:
                if j in mset:
                    srcs.append(("r", reg[j]))
                else:
                    if j not in ext:
                        ext.append(j)
                    srcs.append(("x", ext.index(j)))
            reg[i] = len(program)
            program.append({"op": n.op, "src": srcs, "c": n.attrs.get("c")})
        last = members[-1]
        fused = g.nodes[last]
        fused.op, fused.inputs, fused.attrs = "fused_elementwise", ext, {"program": program}
        for i in members[:-1]:
            del g.nodes[i]
        g.order = [i for i in g.order if i in g.nodes]
        made += 1
    return made


def pattern_fuse(g: IrGraph) -> int:
    """Linear + {relu, gelu, silu, sigmoid, tanh} -> ``fused_linear_act``; ``softmax(q k^T * s) v``
    -> ``fused_attention`` (optimize.rs:523-601)."""
    users, made = g.users(), 0
    for i in list(g.order):
        n = g.nodes.get(i)
        if n is None or n.op not in ("relu", "gelu", "silu", "sigmoid", "tanh") or len(n.inputs) != 1:
            continue
        p = g.nodes[n.inputs[0]]
        if p.op == "call" and p.attrs.get("kind") == "linear" and len(users[p.id]) == 1 and p.id not in g.outputs:
            n.attrs = {"activation": n.op, "kind": "linear", "module": p.attrs.get("module", p.attrs.get("target"))}
            n.op, n.inputs = "fused_linear_act", list(p.inputs)
            del g.nodes[p.id]
            made += 1
    g.order = [i for i in g.order if i in g.nodes]
    users = g.users()
    for i in list(g.order):
        n = g.nodes.get(i)
        if n is None or n.op != "call" or n.attrs.get("kind") != "matmul":
            continue
        sm = g.nodes.get(n.inputs[0])
        if sm is None or sm.op != "call" or sm.attrs.get("kind") != "softmax" or len(users[sm.id]) != 1:
            continue
        sc = g.nodes[sm.inputs[0]]
        scale = 1.0
        if sc.op == "mul_c" and len(users[sc.id]) == 1:
            scale, sc_in = sc.attrs["c"], g.nodes[sc.inputs[0]]
        else:
            sc_in = sc
        if sc_in.op != "call" or sc_in.attrs.get("kind") != "matmul" or len(users[sc_in.id]) != 1:
            continue
        kt = g.nodes[sc_in.inputs[1]]
        if kt.op != "call" or kt.attrs.get("kind") != "transpose_last":
            continue
        q, k, v = sc_in.inputs[0], kt.inputs[0], n.inputs[1]
        for d in {sm.id, sc.id, sc_in.id, kt.id} - {n.id}:
            if d in g.nodes and not [u for u in users[d] if u in g.nodes and u not in (sm.id, sc.id, sc_in.id, n.id)]:
                del g.nodes[d]
        n.op, n.inputs, n.attrs = "fused_attention", [q, k, v], {"scale": scale}
        made += 1
    g.order = [i for i in g.order if i in g.nodes]
    return made


def plan_memory(g: IrGraph) -> dict:
    """Liveness-based buffer assignment: every node output gets a slot, a slot is reused once its
    last user has run.  Returns ``{"slot_of": {node: slot}, "n_slots": k, "peak_bytes": b}``."""
    last_use = {}
    for pos, i in enumerate(g.order):
        for j in g.nodes[i].inputs:
            last_use[j] = pos
    for o in g.outputs:
        last_use[o] = len(g.order)
    free, slot_of, sizes, n_slots, peak, live_bytes = [], {}, {}, 0, 0, 0
    for pos, i in enumerate(g.order):
        n = g.nodes[i]
        if n.op in ("input", "const") or n.shape is None:
            continue
        nbytes = int(torch.tensor(n.shape).prod()) * (torch.empty(0, dtype=n.dtype).element_size() if n.dtype else 4)
        s = free.pop() if free else n_slots
        if s == n_slots:
            n_slots += 1
        slot_of[i], sizes[i] = s, nbytes
        live_bytes += nbytes
        peak = max(peak, live_bytes)
        for j in set(n.inputs):
            if last_use.get(j) == pos and j in slot_of:
                free.append(slot_of[j])
                live_bytes -= sizes[j]
    return {"slot_of": slot_of, "n_slots": n_slots, "peak_bytes": peak}


@dataclass
class OptimizationConfig:
    constant_folding: bool = True
    dead_code_elimination: bool = True
    elementwise_fusion: bool = True
    pattern_fusion: bool = True
    memory_planning: bool = True


def optimize(g: IrGraph, cfg: OptimizationConfig | None = None) -> dict:
    cfg = cfg or OptimizationConfig()
    stats = {}
    if cfg.constant_folding:
        stats["folded"] = constant_fold(g)
    if cfg.dead_code_elimination:
        stats["dead"] = dead_code_eliminate(g)
    if cfg.pattern_fusion:
        stats["patterns"] = pattern_fuse(g)
    if cfg.elementwise_fusion:
        stats["fused_groups"] = fuse_elementwise(g)
    if cfg.dead_code_elimination:
        stats["dead"] = stats.get("dead", 0) + dead_code_eliminate(g)
    if cfg.memory_planning:
        stats["memory"] = plan_memory(g)
    return stats
