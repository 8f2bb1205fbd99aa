"""JIT: tracing, passes, generated source (NVRTC-compiled without a GPU), and GPU numerics."""
import pytest
import torch
from torch import nn

from ferrotorch_b200 import jit as J


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc = nn.Linear(16, 32)
        self.scale = nn.Parameter(torch.full((32,), 0.5))

    def forward(self, x, y):
        h = torch.relu(self.fc(x))
        z = torch.sigmoid(h * self.scale + y) * 2.0 - h.exp().neg()
        unused = z.tanh()  # dead  # noqa: F841
        return torch.sqrt(z.abs() + 1.0)


def test_trace_passes_and_parity_cpu():
    torch.manual_seed(0)
    m, x, y = Block(), torch.randn(4, 16), torch.randn(4, 32)
    g = J.trace(m, (x, y))
    assert g.count("input") == 2 and "relu" in g.ops() and "tanh" in g.ops()
    c = J.compile(m, (x, y))
    ops = c.graph.ops()
    assert "tanh" not in ops, "dead code must be eliminated"
    assert "fused_linear_act" in ops and ops.count("fused_elementwise") == 1
    assert not any(o in ops for o in ("sigmoid", "exp", "sqrt", "abs", "mul", "add"))
    assert c.stats["memory"]["n_slots"] >= 1 and c.stats["memory"]["peak_bytes"] > 0
    assert torch.allclose(c(x, y), m(x, y), atol=1e-6)
    # guard: another batch size falls back to eager and still gives the right answer
    x2, y2 = torch.randn(2, 16), torch.randn(2, 32)
    assert torch.allclose(c(x2, y2), m(x2, y2)) and c.guard_failures == 1
    strict = J.compile(m, (x, y), J.CompileConfig(fallback_to_eager=False))
    with pytest.raises(J.JitError):
        strict(x2, y2)
    assert '"fused_elementwise"' in c.graph.to_json()


def test_constant_folding_and_attention_pattern():
    g = J.IrGraph()
    x = g.add("input", index=0)
    a = g.add("const", value=torch.tensor([1.0, 2.0]))
    b = g.add("mul_c", [a.id], c=3.0)
    c_ = g.add("add_c", [b.id], c=1.0)
    out = g.add("add", [x.id, c_.id])
    g.outputs = [out.id]
    assert J.constant_fold(g) == 2 and J.dead_code_eliminate(g) == 2
    assert torch.equal(g.nodes[c_.id].attrs["value"], torch.tensor([4.0, 7.0])) and g.ops() == ["input", "const", "add"]

    def attn(q, k, v):
        return torch.matmul(torch.softmax(torch.matmul(q, k.transpose(-1, -2)) * 0.25, dim=-1), v)

    q, k, v = (torch.randn(2, 3, 5, 16) for _ in range(3))
    c = J.compile(attn, (q, k, v))
    assert "fused_attention" in c.graph.ops() and "softmax" not in [n.attrs.get("kind") for n in c.graph.nodes.values()]
    assert torch.allclose(c(q, k, v), attn(q, k, v), atol=1e-5)


def test_graph_break_falls_back_to_eager():
    def data_dependent(x):
        return x * 2 if float(x.sum()) > 0 else x - 1

    c = J.compile(data_dependent, (torch.ones(3),))
    assert isinstance(c, J.EagerFallback) and torch.equal(c(torch.ones(3)), torch.full((3,), 2.0))
    with pytest.raises(J.JitError):
        J.compile(data_dependent, (torch.ones(3),), J.CompileConfig(fallback_to_eager=False))


def test_apply_fused_and_script_cpu():
    x = torch.randn(100)
    got = J.apply_fused([("mul_c", 2.0), "relu", ("add_c", 1.0), "log", ("pow_c", 2.0)], x)
    assert torch.allclose(got, torch.log(torch.relu(x * 2) + 1) ** 2, atol=1e-6)

    @J.script
    def f(a, b):
        return (a - b).abs() / (b.exp() + 1.0)

    a, b = torch.randn(8), torch.randn(8)
    assert torch.allclose(f(a, b), (a - b).abs() / (b.exp() + 1.0), atol=1e-6)


def test_generated_source_compiles_for_sm_100a():
    prog = [{"op": "mul", "src": [("x", 0), ("x", 1)], "c": None}, {"op": "add", "src": [("r", 0), ("x", 2)], "c": None},
            {"op": "gelu", "src": [("r", 1)], "c": None}, {"op": "pow_c", "src": [("r", 2)], "c": 2.0}]
    for dt, vec in ((torch.bfloat16, 8), (torch.float32, 4), (torch.float16, 1)):
        src = J.generate_source(prog, [dt, dt, torch.float32], ["full", "row", "scalar"], dt, vec, "k")
        assert "erff" in src and "powf" in src
        cubin = J.compile_cubin(src, "k")
        assert cubin[:4] == b"\x7fELF"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_kernel_numerics_gpu(dtype):
    from ferrotorch_b200 import _native
    from ferrotorch_b200.jit import codegen

    torch.manual_seed(1)
    m = Block().cuda().to(dtype)
    x, y = torch.randn(64, 16, device="cuda", dtype=dtype), torch.randn(64, 32, device="cuda", dtype=dtype)
    with torch.no_grad():
        c = J.compile(m, (x, y))
        before, compiled = _native.launch_count(), codegen.compile_count
        got = c(x, y)
        torch.cuda.synchronize()
        want = m.float()(x.float(), y.float())
    assert _native.launch_count() > before and codegen.compile_count == compiled + 1
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(got.float(), want, atol=tol, rtol=tol)
    z = torch.randn(1001, device="cuda", dtype=dtype)  # odd length: scalar-width kernel
    got = J.apply_fused([("mul_c", 0.5), "tanh", ("add_c", 2.0), "sqrt"], z)
    assert torch.allclose(got.float(), torch.sqrt(torch.tanh(z.float() * 0.5) + 2.0), atol=tol, rtol=tol)


def test_ir_json_round_trip():
    import torch

    from ferrotorch_b200.jit.ir import IrGraph, dead_code_eliminate, fuse_elementwise

    g = IrGraph()
    a, b = g.add("input", name="a"), g.add("input", name="b")
    c = g.add("const", value=torch.ones(4))
    s = g.add("add", [a.id, b.id])
    m = g.add("mul", [s.id, c.id])
    r = g.add("relu", [m.id])
    g.add("neg", [a.id])                      # dead
    g.outputs = [r.id]
    text = g.to_json()
    h = IrGraph.from_json(text, constants={c.id: {"value": torch.ones(4)}})
    assert h.ops() == g.ops() and h.outputs == g.outputs
    assert [h.nodes[i].inputs for i in h.order] == [g.nodes[i].inputs for i in g.order]
    assert torch.equal(h.nodes[c.id].attrs["value"], torch.ones(4))
    assert dead_code_eliminate(h) == dead_code_eliminate(g)
    assert fuse_elementwise(h) == fuse_elementwise(g)
    assert h.ops() == g.ops()
    assert IrGraph.from_json(h.to_json()).ops() == h.ops()
