"""JIT back-ends: interpreter / native / inductor agree with eager, LoopIR lowering, fused chains,
generated reduction source compiles for sm_100a."""
import pytest
import torch
from torch import nn

from ferrotorch_b200 import jit
from ferrotorch_b200.jit import backends as B


def _graph():
    def fn(x, y):
        h = torch.relu(x * 2.0 + y)
        return torch.sigmoid(h) * y, h.exp()

    x, y = torch.randn(6, 8), torch.randn(8)
    g = jit.trace(fn, (x, y))
    jit.optimize(g)
    return fn, g, (x, y)


def test_backends_agree_with_eager():
    fn, g, ins = _graph()
    ref = fn(*ins)
    assert g.count("fused_elementwise") >= 1
    for be in (B.InterpreterBackend(), B.NativeBackend(), B.InductorBackend(B.InductorTarget.CpuTorch),
               B.InductorBackend(B.InductorTarget.GpuCuda)):
        cg = be.compile(g)
        outs = cg(ins)
        assert cg.backend == be.name and len(outs) == 2
        for o, r in zip(outs, ref):
            torch.testing.assert_close(o, r, rtol=1e-5, atol=1e-6)
    ind = B.InductorBackend(B.InductorTarget.CpuTorch)
    cg = ind.compile(g)
    assert ind.status is B.InductorCompileStatus.Compiled and all(s.startswith("def fused_") for s in cg.sources.values())
    cuda = B.InductorBackend(B.InductorTarget.GpuCuda).compile(g)
    assert all("__global__" in s for s in cuda.sources.values())
    torch.testing.assert_close(B.interpret_multi(g, ins)[1], ref[1])
    with pytest.raises(jit.JitError):
        B.interpret(g, ins)
    outs, caps = B.interpret_multi_with_captures(g, ins, [g.outputs[0]])
    torch.testing.assert_close(caps[0], outs[0])
    plan = B.MemoryPlan.of(g)
    assert plan.n_slots >= 1 and plan.peak_bytes > 0 and plan.reuse_count() >= 0


def test_graph_without_fusion_and_with_a_module():
    net = nn.Sequential(nn.Linear(8, 4), nn.Tanh())
    g = jit.trace(net, (torch.randn(3, 8),))
    x = torch.randn(3, 8)
    ref = net(x)
    for be in (B.NativeBackend(), B.InductorBackend()):
        torch.testing.assert_close(be.compile(g)([x])[0], ref)
    m = B.compile_with_config(net, (x,), jit.CompileConfig())
    torch.testing.assert_close(m(x), ref)


def test_loop_ir_and_fused_chain():
    ch = B.FusedChain().push(B.FusedOp.MulScalar, 0.5).push(B.FusedOp.Tanh).push(B.FusedOp.AddScalar, 1.0).push(B.FusedOp.Abs)
    assert len(ch) == 4
    x = torch.randn(1000)
    ref = (torch.tanh(x * 0.5) + 1.0).abs()
    torch.testing.assert_close(ch.execute(x), ref)
    ir = ch.loop_ir()
    assert ir.n_inputs == 1 and ir.body.depth() == 5 and ir.body.loads() == {0}
    torch.testing.assert_close(B.CpuCodegen().compile(ir)(x), ref)
    src = B.GpuCodegen().generate(ir, "k")
    assert 'extern "C" __global__ void k(' in src and "fabsf" in src
    assert "__global__" in ch.generate_source(torch.bfloat16, 8)
    with pytest.raises(jit.JitError):
        B.FusedChain().push(B.FusedOp.Relu, 1.0)
    with pytest.raises(jit.JitError):
        B.FusedChain().push(B.FusedOp.PowScalar)
    with jit.with_fusion(False):
        assert not B.is_fusion_enabled()
        torch.testing.assert_close(ch.execute(x), ref)
    assert B.is_fusion_enabled()
    assert B.estimate_numel_for_inputs([(4, 1, 8), (3, 1), ()]) == 96
    prog = [{"op": "mul", "src": [("x", 0), ("x", 1)], "c": None}, {"op": "rsub_c", "src": [("r", 0)], "c": 2.0},
            {"op": "div", "src": [("r", 1), ("x", 0)], "c": None}]
    a, b = torch.rand(5) + 1, torch.rand(5)
    torch.testing.assert_close(B.CpuCodegen().compile(B.LoopIR.from_program(prog, 2))(a, b), (2.0 - a * b) / a)


def test_generated_sources_compile_for_sm_100a():
    ch = B.FusedChain().push(B.FusedOp.Exp)
    x = torch.randn(7, 33)
    for kind in B.ReductionKind:
        src = B.generate_reduction_source(kind, ch, "red_" + kind.value)
        try:
            cubin = jit.compile_cubin(src, "red_" + kind.value)
        except Exception as e:                                   # no NVRTC in this environment
            pytest.skip("NVRTC unavailable: %s" % e)
        assert len(cubin) > 500
        ref = B.reduce_reference(kind, x, ch)
        assert ref.shape == (7,)
    torch.testing.assert_close(B.reduce_reference(B.ReductionKind.Mean, x), x.mean(-1))
    src, cubin = B.compile_loop_ir_kernel(ch.loop_ir(), "loop_k")
    assert "loop_k" in src and len(cubin) > 500


def test_remaining_reference_names():
    fn, g, ins = _graph()
    groups = B.FusionGroup.of(g)
    assert groups and all(gr.kind is B.FusionGroupKind.Elementwise and gr.n_ops >= 2 for gr in groups)
    assert B.estimate_matmul_dims([(4, 3, 8), (8, 5)]) == (12, 5, 8)
    with pytest.raises(jit.JitError):
        B.estimate_matmul_dims([(3, 8), (7, 5)])
    net = nn.Sequential(nn.Linear(8, 4), nn.ReLU())
    x = torch.randn(3, 8)
    m = jit.compile(net, (x,))
    cache = {}
    r = B.autotune(m, (x,), cache=cache)
    assert r.best.block_size == m.cfg.block_size and B.autotune(m, (x,), cache=cache) is r and r.key == B.AutotuneKey.of(m)
    prog = B.export_with_dynamic_shapes(net, (x,), {0: {0: "batch"}})
    assert prog.meta.input_specs[0].has_dynamic_dims() and prog.run(torch.randn(5, 8)).shape == (5, 4)
    ch = B.FusedChain().push(B.FusedOp.Exp)
    src = B.generate_reduction_rust(B.ReductionKind.Sum, ch, "r")
    scope = {"torch": torch}
    exec(src, scope)
    t = torch.randn(3, 7)
    torch.testing.assert_close(scope["r"](t), t.exp().sum(-1))
    assert "__global__" in B.generate_reduction_ptx(B.ReductionKind.Max) and jit.AotCompiledModule is jit.AotModule
