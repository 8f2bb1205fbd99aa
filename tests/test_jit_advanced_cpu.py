"""Symbolic shapes + guards, segment-level graph breaks, AOT autograd, exported programs."""
import pytest
import torch
from torch import nn

from ferrotorch_b200 import jit as J


class _Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l = nn.Linear(8, 8)

    def forward(self, x):
        h = torch.tanh(self.l(x)) * 2.0 + 1.0
        return h.reshape(6, 2, 4).sum(1) + h.reshape(h.shape[0], -1).mean()


def test_symbolic_shapes_and_guards():
    torch.manual_seed(0)
    m = _Net().eval()
    sig = J.ShapeSignature().symbolic_dim_with_range(0, 0, 2, 64)
    assert sig.is_symbolic(0, 0) and not sig.is_symbolic(0, 1) and len(sig.symbolic_dims_for(0)) == 1
    sm = J.compile_symbolic(m, (torch.randn(6, 8),), sig)
    assert "fused_elementwise" in sm.inner().graph.ops()
    for rows in (6, 10, 2, 64):
        y = torch.randn(rows, 8)
        h = torch.tanh(m.l(y)) * 2.0 + 1.0
        assert torch.allclose(sm(y), h.reshape(rows, 2, 4).sum(1) + h.mean(), atol=1e-6), rows   # the baked 6 became -1
    for bad, why in ((torch.randn(1, 8), "outside"), (torch.randn(6, 9), "not symbolic"), (torch.randn(6, 8, 1), "rank")):
        with pytest.raises(J.JitError, match=why):
            sm(bad)
    with pytest.raises(J.JitError, match="inputs"):
        sm.guard().check([(6, 8), (6, 8)])
    with pytest.raises(ValueError):
        J.Guard([(6, 8)], J.ShapeSignature().symbolic_dim(0, 5))
    with pytest.raises(ValueError):
        J.ShapeSignature().symbolic_dim_with_range(0, 0, 5, 2)
    # equal sizes by coincidence are left alone: (8, 8) reshaped to (8, 2, 4) keeps its 8
    g = J.trace(lambda t: t.reshape(8, 2, 4), (torch.randn(8, 8),))
    assert J.patch_reshape_for_symbolic_dims(g, [(8, 8)], J.ShapeSignature().symbolic_dim(0, 0)) == 0


class _Dyn(nn.Module):
    def forward(self, x):
        return x * 2 if x.sum() > 0 else x - 1        # data-dependent branch: cannot be traced


def test_graph_breaks_keep_untraceable_stages_eager():
    torch.manual_seed(0)
    seq = nn.Sequential(nn.Linear(4, 4), nn.Tanh(), _Dyn(), nn.Linear(4, 2), nn.ReLU())
    x = torch.randn(3, 4)
    sm = J.trace_with_breaks(seq, x)
    assert sm.segment_count() == 3 and [s.is_compiled() for s in sm.segments()] == [True, False, True]
    assert not sm.is_fully_compiled() and "cannot trace" in sm.segments()[1].reason
    for inp in (x, -x.abs(), x.abs()):                                    # both sides of the branch
        assert torch.allclose(sm(inp), seq(inp), atol=1e-6)
    full = J.trace_with_breaks([nn.Linear(4, 4), torch.sigmoid, lambda t: t * 3.0 + 1.0], x)
    assert full.is_fully_compiled() and full.segment_count() == 1
    assert "fused_elementwise" in full.segments()[0].compiled.graph.ops()


def test_aot_autograd_gradients_match_eager():
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 1))
    x = torch.randn(3, 4)
    am = J.compile_aot(m, (x,))
    assert am.pair.n_params == 4 and am.pair.n_inputs == 1 and am.pair.backward.count("input") == 6
    xa = x.clone().requires_grad_()
    ya = am(xa)
    ya.sum().backward()
    got = [p.grad.clone() for p in m.parameters()] + [xa.grad]
    for p in m.parameters():
        p.grad = None
    xr = x.clone().requires_grad_()
    m(xr).sum().backward()
    want = [p.grad for p in m.parameters()] + [xr.grad]
    assert torch.allclose(ya, m(x), atol=1e-6) and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(got, want))
    # a plain function: the backward graph's elementwise chains are fused kernels as well
    f = lambda a, b: torch.sigmoid(a * b + 1.0) * a            # noqa: E731
    af = J.compile_aot(f, (torch.randn(5), torch.randn(5)))
    assert "fused_elementwise" in af.pair.backward.ops()
    a, b = torch.randn(5, requires_grad=True), torch.randn(5, requires_grad=True)
    af(a, b).sum().backward()
    ga, gb = a.grad.clone(), b.grad.clone()
    a.grad = b.grad = None
    f(a, b).sum().backward()
    assert torch.allclose(ga, a.grad, atol=1e-6) and torch.allclose(gb, b.grad, atol=1e-6)
    # training with the compiled pair moves the loss like eager training does
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    first = None
    for _ in range(20):
        opt.zero_grad()
        loss = (am(x) - 1.0).pow(2).mean()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < 0.5 * first
    with pytest.raises(J.JitError):
        J.compile_aot(lambda t: (t, t), (x,))


def test_exported_program_round_trip_and_guards(tmp_path):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(4, 8), nn.Tanh(), nn.Linear(8, 2)).eval()
    x = torch.randn(3, 4)
    spec = J.InputSpec([J.DimSpec.dynamic_range("batch", 2, 32), J.DimSpec.static(4)])
    assert spec.has_dynamic_dims() and spec.rank() == 2 and not J.InputSpec.all_static((3, 4)).has_dynamic_dims()
    ep = J.export(m, (x,), [spec])
    assert torch.allclose(ep(x), m(x)) and ep.run(torch.randn(7, 4)).shape == (7, 2)
    path = tmp_path / "model.ftep"
    ep.save(str(path))
    back = J.ExportedProgram.load(str(path))
    y = torch.randn(9, 4)
    assert torch.allclose(back(y), m(y), atol=1e-6) and back.meta.ir_ops == ["input", "call", "tanh", "call"]
    assert back.meta.output_shape == [3, 2] and back.meta.input_dtypes == ["torch.float32"]
    meta = J.ExportedProgram.parse_json_metadata(back.to_json())
    assert meta.input_specs[0].shape[0] == J.DimSpec(name="batch", min=2, max=32)
    for bad, why in ((torch.randn(1, 4), "outside"), (torch.randn(3, 5), "exported as 4"),
                     (torch.randn(3, 4).double(), "dtype"), (torch.randn(3, 4, 1), "rank")):
        with pytest.raises(J.JitError, match=why):
            back(bad)
    with pytest.raises(J.JitError, match="inputs"):
        back(x, x)
    static = J.export(m, (x,))
    with pytest.raises(J.JitError):
        static(torch.randn(4, 4))
    for junk in (b"nope", b"FTEP1\n" + (1 << 40).to_bytes(8, "little") + b"{}"):
        with pytest.raises(J.JitError):
            J.ExportedProgram.deserialize(junk)
    with pytest.raises(J.JitError):
        J.ExportedProgram.parse_json_metadata("{}")
    with pytest.raises(J.JitError):
        J.export(m, (x,), [J.InputSpec.all_static((5, 4))])
