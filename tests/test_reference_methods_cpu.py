"""Method-level parity: classes that share a name with a reference type answer the reference's
method names with the reference's meaning (each block cites the file whose ``impl`` it follows)."""
import json
import threading

import pytest
import torch

from ferrotorch_b200 import optim as O
from ferrotorch_b200 import profiler as P
from ferrotorch_b200 import train as T


def test_exponential_moving_average_methods():
    # ferrotorch-optim/src/ema.rs:93-400
    m = torch.nn.Linear(3, 2)
    w0 = m.weight.detach().clone()
    e = O.ExponentialMovingAverage(list(m.parameters()), 0.9).with_foreach().with_decay_warmup(True)
    assert e.num_updates() == 0 and e.decay == 0.9
    with torch.no_grad():
        m.weight += 1
    e.update()
    assert e.num_updates() == 1 and abs(e.effective_decay() - 2 / 11) < 1e-12          # min(0.9, (1 + 1) / (10 + 1))
    torch.testing.assert_close(e.shadow_values(0), w0 * (2 / 11) + (w0 + 1) * (9 / 11))
    assert len(e.shadow_params()) == 2
    e.apply_shadow()
    torch.testing.assert_close(m.weight.detach(), e.shadow_values(0))
    e.restore()
    torch.testing.assert_close(m.weight.detach(), w0 + 1)
    other = torch.nn.Linear(3, 2)
    e.apply_shadow(list(other.parameters()))                                           # an explicit parameter list
    torch.testing.assert_close(other.weight.detach(), e.shadow_values(0))
    with pytest.raises(ValueError):
        e.update(list(m.parameters())[:1])
    with pytest.raises(IndexError):
        e.shadow_values(2)
    with pytest.raises(ValueError):
        O.ExponentialMovingAverage(m, 1.5)
    plain = O.ExponentialMovingAverage(m, 0.5)                                          # a module works too; no warm-up
    plain.update()
    assert plain.effective_decay() == 0.5


def test_averaged_model_methods():
    # ferrotorch-optim/src/swa.rs:133-400
    m = torch.nn.Linear(3, 2)
    w0 = m.weight.detach().clone()
    a = O.AveragedModel.from_module(m, O.AveragingStrategy.Swa).with_foreach()
    for _ in range(2):
        with torch.no_grad():
            m.weight += 2
        a.update_parameters_from_module(m)
    assert int(a.n_averaged) == 2 and a.strategy() is O.AveragingStrategy.Swa
    torch.testing.assert_close(a.averaged_values(0), w0 + 3)                            # mean of w0 + 2 and w0 + 4
    assert len(a.averaged_params()) == 2
    m2 = torch.nn.Linear(3, 2)
    a.apply_to_module(m2)
    torch.testing.assert_close(m2.weight.detach(), w0 + 3)
    m3 = torch.nn.Linear(3, 2)
    a.apply_to(m3.parameters())
    torch.testing.assert_close(m3.bias.detach(), m.bias.detach())
    ema = O.AveragedModel(m, strategy=(O.AveragingStrategy.Ema, 0.5))
    ema.update_parameters(m)                                                            # first update copies
    with torch.no_grad():
        m.weight += 2
    ema.update_parameters(m)
    torch.testing.assert_close(ema.averaged_values(0), w0 + 5)                          # 0.5 * (w0 + 4) + 0.5 * (w0 + 6)
    with pytest.raises(ValueError):
        a.apply_to(list(m.parameters())[:1])
    with pytest.raises(ValueError):
        O.AveragedModel(m, strategy=(O.AveragingStrategy.Ema, 2.0))
    assert torch.equal(a(torch.ones(1, 3)), a.module(torch.ones(1, 3)))                 # still torch's callable wrapper


def test_training_history_methods():
    # ferrotorch-train/src/history.rs:158-210
    h = T.TrainingHistory()
    assert h.is_empty() and h.len() == 0 and h.best_val_loss() is None and h.best_train_loss() is None
    h.push(T.EpochResult(0, {"loss": 2.0}, {"loss": 2.5}))
    h.push(T.EpochResult(1, {"loss": 1.0}))
    h.push(T.EpochResult(2, {"loss": 1.5}, {"loss": 1.2}))
    assert len(h) == 3 and h.train_losses() == [2.0, 1.0, 1.5] and h.val_losses() == [2.5, None, 1.2]
    assert h.best_train_loss() == (1, 1.0) and h.best_val_loss() == (2, 1.2)


def test_profile_schedule_profiler_and_report_methods(tmp_path):
    # ferrotorch-profiler/src/schedule.rs:138-240, profiler.rs:121-330, report.rs:94-560
    calls = []
    s = P.ProfileSchedule(1, 1, 2, 2)
    s.set_on_trace_ready(calls.append)
    phases = [s.phase()] + [s.step() for _ in range(9)]
    assert phases == ["wait", "warmup", "active", "active", "wait", "warmup", "active", "active", "done", "done"]
    assert calls == [0, 1] and s.current_step() == 9 and s.current_cycle() == 2 and not s.is_active()
    pr = P.Profiler(P.ProfileConfig(cuda_events=False))
    with pr.scope("mm", shapes=[(4, 8), (8, 16)], op="matmul"):
        pass
    pr.record_with_duration("x", "manual", 12.0)
    pr.record_memory_categorized("w", 1000, P.MemoryCategory.PARAMETERS)
    pr.record_memory_categorized("a", 500, P.MemoryCategory.ACTIVATIONS)
    pr.record_memory_categorized("a", -200, P.MemoryCategory.ACTIVATIONS)
    assert pr.is_active() and pr.pending_cuda_count() == 0
    pr.flush_cuda_kernels()
    pr.stop()
    pr.record_with_duration("late", "manual", 5.0)
    pr.record_memory_categorized("late", 7, P.MemoryCategory.OTHER)
    assert not pr.is_active() and [e.name for e in pr.events] == ["mm", "x"]
    r = pr.report()
    assert r.total_flops() == 2 * 4 * 8 * 16 and r.flops_per_second() > 0
    assert r.memory_by_category() == [("parameters", 1000), ("activations", 300)]
    assert not r.has_gpu_events() and not r.has_stack_traces()
    assert [o.name for o in r.top_ops(5)] == ["x", "mm"] or [o.name for o in r.top_ops(5)] == ["mm", "x"]
    assert abs(r.total_time_us() - sum(e.dur_us for e in r.events)) < 1e-6
    path = r.save_tensorboard_trace(str(tmp_path), None, "nodeA")
    assert path.endswith("plugins/profile/run0/nodeA.pt.trace.json") and "traceEvents" in json.load(open(path))
    assert r.save_tensorboard_trace(str(tmp_path), "second").startswith(str(tmp_path / "plugins" / "profile" / "second"))
    # a schedule driven through the profiler still hands the profiler to its callback
    seen = []
    pr2 = P.Profiler(P.ProfileConfig(cuda_events=False), P.ProfileSchedule(0, 0, 1, 2, on_trace_ready=seen.append))
    for _ in range(3):
        pr2.step()
    assert seen == [pr2, pr2, pr2][:len(seen)] and len(seen) >= 2


def test_device_mesh_and_mesh_tensor_methods():
    # ferrotorch-distributed/src/device_mesh.rs:48-203, dtensor.rs:88-230
    from ferrotorch_b200.parallel import DeviceMesh, DTensor, Partial, Replicate, Shard
    from ferrotorch_b200.parallel.backend import SimulatedGroup

    mesh = DeviceMesh.new_with_names([2, 2], ["dp", "tp"], 4)
    assert (mesh.ndim, mesh.size, mesh.shape, mesh.dim_index("tp")) == (2, 4, (2, 2), 1)
    for bad in (lambda: DeviceMesh.new([2, 2], 6), lambda: DeviceMesh.new_with_names([2, 2], ["a", "a"], 4), lambda: mesh.dim_index("pp")):
        with pytest.raises(ValueError):
            bad()
    world = SimulatedGroup.create_group(4)
    full = torch.arange(48.0).reshape(8, 6)
    res = {}

    def run(r):
        groups = [mesh.subgroup(world[r], d) for d in range(2)]
        c = mesh.coords(r)
        local = full.chunk(2, 0)[c[0]].chunk(2, 1)[c[1]].contiguous()
        t = DTensor.from_local(local, mesh, [Shard(0), Shard(1)], groups=groups)
        assert t.shape == (8, 6) and t.numel() == 48 and t.placements == [Shard(0), Shard(1)] and t.mesh is mesh
        assert t.to_local() is local
        a = t.redistribute([Replicate(), Shard(1)])
        b = a.redistribute([Shard(1), Replicate()])             # tensor dim 1 handed from mesh dim 1 to mesh dim 0
        p = DTensor.from_local(torch.ones(2, 2) * (r + 1), mesh, [Partial(), Replicate()], groups=groups)
        rep = DTensor.from_local_replicated(full, mesh, groups=groups).redistribute([Shard(0), Shard(1)])
        res[r] = (a.local, b.local, b.full_tensor(), p.redistribute([Replicate(), Replicate()]).local, rep.local, local)

    ts = [threading.Thread(target=run, args=(r,)) for r in range(4)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    for r in range(4):
        c = mesh.coords(r)
        a, b, f, p, rep, local = res[r]
        assert torch.equal(a, full.chunk(2, 1)[c[1]]) and torch.equal(b, full.chunk(2, 1)[c[0]]) and torch.equal(f, full)
        assert float(p[0, 0]) == (4.0 if c[1] == 0 else 6.0) and torch.equal(rep, local)
    # without groups the placement list is rewritten and nothing moves, as in the reference
    meta = DTensor.from_local(full, mesh, [Replicate(), Replicate()]).redistribute([Shard(0), Replicate()])
    assert meta.placements == [Shard(0), Replicate()] and meta.to_local() is full
    for bad in (lambda: DTensor.from_local(full, mesh, [Replicate()]), lambda: DTensor.from_local(full, mesh, [Shard(0), Shard(0)]),
                lambda: DTensor.from_local(full, mesh, [Shard(2), Replicate()]), lambda: meta.redistribute([Shard(5), Replicate()])):
        with pytest.raises(ValueError):
            bad()
    one = DTensor(full.chunk(2, 0)[0], world[0].__class__.create_group(1)[0], Replicate())
    assert one.shape == (4, 6) and one.numel() == 24 and one.placements == [Replicate()] and one.to_local().shape == (4, 6)


def test_memory_guard_methods():
    # ferrotorch-gpu/src/memory_guard.rs:356-770
    from ferrotorch_b200.utils.memory_guard import MemoryBudgetExceeded, MemoryGuard, OomPolicy

    class FakeAllocator:
        def __init__(self, total):
            self.total, self.used, self.device = total, 0, 3

        def used_bytes(self):
            return self.used

        def total_bytes(self):
            return self.total

        def empty_cache(self):
            pass

    a = FakeAllocator(1000)
    g = MemoryGuard(a, policy=OomPolicy.FAIL)
    seen = []
    g.on_oom(lambda: seen.append("oom"))
    t = g.safe_alloc_copy([1.0, 2.0, 3.0])
    assert t.tolist() == [1.0, 2.0, 3.0] and g.device_ordinal() == 3 and g.device().type == "cpu" and g.device_arc() == g.device()
    a.used = 990
    with pytest.raises(MemoryBudgetExceeded):
        g.safe_alloc((100,))                                    # policy Fail: hooks are not consulted
    assert seen == ["oom"]

    def hook(need):
        a.used = 0
        return 990

    g.register_hook(hook)
    with pytest.raises(MemoryBudgetExceeded):
        g.safe_alloc((100,))
    a.used = 990
    assert g.safe_alloc_with_hooks((100,)).shape == (100,) and g.policy == OomPolicy.FAIL       # hooks ran for this call only
    assert g.free(t) == 12 and t.numel() == 0


def test_ir_graph_builder_and_backend_autotuner():
    # ferrotorch-jit/src/graph.rs ``impl IrGraph``; autotune.rs ``impl Autotuner``
    from ferrotorch_b200 import jit as J
    from ferrotorch_b200.jit.backends import InterpreterBackend, NativeBackend, interpret
    from ferrotorch_b200.jit.ir import IrGraph

    def build():
        g = IrGraph()
        a, b = g.add_input([2, 3]), g.add_input_with_dtype([2, 3], torch.float32)
        c = g.add_constant([2.0] * 6, [2, 3])
        _, (v1,) = g.add_node("add", [a, b], [[2, 3]])
        _, (v2,) = g.add_node("mul", [v1, c], [[2, 3]])
        _, (v3,) = g.add_node_with_dtype("relu", [v2], [[2, 3]], [torch.float32])
        dead, _ = g.add_node("neg", [v1], [[2, 3]])
        g.set_outputs([v3])
        return g, dead

    g, dead = build()
    assert g.node_count() == g.value_count() == 7 and g.is_constant(2) and not g.is_constant(0) and not g.is_constant(99)
    order = g.topological_order()
    assert sorted(order) == list(range(7)) and all(order.index(i) < order.index(n) for n in order for i in g.nodes[n].inputs)
    assert g.fingerprint() == build()[0].fingerprint()                       # same construction, same digest
    x, y = torch.randn(2, 3), torch.randn(2, 3)
    torch.testing.assert_close(interpret(g, [x, y]), torch.relu((x + y) * 2))
    before = g.fingerprint()
    g.remove_node(dead)
    assert g.node_count() == 6 and g.fingerprint() != before
    with pytest.raises(ValueError):
        g.remove_node(3)                                                     # still feeds the multiply
    with pytest.raises(KeyError):
        g.add_node("add", [0, 42], [[2, 3]])
    with pytest.raises(KeyError):
        g.set_outputs([42])
    assert g.alloc_node_id() == 7 and g.alloc_value_id() == 8
    cyc = IrGraph()
    p = cyc.add_input([1])
    _, (q,) = cyc.add_node("neg", [p], [[1]])
    cyc.nodes[p].inputs.append(q)
    with pytest.raises(ValueError):
        cyc.topological_order()

    class Broken(InterpreterBackend):
        def compile(self, graph):
            raise RuntimeError("cannot take this graph")

    tuner = (J.Autotuner().with_candidate("interpreter", InterpreterBackend()).with_candidate("native", NativeBackend())
             .with_candidate("broken", Broken()).with_iterations(3).with_warmup(1))
    assert (tuner.iterations(), tuner.warmup(), tuner.candidate_count(), tuner.cache_size()) == (3, 1, 3, 0)
    key = tuner.key_of(g, [x, y])
    assert tuner.cached(key) is None
    res = tuner.tune(g, [x, y])
    assert res.winner in ("interpreter", "native") and not res.from_cache and set(n for n, _ in res.all_timings) == {"interpreter", "native"}
    assert "broken" in res.failed and res.median_s == min(t for _, t in res.all_timings)
    torch.testing.assert_close(res.compiled.execute([x, y])[0], torch.relu((x + y) * 2))
    assert tuner.cache_size() == 1 and tuner.cached(key)[0] == res.winner
    again = tuner.tune(g, [x, y])
    assert again.from_cache and [n for n, _ in again.all_timings] == [res.winner]        # only the winner is timed again
    assert tuner.tune(g, [torch.randn(2, 3, dtype=torch.float64), y.double()]).from_cache is False     # another signature
    tuner.clear_cache()
    assert tuner.cache_size() == 0
    with pytest.raises(J.JitError):
        J.Autotuner().tune(g, [x, y])
    with pytest.raises(J.JitError):
        J.Autotuner().with_candidate("broken", Broken()).tune(g, [x, y])


def test_kfac_preconditioner_equals_the_dense_kronecker_fisher_and_trains():
    # ferrotorch-optim/src/natural_gradient.rs: F_W ~ A (x) G, natural gradient = G_d^-1 grad A_d^-1
    torch.manual_seed(0)
    lin = torch.nn.Linear(5, 3)
    a, g = torch.randn(16, 5), torch.randn(16, 3)
    opt = O.Kfac(lin.parameters(), lr=0.1, damping=0.05, momentum=0.0, stat_decay=0.5, update_freq=1)
    opt.update_factors(lin.weight, a, g)
    A, G = a.t() @ a / 16, g.t() @ g / 16
    grad = torch.randn(3, 5)
    # row-major vec: (G_d^-1 (x) A_d^-1) vec(grad) = vec(G_d^-1 grad A_d^-1)
    dense = torch.kron(G + 0.05 * torch.eye(3), A + 0.05 * torch.eye(5))
    want = torch.linalg.solve(dense, grad.reshape(-1)).reshape(3, 5)
    torch.testing.assert_close(opt.preconditioned(lin.weight, grad, 0.05), want, rtol=1e-4, atol=1e-5)
    # the first update seeds, later ones blend with stat_decay
    a2, g2 = torch.randn(16, 5), torch.randn(16, 3)
    opt.update_factors(lin.weight, a2, g2)
    torch.testing.assert_close(opt._factors[id(lin.weight)]["A"], 0.5 * A + 0.5 * (a2.t() @ a2 / 16))
    # a step: the weight moves along the preconditioned gradient, the bias (no factors) along the plain one
    w0, b0 = lin.weight.detach().clone(), lin.bias.detach().clone()
    lin.weight.grad, lin.bias.grad = grad.clone(), torch.ones(3)
    pre = opt.preconditioned(lin.weight, grad, 0.05)
    opt.step()
    torch.testing.assert_close(lin.weight.detach(), w0 - 0.1 * pre)
    torch.testing.assert_close(lin.bias.detach(), b0 - 0.1)
    with pytest.raises(ValueError):
        opt.update_factors(lin.weight, a[:, :4], g)
    with pytest.raises(ValueError):
        opt.update_factors(lin.weight, a[0], g[0])
    # hooks: factors of every Linear are collected during forward / backward; the loss goes down
    torch.manual_seed(1)
    net = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh(), torch.nn.Linear(8, 2))
    x, y = torch.randn(64, 6), torch.randn(64, 2)
    cfg = O.KfacConfig().with_lr(0.05).with_damping(1e-2).with_momentum(0.5).with_update_freq(2).with_weight_decay(1e-4)
    k = cfg.build(net.parameters()).watch(net)
    losses = []
    for _ in range(25):
        k.zero_grad()
        loss = torch.nn.functional.mse_loss(net(x), y)
        loss.backward()
        k.step()
        losses.append(float(loss.detach()))
    assert len(k._factors) == 2 and losses[-1] < 0.6 * losses[0]
    k.unwatch()
    # maximize climbs
    p = torch.nn.Parameter(torch.tensor([1.0]))
    up = O.Kfac([p], lr=0.1, momentum=0.0, maximize=True)
    p.grad = torch.tensor([2.0])
    up.step()
    assert float(p.detach()) == pytest.approx(1.2)


def test_muon_and_adafactor_options():
    # ferrotorch-optim/src/muon.rs (ns_coefficients, decoupled_weight_decay, strict_2d, maximize); adafactor.rs
    from ferrotorch_b200.optim.extra import CUBIC_NS, QUINTIC_NS, _newton_schulz

    torch.manual_seed(0)
    m = torch.randn(6, 4)
    for coeff, steps in ((CUBIC_NS, 30), (QUINTIC_NS, 8)):
        q = _newton_schulz(m, steps, coeff)
        sv = torch.linalg.svdvals(q)
        assert float(sv.min()) > 0.6 and float(sv.max()) < 1.3            # singular values driven towards one
    cubic = _newton_schulz(m, 1, CUBIC_NS)
    x = m / (m.norm() + 1e-7)
    torch.testing.assert_close(cubic, 1.5 * x - 0.5 * x @ (x.t() @ x))          # one cubic step: G (3 I - G^T G) / 2
    w = torch.nn.Parameter(torch.randn(4, 3))
    b = torch.nn.Parameter(torch.randn(4))
    with pytest.raises(ValueError):
        O.Muon([w, b], strict_2d=True)
    with pytest.raises(ValueError):
        O.Muon([w], ns_coefficients=(1.0, 2.0))
    # folded (L2) weight decay goes through the orthogonalisation, decoupled decay shrinks the weight directly
    g = torch.randn(4, 3)
    outs = {}
    for dec in (True, False):
        p = torch.nn.Parameter(w.detach().clone())
        opt = O.MuonConfig().with_lr(0.1).with_momentum(0.0).with_nesterov(False).with_weight_decay(0.5) \
            .with_decoupled_weight_decay(dec).build([p])
        p.grad = g.clone()
        opt.step()
        outs[dec] = p.detach().clone()
    scale = max(1.0, 4 / 3) ** 0.5
    torch.testing.assert_close(outs[True], w.detach() * (1 - 0.05) - 0.1 * scale * _newton_schulz(g, 5))
    torch.testing.assert_close(outs[False], w.detach() - 0.1 * scale * _newton_schulz(g + 0.5 * w.detach(), 5))
    pm = torch.nn.Parameter(w.detach().clone())
    om = O.Muon([pm], lr=0.1, momentum=0.0, nesterov=False, maximize=True)
    pm.grad = g.clone()
    om.step()
    torch.testing.assert_close(pm.detach(), w.detach() + 0.1 * scale * _newton_schulz(g, 5))
    # Adafactor: relative step size and first moment
    p = torch.nn.Parameter(torch.full((3, 2), 2.0))
    af = O.AdafactorConfig().with_lr(None).with_relative_step(True).with_warmup_init(True).with_beta1(0.9).build([p])
    p.grad = torch.ones(3, 2)
    af.step()
    # step 1: u = g / sqrt(v) clipped to rms 1 -> ones; first moment 0.1 * u; lr = min(1e-6, 1) * max(1e-3, rms(p) = 2)
    torch.testing.assert_close(p.detach(), torch.full((3, 2), 2.0 - 2e-6 * 0.1), rtol=0, atol=1e-9)
    assert "exp_avg" in af.state[p]
    p2 = torch.nn.Parameter(torch.full((3, 2), 2.0))
    af2 = O.Adafactor([p2], lr=None)
    p2.grad = torch.ones(3, 2)
    af2.step()
    torch.testing.assert_close(p2.detach(), torch.full((3, 2), 2.0 - 1e-2 * 2.0), rtol=1e-5, atol=1e-6)
    assert O.AdafactorConfig().with_decay_rate(0.7).beta2_decay == -0.7 and O.AdafactorConfig().with_eps_rms(0.5).eps == (1e-30, 0.5)
    assert O.GradScalerConfig().with_init_scale(128.0).with_enabled(False).init_scale == 128.0
    assert O.AdamWConfig().with_lr(3e-4).with_betas((0.9, 0.95)).build([p]).defaults["betas"] == (0.9, 0.95)


def test_jit_persistence_and_accessor_methods(tmp_path):
    # ferrotorch-jit/src/module.rs (TracedModule save / load / to_bytes), serialize.rs (IrGraph), codegen_ir.rs (Expr),
    # fusion.rs (FusedChain), codegen.rs (InductorBackend::compile_with_status), memory_plan.rs
    from ferrotorch_b200 import jit as J
    from ferrotorch_b200.jit.backends import (AutotuneKey, CpuCodegen, Expr, FusedChain, FusedOp, InductorBackend, LoopIR, MemoryPlan,
                                              NativeBackend)

    w = torch.randn(4, 4)

    def f(x, y):
        return torch.relu(x * 2.0 + y) @ w, (x - y).exp().sum(-1, keepdim=True).to(torch.float64)

    x, y = torch.randn(3, 4), torch.randn(3, 4)
    m = J.compile(f, (x, y))
    assert m.input_count() == 2 and m.output_shape() == (3, 4)
    m2 = J.TracedModule.from_bytes(m.to_bytes())
    for a, b in zip(m(x, y), m2(x, y)):
        assert torch.equal(a, b) and a.dtype == b.dtype
    assert [tuple(t.shape) for t in m2.forward_multi([x, y])] == [(3, 4), (3, 1)]
    m.save(str(tmp_path / "m.ftjm"))
    m3 = J.TracedModule.load(str(tmp_path / "m.ftjm"))
    assert torch.equal(m3(x, y)[0], m(x, y)[0])
    with pytest.raises(J.JitError):
        m3(x[:2], y[:2])                                         # a loaded module has no eager original to fall back to
    with pytest.raises(J.JitError):
        J.TracedModule.from_bytes(b"nope" + bytes(20))
    g2 = J.IrGraph.deserialize(m.graph.serialize())
    assert g2.fingerprint() == m.graph.fingerprint() and g2.ops() == m.graph.ops()
    with pytest.raises(ValueError):
        J.IrGraph.deserialize(m.graph.serialize()[:20])
    net = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.ReLU())
    traced = J.compile(net, (x,))
    if isinstance(traced, J.TracedModule) and any(n.op in ("call", "fused_linear_act") for n in traced.graph.nodes.values()):
        with pytest.raises(J.JitError):
            traced.to_bytes()                                    # the Linear module is a Python object
    # expression constructors
    e = Expr.call("exp", Expr.bin("add", Expr.var(0), Expr.prod([Expr.var(1), Expr.int(3), Expr.constant(0.5)])))
    fn = CpuCodegen().compile(LoopIR(2, e), "t")
    torch.testing.assert_close(fn(x, y), (x + y * 1.5).exp())
    assert Expr.sum([]).value == 0.0 and Expr.prod([]).value == 1.0 and e.depth() == 5
    # fused chain
    c = FusedChain().push(FusedOp.MulScalar, 2.0).push(FusedOp.Relu).push(FusedOp.Exp)
    assert c.len() == 3 and not c.is_empty() and FusedChain().is_empty()
    torch.testing.assert_close(c.execute_cpu(x), torch.relu(x * 2).exp())
    assert "my_kernel" in c.generate_ptx_named("my_kernel") and "double" in c.generate_ptx_f64_named("k") and c.generate_rust() and c.generate_ptx()
    # back-ends
    out = InductorBackend().with_block_size(128).compile_with_status(m.graph)
    assert out.is_compiled() != out.is_fallback() and out.compiled_graph() is out.into_compiled_graph()
    assert out.compiled_graph().num_inputs() == 2 and out.compiled_graph().output_shape() == (3, 4)
    torch.testing.assert_close(out.compiled_graph().execute([x, y])[0], m(x, y)[0])
    assert isinstance(InductorBackend().generate(m.graph), dict)
    plan = MemoryPlan.of(m.graph)
    assert 0.0 <= plan.savings_percent() < 100.0 and plan.naive_bytes >= plan.peak_bytes
    assert AutotuneKey.from_graph(m.graph, [x, y]) == AutotuneKey.from_graph(g2, [x, y]) != AutotuneKey.from_graph(m.graph, [x])
    assert isinstance(J.CompileConfig.from_optimization(J.OptimizationConfig()), J.CompileConfig)
    res = J.Autotuner().with_candidate("native", NativeBackend()).with_iterations(2).tune(m.graph, [x, y])
    assert res.winner_name() == "native" and res.winner_time() == res.median_s and res.winner_compiled() is res.compiled
    tuned = J.autotune(m, (x, y))
    assert tuned.winner_name().startswith("block_size=") and len(tuned.all_timings()) == len(tuned.candidates)
    assert J.JitCompiledKernel.output_len(torch.zeros(3, 1), torch.zeros(1, 4)) == 12


def test_train_and_distributed_accessor_methods(tmp_path):
    # ferrotorch-train/src/{amp,callback,metric,history,tensorboard}.rs; ferrotorch-optim/src/grad_accumulator.rs;
    # ferrotorch-distributed/src/{rpc,checkpoint,async_collective}.rs
    from ferrotorch_b200.parallel import dist_checkpoint as DC

    amp = T.AmpContext(torch.bfloat16, "cpu")
    assert amp.is_enabled() and amp.get_scale() == 1.0 and amp.scaler_mut() is amp.scaler
    out = amp.autocast_forward(lambda a, b: a @ b, torch.randn(4, 4), torch.randn(4, 4))
    assert out.dtype == torch.bfloat16
    amp.load_scaler_state_dict(amp.scaler_state_dict())
    assert not T.AmpContext(torch.float32, "cpu").is_enabled()
    lin = torch.nn.Linear(2, 2)
    cb = T.EMACallback(0.5)
    assert not cb.is_initialized() and cb.num_updates() == 0 and cb.shadow_params() == []
    cb.init_from_params(lin.parameters())
    w0 = lin.weight.detach().clone()
    with torch.no_grad():
        lin.weight += 2
    cb.update_from_params(list(lin.parameters()))
    assert cb.is_initialized() and cb.num_updates() == 1
    torch.testing.assert_close(cb.shadow_params()[0], w0 + 1)
    es = T.EarlyStopping(patience=2)

    class L:
        should_stop = False

    for i, v in enumerate((1.0, 0.5, 0.7, 0.8)):
        es.on_epoch_end(L, T.EpochResult.new_with_defaults(i, v))
    assert es.best_loss() == 0.5 and es.wait() == 2 and L.should_stop
    assert T.EpochResult.new_with_defaults(0, 1.0, 2.0).val == {"loss": 2.0} and T.EvalResult.new_with_defaults(0.25).get("loss") == 0.25
    assert T.RunningAverage(0.98).window_size() == 50
    tbw = T.TensorBoardWriter(str(tmp_path / "tb"))
    assert tbw.log_dir() == str(tmp_path / "tb")
    tbw.close()
    acc = O.GradientAccumulator(3)
    assert acc.accumulation_steps() == 3 and float(acc.scale_loss(torch.tensor(6.0))) == 2.0
    assert [acc.should_step() for _ in range(4)] == [False, False, True, False] and acc.current_step() == 1
    acc.reset()
    assert acc.current_step() == 0
    # RPC: a request frame dispatched in memory
    agent = DC.RpcAgent("worker", rank=1, world_size=4)
    try:
        agent.register("add", lambda a, b=0: a + b)
        assert (agent.rank(), agent.world_size()) == (1, 4)
        rid, ok, val = DC.decode_rpc_response(agent.handle_request(0, DC.encode_rpc_request(7, "add", 2, b=5)))
        assert (rid, ok, val) == (7, True, 7)
        rid, ok, val = DC.decode_rpc_response(agent.handle_request(2, DC.encode_rpc_request(8, "nope")))
        assert rid == 8 and not ok and "no handler" in val and "rank 2" in val
        rid, ok, val = DC.decode_rpc_response(agent.handle_request(0, DC.encode_rpc_request(9, "add", "x", b=1)))
        assert rid == 9 and not ok and "TypeError" in val
        _, ok, _ = DC.decode_rpc_response(agent.handle_request(0, b"\\x00\\x01"))
        assert not ok
        assert DC.RpcAgent.rpc_sync(agent.address, "add", 1, b=2) == 3              # and the same handler over TCP
    finally:
        agent.shutdown()
    with pytest.raises(DC.InvalidRank):
        DC.RpcAgent("bad", rank=4, world_size=4)
    ck = DC.AsyncDistributedCheckpointer(str(tmp_path / "ck"), rank=0, world_size=1)
    assert (ck.dir(), ck.rank(), ck.world_size()) == (str(tmp_path / "ck"), 0, 1)
    ck.save({"w": torch.arange(6.0).reshape(3, 2)}, {"w": 0}).wait()
    assert not ck.is_saving()
    state, _ = DC.load_distributed(str(tmp_path / "ck"), 0, 1)
    assert torch.equal(state["w"], torch.arange(6.0).reshape(3, 2))
    with pytest.raises(ValueError):
        DC.AsyncDistributedCheckpointer().save({}, {})
    pend = DC.PendingCollective(lambda: 5, op_name="all_reduce")
    assert pend.wait(5) == 5 and pend.op_name() == "all_reduce"


def test_vision_builder_and_accessor_methods(tmp_path):
    # ferrotorch-vision/src/transforms/*.rs builders, datasets/folder.rs, models/registry.rs,
    # models/detection/{anchor_utils,faster_rcnn,rpn}.rs
    import torchvision.transforms.functional as TF
    from torchvision.transforms import InterpolationMode as IM

    from ferrotorch_b200 import vision as V
    from ferrotorch_b200.ops.det_ops import AnchorGenerator
    from ferrotorch_b200.vision import own_transforms as OT

    torch.manual_seed(0)
    x = torch.rand(3, 17, 23)
    for ang in (30.0, -75.0, 90.0):
        for expand in (False, True):
            for center in (None, (5.0, 4.0)):
                for mode, im in (("nearest", IM.NEAREST), ("bilinear", IM.BILINEAR)):
                    a = OT.rotate(x, ang, 0.25, mode, expand, center)
                    b = TF.rotate(x, ang, im, expand, list(center) if center else None, [0.25])
                    assert a.shape == b.shape and float((a - b).abs().max()) < 1e-5, (ang, expand, center, mode)
    for interp, im in (("nearest", IM.NEAREST), ("bilinear", IM.BILINEAR), ("bicubic", IM.BICUBIC)):
        assert torch.equal(OT.Resize((9, 31)).with_interpolation(interp)(x), TF.resize(x, [9, 31], im, antialias=True))
    with pytest.raises(ValueError):
        OT.resize(x, 8, True, "lanczos")
    padded = OT.CenterCrop((21, 29)).with_fill(0.5)(x)
    assert padded.shape == (3, 21, 29) and float(padded[0, 0, 0]) == 0.5 and torch.equal(padded[:, 2:19, 3:26], x)
    V.vision_manual_seed(3)
    rc = OT.RandomCrop.square(20).with_padding_hw(4, 0).with_fill(0.75).with_pad_if_needed(True)
    out = rc(x)
    assert out.shape == (3, 20, 20) and rc.padding == (4, 0) and OT.RandomCrop.square(20).padding == 0       # builders return copies
    assert OT.RandomCrop(8).with_padding(2).padding == 2
    rr = OT.RandomRotation(30).with_expand(True).with_center((3, 3)).with_fill(0.1).with_interpolation("bilinear")
    assert rr.expand and rr.center == (3.0, 3.0) and rr.mode == "bilinear" and rr(x).shape[0] == 3
    with pytest.raises(ValueError):
        OT.RandomRotation(30).with_interpolation("bicubic")
    rz = OT.RandomResizedCrop(12).with_antialias(False).with_interpolation("nearest")
    assert rz(x).shape == (3, 12, 12) and not rz.antialias
    comp = OT.Compose([OT.RandomHorizontalFlip(1.0), OT.CenterCrop(8)])
    assert len(comp) == comp.len() == 2 and not comp.is_empty() and OT.Compose([]).is_empty()
    first = OT.RandomChoice([lambda t: t * 0, lambda t: t + 1]).with_p([1.0, 0.0])
    assert float(first(x).abs().max()) == 0.0
    with pytest.raises(ValueError):
        OT.RandomChoice([lambda t: t]).with_p([0.5, 0.5])
    cj = OT.ColorJitter.from_ranges(brightness=(2.0, 2.0), hue=None)
    torch.testing.assert_close(cj(x), (x * 2).clamp(0, 1))
    with pytest.raises(ValueError):
        OT.ColorJitter.from_ranges(hue=(-0.7, 0.1))
    el = OT.ElasticTransform.new_range((10.0, 20.0), (3.0, 4.0)).with_fill(0.5).with_interpolation("nearest")
    assert el(x).shape == x.shape and el.fill == 0.5
    with pytest.raises(ValueError):
        OT.ElasticTransform.new_range((5.0, 1.0), (3.0, 4.0))
    n = V.io.VisionNormalize.imagenet()
    torch.testing.assert_close(n(torch.full((3, 2, 2), 0.485))[0], torch.zeros(2, 2))
    assert not V.io.GaussianNoise(0.0, 0.1).with_clip(False).clip
    # image folder constructors
    for cls, names in (("cat", ("a.png", "b.jpg", "c.txt")), ("dog", ("d.png",))):
        (tmp_path / cls).mkdir()
        for nm in names:
            if nm.endswith(".txt"):
                (tmp_path / cls / nm).write_text("x")
            else:
                from PIL import Image

                Image.new("RGB", (4, 4)).save(str(tmp_path / cls / nm))
    ds = V.ImageFolder.from_dir(str(tmp_path))
    assert len(ds) == 3 and ds.num_classes() == 2
    assert len(V.ImageFolder.from_dir_with_extensions(str(tmp_path), ["png"])) == 2
    assert len(V.ImageFolder.from_dir_with_filter(str(tmp_path), lambda p: "dog" in p)) == 1
    # registry and anchors
    reg = V.ModelRegistry()
    reg.register_model("tiny_test_net", lambda **kw: torch.nn.Linear(2, 2))
    assert "tiny_test_net" in reg.list_models() and isinstance(reg.get_model("tiny_test_net"), torch.nn.Linear)
    assert V.RpnConfig.default_eval().nms_thresh == 0.7
    g = AnchorGenerator.default_fasterrcnn()
    grids = [(200, 272), (100, 136), (50, 68), (25, 34), (13, 17)]
    parts = [g.generate_anchors_for_image(l, gs, (800, 1088)) for l, gs in enumerate(grids)]
    assert torch.equal(torch.cat(parts), g((800, 1088), grids))
    canon = g.generate_anchors(4, (13, 17))                       # p6: canonical stride 64, image-derived 61 vertically
    assert canon.shape == parts[4].shape and not torch.equal(canon, parts[4])
    assert torch.equal(canon[:, [0, 2]], parts[4][:, [0, 2]])     # the horizontal stride is 64 either way
    assert torch.equal(g.generate_anchors(0, (4, 4)), g((16, 16), [(4, 4)] + [(1, 1)] * 4)[:4 * 4 * 3])


def test_detector_pieces_under_the_reference_names():
    from ferrotorch_b200.models.detection import FasterRCNN

    torch.manual_seed(0)
    det = FasterRCNN(num_classes=5).eval()
    img = torch.rand(1, 3, 64, 64)
    c = det.forward_backbone(img)
    assert sorted(c) == ["layer1", "layer2", "layer3", "layer4"] and c["layer1"].shape == (1, 256, 16, 16) and c["layer4"].shape == (1, 2048, 2, 2)
    p = det.forward_fpn(c)
    assert sorted(p) == ["p2", "p3", "p4", "p5", "p6"] and all(v.shape[1] == 256 for v in p.values())
    with torch.no_grad():
        whole = det.backbone(img)
    for a, b in zip(p.values(), whole.values()):
        assert torch.equal(a, b)
    assert det.num_classes() == 5 and det.num_parameters() == sum(q.numel() for q in det.parameters() if q.requires_grad)
    with torch.no_grad():
        obj, deltas = det.rpn.head.forward_level(p["p3"])
        all_obj, all_deltas = det.rpn.head([p["p3"]])
    assert torch.equal(obj, all_obj[0]) and torch.equal(deltas, all_deltas[0]) and deltas.shape[1] == 4 * obj.shape[1]


def test_core_wrapper_methods():
    # ferrotorch-core/src/{masked,sparse,dispatch,device}.rs, ferrotorch-nn/src/{flex_attention,qat}.rs, core quantize.rs
    import ferrotorch_b200 as ft
    from ferrotorch_b200 import nn as N

    m = ft.MaskedTensor.from_data(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([True, False, True])).with_fill_value(-1.0)
    assert (m.count_valid(), m.count_masked(), m.numel(), m.shape, m.fill_value()) == (2, 1, 3, (3,), -1.0)
    assert m.to_tensor().tolist() == [1.0, -1.0, 3.0] and m.to_ferray().mask.tolist() == [False, True, False]
    w = torch.randn(4, 16)
    s = ft.SemiStructuredSparseTensor.compress(w)
    assert s.num_groups() == 16 and int(s.mask().sum()) == 32 and sum(s.group_mask(5)) == 2
    assert torch.equal(s.decompress(), s.to_dense()) and torch.equal(s.decompress() != 0, s.mask())
    assert s.values_shape() == (4, 8) and s.indices_shape() == tuple(s.indices.shape) and s.packed is s.values and s.compression_ratio() > 1.7
    with pytest.raises(ft.FerrotorchError):
        ft.SemiStructuredSparseTensor.compress(torch.randn(4, 6))
    D = ft.Device
    assert D.is_cpu("cpu") and D.is_cuda(D.Cuda(1)) and D.is_meta(D.Meta) and not D.is_xpu("cpu") and not D.is_mps("cpu")
    bm = N.BlockMask.causal_mask(10, 4)
    assert (bm.num_q_blocks(), bm.num_k_blocks()) == (3, 3) and bm.is_active(1, 0) and not bm.is_active(0, 1)
    assert bm.allows_position(5, 7) and not bm.allows_position(2, 9) and not bm.allows_position(11, 0)      # block granularity
    assert N.BlockMask.full_mask(10, 6, 4).keep.all() and N.BlockMask.full_mask(10, 6, 4).keep.shape == (3, 2)
    sw = N.BlockMask.sliding_window_mask(16, 2, 4)
    assert sw.is_active(1, 0) and sw.is_active(0, 1) and not sw.is_active(0, 2) and not sw.is_active(3, 1)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 6), torch.nn.ReLU(), torch.nn.Linear(6, 3))
    qm = N.QatModel(net, N.QatConfig.int4_weight_int8_activation()).train()
    x = torch.randn(16, 8)
    fq_out = qm(x)
    plain = qm.fake_quantize_weights(False).fake_quantize_activations(False)(x)
    torch.testing.assert_close(plain, torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(x, qm.model[0].weight, qm.model[0].bias)),
                                                               qm.model[2].weight, qm.model[2].bias))
    assert not torch.equal(fq_out, plain)
    q = qm.fake_quantize_weights(True).convert()
    assert q.weight_names() == ["0", "2"] and q.num_weights() == 2 and q.weight("0").dtype == torch.int8
    assert int(q.weight("0").abs().max()) <= 8 and q.weight_qparams("0")[0].shape == (6,)
    assert q.quantized_size_bytes() == (48 * 4 + 7) // 8 + 24 + (18 * 4 + 7) // 8 + 12 and q.compression_ratio() > 3.5
    assert float((q.dequantize_weight("0") - qm.model[0].weight.detach()).abs().max()) < float(q.weight_qparams("0")[0].max())
    with pytest.raises(KeyError):
        q.weight("9")
    skipped = N.QatModel(torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.Linear(4, 2)), N.QatConfig(skip=("1",)))
    assert type(skipped.model[1]) is torch.nn.Linear
    skipped.register_layer("1")
    assert isinstance(skipped.model[1], N.QatLinear) and N.QatConfig.default_symmetric_int8().weight_bits == 8
    fq = N.FakeQuantize(8).train()
    fq(x)
    scale, zero = fq.calculate_qparams()
    assert float(scale) > 0 and float(zero) == 0
    assert torch.equal(fq.disable_fake_quant()(x), x)
    lo = fq.enable_fake_quant().disable_observer().observer.max_val.clone()
    fq(x * 100)
    assert torch.equal(fq.observer.max_val, lo)                                   # the range is frozen
    fq.enable_observer()(x * 100)
    assert float(fq.observer.max_val) > float(lo)


def test_model_and_distributed_leftover_methods(tmp_path):
    # ferrotorch-llama/src/{attention,layer}.rs forward_with_cache; ferrotorch-diffusion/src/unet.rs forward_t;
    # ferrotorch-bert / -whisper config loaders; ferrotorch-distributed dtensor / backend / sync_batch_norm; serialize
    import json as _json

    from ferrotorch_b200.models import diffusion as D
    from ferrotorch_b200.models import generation as G
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.models.pretrained import BertConfig, BertEmbeddings, WhisperConfig
    from ferrotorch_b200.parallel import Partial, Replicate, Shard
    from ferrotorch_b200.parallel.backend import InvalidRank, SimulatedGroup, SubGroup
    from ferrotorch_b200.parallel.p2p import Placement
    from ferrotorch_b200.serialize import AsyncCheckpointer, load_checkpoint

    torch.manual_seed(0)
    m = LlamaForCausalLM(LlamaConfig.tiny()).eval()
    ids = torch.tensor([[3, 17, 5, 99]])
    with torch.no_grad():
        x = m.model.embed_tokens(ids)
        layer = m.model.layers[0]
        h, d = layer(x)
        cache, outs = None, []
        for t in range(4):
            o, cache = layer.forward_with_cache(x[:, t:t + 1], cache)
            outs.append(o)
        torch.testing.assert_close(torch.cat(outs, 1), h + d)
        att, hn = layer.self_attn, layer.input_layernorm(x)
        o1, c1 = att.forward_with_cache(hn[:, :3], None)
        o2, c2 = att.forward_with_cache(hn[:, 3:], c1, seq_offset=3)
        torch.testing.assert_close(torch.cat([o1, o2], 1), att(hn))
    assert (c1.seq_len(), c2.seq_len(), cache.seq_len()) == (3, 4, 4) and (att.num_heads(), att.num_kv_heads()) == (4, 2)
    with pytest.raises(ValueError):
        att.forward_with_cache(hn[:, 3:], c1, seq_offset=1)
    with pytest.raises(ValueError):
        G.SpecDecodeConfig(gamma=0).validate()
    # UNet blocks one by one
    cfg = D.UNet2DConditionConfig(block_out_channels=(32, 64), layers_per_block=1, cross_attention_dim=16, attention_head_dim=4,
                                  norm_num_groups=8, down_block_types=("CrossAttnDownBlock2D", "DownBlock2D"),
                                  up_block_types=("UpBlock2D", "CrossAttnUpBlock2D"))
    assert cfg.num_blocks() == 2 and cfg.time_embed_dim() == 128
    u = D.UNet2DConditionModel(cfg).eval()
    lat, ctx = torch.randn(1, 4, 8, 8), torch.randn(1, 5, 16)
    with torch.no_grad():
        want = u(lat, 10, ctx)
        temb = u.time_embedding(D.timestep_embedding(torch.tensor([10]), 32, cfg.flip_sin_to_cos, cfg.freq_shift))
        hcur = u.conv_in(lat)
        skips = [hcur]
        for blk in u.down_blocks:
            hcur, sk = blk.forward_t(hcur, temb, ctx)
            skips += sk
        hcur = u.mid_block.forward_t(hcur, temb, ctx)
        for blk in u.up_blocks:
            n = len(blk.resnets)
            take, skips = skips[-n:], skips[:-n]
            hcur = blk.forward_t(hcur, temb, ctx, skips=take)
        got = u.conv_out(torch.nn.functional.silu(u.conv_norm_out(hcur)))
        assert torch.equal(got, want) and torch.equal(u.forward_t(lat, 10, ctx), want) and not skips
        with pytest.raises(ValueError):
            u.up_blocks[0].forward_t(hcur, temb, ctx, skips=[])
    u.load_hf_state_dict(u.state_dict())
    raw = {"vocab_size": 50, "hidden_size": 16, "num_hidden_layers": 1, "num_attention_heads": 2, "intermediate_size": 32}
    (tmp_path / "config.json").write_text(_json.dumps(raw))
    assert BertConfig.from_file(str(tmp_path)) == BertConfig.from_file(str(tmp_path / "config.json")) == BertConfig.from_json_str(_json.dumps(raw))
    assert hasattr(WhisperConfig, "from_file") and hasattr(WhisperConfig, "from_json_str")
    emb = BertEmbeddings(BertConfig.from_json_str(_json.dumps(raw)))
    assert torch.equal(emb.forward_from_ids([1, 2, 3]), emb(torch.tensor([[1, 2, 3]])))
    # placements, sub-groups, synchronised batch norm
    assert Shard(1).is_shard() and Shard(1).shard_dim() == 1 and Replicate().is_replicate() and Partial().is_partial()
    assert Replicate().shard_dim() is None and Placement.is_shard(Shard(0)) and Placement.shard_dim(Shard(2)) == 2
    world = SimulatedGroup.create_group(4)
    sub = SubGroup(world[2], [3, 2])
    assert sub.to_global(0) == 2 and sub.to_local(3) == 1
    with pytest.raises(InvalidRank):
        sub.to_local(0)
    from ferrotorch_b200.parallel import SyncBatchNorm2d

    one = SimulatedGroup.create_group(1)[0]
    bn = SyncBatchNorm2d(3, one).train()
    bn(torch.randn(4, 3, 2, 2))
    assert int(bn.num_batches_tracked) == 1
    other = bn.with_backend(SimulatedGroup.create_group(1)[0])
    assert other.weight is bn.weight and other.group is not bn.group and other.running_mean is bn.running_mean
    ck = AsyncCheckpointer()
    assert not ck.is_saving()
    ck.save(str(tmp_path / "ck.pt"), {"w": torch.arange(4.0)})
    ck.wait()
    assert not ck.is_saving() and torch.equal(load_checkpoint(str(tmp_path / "ck.pt"))["model"]["w"], torch.arange(4.0))


def test_gpu_side_helper_objects_without_a_gpu(tmp_path):
    # ferrotorch-gpu/src/{graph,memory_guard,device}.rs names that are host logic; ferrotorch-llama/src/gpu_gguf.rs
    import time as _time

    from ferrotorch_b200 import cuda as C
    from ferrotorch_b200 import jit as J
    from ferrotorch_b200.utils.memory_guard import MemoryGuard, MemoryReservation

    class Alloc:
        used, device = 0, 0

        def used_bytes(self):
            return self.used

        def total_bytes(self):
            return 1000

        def empty_cache(self):
            pass

    a = Alloc()
    g = MemoryGuard(a, pressure_threshold=0.5)
    w = C.MemoryWatchdog(g, 0.01)
    assert w.pressure_threshold_bytes() == 500 and not w.check_pressure() and w.memory_info() == (1000, 1000) and w.guard() is g
    w.start()
    a.used = 900
    _time.sleep(0.1)
    assert g.paused.is_set() and w.wait_for_first_check(0.5) and not w.wait_if_paused(0.05) and w.check_pressure()
    a.used = 0
    assert w.wait_if_paused(1.0)
    w.stop()
    r = MemoryReservation(g, 100)
    assert r.reserved_bytes() == 100 and r.device_ordinal() == 0
    r.release()
    assert r.reserved_bytes() == 0
    d = C.MemoryGuardedDevice(g)
    assert d.guard() is g and d.safe_alloc((3,)).shape == (3,) and d.safe_alloc_copy([1.0]).tolist() == [1.0]
    assert C.CaptureMode.Relaxed.to_cuda() == 2 and C.CaptureStatus.Active.is_capturing() and C.CaptureStatus.Invalidated.is_invalidated()
    assert not C.CaptureStatus.NotCapturing.is_capturing()
    for name in ("begin", "begin_with_mode", "begin_with_pool", "begin_with_pool_mode", "finish", "status"):
        assert hasattr(C.GraphCaptureGuard, name)
    for name in ("with_private_pool", "record_buffer", "seal", "unseal", "buffer_count", "clear_buffers", "activate", "raw"):
        assert hasattr(C.CapturePool, name)
    # AOT module: both directions by hand
    lin = torch.nn.Linear(3, 2)
    x = torch.randn(4, 3, requires_grad=True)
    aot = J.compile_aot(lin, (x.detach(),))
    out, ctx = aot.forward_with_ctx(x.detach())
    torch.testing.assert_close(out, lin(x).detach())
    go = torch.randn(4, 2)
    grads = aot.backward(ctx, go)
    want = torch.autograd.grad(lin(x), [*lin.parameters(), x], go)
    for got, exp in zip(grads, want):
        torch.testing.assert_close(got, exp)
    assert aot.saved_tensor_indices() == [0, 1, 2] and len(aot.saved_tensors(ctx)) == 3
    assert aot.forward_graph() is aot.pair.forward and aot.backward_graph() is aot.pair.backward
    # inferencer from a GGUF file, and greedy decoding under a grammar
    from ferrotorch_b200.models.inferencer import LlamaGpuInferencer
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.serialize import gguf as GG
    from ferrotorch_b200.utils.grammar import JsonSchemaProcessor

    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1, max_position_embeddings=64)
    torch.manual_seed(0)
    src = LlamaForCausalLM(cfg).eval()
    inv = {v: k for k, v in (("token_embd", "model.embed_tokens"), ("output_norm", "model.norm"), ("output", "lm_head"))}
    layer_inv = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
                 "self_attn.o_proj": "attn_output", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate",
                 "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    tensors = {}
    for k, v in src.hf_state_dict().items():
        base, _, _suffix = k.rpartition(".")
        if base.startswith("model.layers."):
            _, _, idx, rest = base.split(".", 3)
            name = "blk.%s.%s.weight" % (idx, layer_inv[rest])
        else:
            name = inv[base] + ".weight"
        t = v.detach().float().contiguous()
        tensors[name] = (GG.GGML_F32, tuple(t.shape), t.numpy().tobytes())
    md = {"general.architecture": "llama", "llama.embedding_length": 32, "llama.feed_forward_length": 64, "llama.block_count": 1,
          "llama.attention.head_count": 2, "llama.attention.head_count_kv": 1, "llama.context_length": 64, "llama.vocab_size": 64,
          "llama.attention.layer_norm_rms_epsilon": float(cfg.rms_norm_eps), "llama.rope.freq_base": float(cfg.rope_theta)}
    path = str(tmp_path / "tiny.gguf")
    GG.write_gguf(path, tensors, md)
    inf = LlamaGpuInferencer.from_gguf_gpu_dequant(path, device="cpu")
    ids = [3, 9, 27]
    torch.testing.assert_close(inf.forward_from_ids(ids), src(torch.tensor([ids]))[0, -1].detach().float(), rtol=1e-4, atol=1e-4)
    vocab = [chr(97 + i % 26) * (1 + i // 26) for i in range(60)] + ["true", "false", "tr", "ue"]
    proc = JsonSchemaProcessor({"type": "boolean"}, vocab)
    gen = inf.generate_masked(ids, proc, 8)
    text = "".join(vocab[t] for t in gen)
    assert text in ("true", "false") and proc.is_complete()
    assert len(inf.generate_masked(ids, None, 3)) == 3


def test_box_operators_losses_and_roi_pooling_match_torchvision_ops():
    # ferrotorch-vision/src/ops.rs (box_area / box_convert / *_box_iou / roi_pool / focal loss), roi_heads_postprocess.rs
    import torchvision.ops as TO

    from ferrotorch_b200 import vision as V

    torch.manual_seed(0)

    def boxes(n):
        xy, wh = torch.rand(n, 2) * 50, torch.rand(n, 2) * 30 + 1
        return torch.cat([xy, xy + wh], 1)

    a, b = boxes(7), boxes(5)
    for ours, theirs in ((V.generalized_box_iou, TO.generalized_box_iou), (V.distance_box_iou, TO.distance_box_iou),
                         (V.complete_box_iou, TO.complete_box_iou), (V.box_iou, TO.box_iou)):
        torch.testing.assert_close(ours(a, b), theirs(a, b), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(V.box_area(a), TO.box_area(a))
    for i in ("xyxy", "xywh", "cxcywh"):
        src = TO.box_convert(a, "xyxy", i)
        for o in ("xyxy", "xywh", "cxcywh"):
            torch.testing.assert_close(V.box_convert(src, i, o), TO.box_convert(src, i, o))
    with pytest.raises(ValueError):
        V.box_convert(a, "xyxy", "polar")
    torch.testing.assert_close(V.clip_boxes_to_image(a * 3 - 20, (40, 60)), TO.clip_boxes_to_image(a * 3 - 20, (40, 60)))
    assert torch.equal(V.remove_small_boxes(a, 12.0), TO.remove_small_boxes(a, 12.0))
    x, t = torch.randn(6, 4), (torch.rand(6, 4) > 0.5).float()
    for red in ("none", "mean", "sum"):
        torch.testing.assert_close(V.sigmoid_focal_loss(x, t, 0.25, 2.0, red), TO.sigmoid_focal_loss(x, t, 0.25, 2.0, red))
    torch.testing.assert_close(V.focal_loss(x, t, -1.0, 1.5), TO.sigmoid_focal_loss(x, t, -1.0, 1.5))
    feat = torch.randn(2, 3, 16, 20)
    rois = torch.tensor([[0, 2.0, 3.0, 30.0, 25.0], [1, 0.0, 0.0, 39.0, 31.0], [0, 10.0, 4.0, 12.0, 9.0], [1, 35.0, 20.0, 80.0, 60.0]])
    for scale in (1.0, 0.5, 0.25):
        for size in ((3, 4), 7, 1):
            assert torch.equal(V.roi_pool(feat, rois, size, scale), TO.roi_pool(feat, rois, size, scale))
    assert torch.equal(V.roi_pool(feat, [rois[[0, 2], 1:], rois[[1, 3], 1:]], 2), TO.roi_pool(feat, [rois[[0, 2], 1:], rois[[1, 3], 1:]], 2))
    torch.testing.assert_close(V.roi_align_with_aligned(feat, rois, 3, 0.5, 2), TO.roi_align(feat, rois, 3, 0.5, 2, True))
    # second-stage post-processing as free functions
    logits, reg = torch.randn(6, 4), torch.randn(6, 16) * 0.1
    props = [boxes(4), boxes(2)]
    det = V.postprocess_detections(logits, reg, props, (80, 80), score_thresh=0.0, nms_thresh=0.5, detections_per_img=5)
    assert len(det) == 2 and all(len(d["boxes"]) <= 5 and d["labels"].min() >= 1 for d in det if len(d["boxes"]))
    per_class = V.decode_per_class(reg, torch.cat(props))
    assert per_class.shape == (6, 4, 4)
    ml = torch.randn(3, 4, 5, 5)
    pm = V.postprocess_masks(ml, torch.tensor([1, 3, 2]))
    assert pm.shape == (3, 1, 5, 5) and torch.allclose(pm[1, 0], torch.sigmoid(ml[1, 3]))
    bn_src, bn_dst = torch.nn.BatchNorm2d(3), torch.nn.BatchNorm2d(3)
    bn_src.running_mean.fill_(2.0)
    assert V.apply_bn_buffers_from_state_dict(bn_dst, bn_src.state_dict()) == 3 and float(bn_dst.running_mean[0]) == 2.0
    for name in ("vgg11", "swin_tiny", "retinanet_resnet50_fpn", "mobilenet_v3_large_dilated", "resnet50_dilated", "yolo", "unet"):
        assert callable(getattr(V, name))
    assert type(V.mobilenet_v3_small(num_classes=7)).__name__ == "MobileNetV3"
    with pytest.raises(AttributeError):
        V.no_such_model


def test_free_functions_of_the_core_nn_and_distributions_crates():
    # ferrotorch-core/src/{ops,linalg,signal,shape,stride_tricks,meta_propagate,vmap}/, ferrotorch-nn/src/{functional,padding,init}.rs,
    # ferrotorch-distributions/src/{constraints,kl,exp_family}.rs, ferrotorch-profiler/src/flops.rs
    import numpy as np
    from scipy.signal import windows as W

    import ferrotorch_b200 as ft
    from ferrotorch_b200 import distributions as Dn
    from ferrotorch_b200 import nn as N
    from ferrotorch_b200 import profiler as Pf

    for n in (1, 2, 7, 16):
        for sym in (True, False):
            for name, args in (("parzen", ()), ("tukey", (0.3,)), ("tukey", (0.0,)), ("tukey", (1.0,)), ("taylor", (4, 30.0)),
                               ("taylor", (3, 40.0, False))):
                got = getattr(ft, name)(n, *args, sym=sym, dtype=torch.float64).numpy()
                assert np.allclose(got, getattr(W, name)(n, *args, sym=sym), atol=1e-12), (name, n, sym, args)
    assert torch.equal(ft.hanning(5), torch.signal.windows.hann(5)) and ft.kaiser(5, beta=3.0).shape == (5,)     # torch's, through the root
    x = torch.randn(3, 4, 5)
    assert torch.equal(ft.amax_dim(x, 1), x.amax(1)) and torch.equal(ft.argmin_dim(x, 2, True), x.argmin(2, True))
    assert torch.equal(ft.reduce_dim(x, 0, "prod"), x.prod(0)) and torch.equal(ft.reverse_cumsum(x, 1), x.flip(1).cumsum(1).flip(1))
    torch.testing.assert_close(ft.std_with_correction(x, 1, 0), x.std(1, correction=0))
    torch.testing.assert_close(ft.logsumexp_dim(x, 2), x.logsumexp(2))
    assert torch.equal(ft.add_scaled(x, x, 0.5), x * 1.5) and torch.equal(ft.mm_bt_differentiable(x[0], x[1]), x[0] @ x[1].t())
    assert ft.channels_last_strides((2, 3, 4, 5)) == torch.empty(2, 3, 4, 5).contiguous(memory_format=torch.channels_last).stride()
    assert ft.channels_last_3d_strides((2, 3, 4, 5, 6)) == torch.empty(2, 3, 4, 5, 6).contiguous(memory_format=torch.channels_last_3d).stride()
    assert ft.c_contiguous_strides((2, 3, 4)) == (12, 4, 1) and ft.checked_numel((2, 3)) == 6 and ft.checked_byte_count((2, 3), 4) == 24
    with pytest.raises(ft.FerrotorchError):
        ft.checked_numel((2 ** 40, 2 ** 40))
    with pytest.raises(ft.FerrotorchError):
        ft.channels_last_strides((2, 3))
    assert ft.zeros_meta((2, 3)).device.type == "meta" and ft.meta_like(x).shape == x.shape and ft.fft_norm_from_str(None) == "backward"
    v, tau = torch.randn(5, 3), torch.rand(3)
    q = ft.householder_product_full(v, tau)
    assert q.shape == (5, 5) and torch.allclose(q[:, :3], torch.linalg.householder_product(v, tau), atol=1e-6)
    g = ft.per_sample_grad(lambda p, row: (p * row).sum() ** 2, torch.ones(3), torch.arange(6.0).view(2, 3))
    assert torch.equal(g, torch.tensor([[0.0, 6.0, 12.0], [72.0, 96.0, 120.0]]))
    assert torch.equal(ft.masked_fill_bcast(x, torch.tensor([True, False, False, False, True]), 0.0)[..., 0], torch.zeros(3, 4))
    assert torch.equal(ft.unary_map_named(x, "erf"), torch.erf(x)) and torch.equal(ft.binary_broadcast(x, x[0], torch.add), x + x[0])
    with pytest.raises(ft.FerrotorchError):
        ft.binary_map(x, x[0], torch.add)
    # torch's own spellings reached through the package root
    assert ft.pinv(torch.eye(2)).shape == (2, 2) and ft.glu(torch.randn(2, 4)).shape == (2, 2)
    assert float(ft.chebyshev_polynomial_t(torch.tensor([0.5]), torch.tensor([3]))) == -1.0
    # autocast / saved-tensor / profiler plumbing
    assert ft.autocast_log("matmul", "cpu") is None
    with torch.autocast("cpu", dtype=torch.bfloat16):
        assert (ft.autocast_log("matmul", "cpu"), ft.autocast_log("softmax", "cpu"), ft.autocast_log("relu", "cpu")) == ("reduced", "full", "keep")
        snap = ft.current_autocast_snapshot()
    with ft.with_autocast_state(snap):
        assert (torch.ones(2, 2) @ torch.ones(2, 2)).dtype == torch.bfloat16
    assert not ft.has_saved_tensor_hooks()
    with ft.tracked_saved_tensors_hooks(lambda t: t.half(), lambda p: p.float()):
        assert ft.has_saved_tensor_hooks() and ft.pack_saved_tensor(torch.ones(2)).dtype == torch.float16
        y = torch.ones(2, requires_grad=True)
        (y * y).sum().backward()
    assert torch.equal(y.grad, torch.full((2,), 2.0)) and ft.unpack_saved_tensor(3) == 3
    prof = Pf.Profiler(Pf.ProfileConfig(cuda_events=False))
    ft.set_current(prof)
    with ft.profile_op_scope("matmul", "linalg", [(2, 2), (2, 2)]):
        pass
    ft.set_current(None)
    with ft.profile_op_scope("ignored"):
        pass
    assert ft.current() is None and [e.name for e in prof.events] == ["matmul"]
    before = torch.rand(1)
    torch.manual_seed(5)
    a = torch.rand(1)
    torch.manual_seed(5)
    ft.with_default_rng_test_lock(lambda: torch.rand(100))
    assert torch.equal(torch.rand(1), a) and before is not None
    o1, o2 = ft.checkpoint_multi(lambda p, r: (p * r, p + r), torch.ones(2, requires_grad=True), torch.ones(2))
    assert o1.requires_grad and torch.equal(o2, torch.full((2,), 2.0))
    # nn: padding, parameterised activations, seeded initialisers
    seq = torch.arange(6.0).view(1, 1, 6)
    assert N.functional_pad_1d(seq, 2, -1, "reflect").tolist() == [[[2.0, 1.0, 0.0, 1.0, 2.0, 3.0, 4.0]]]
    assert N.functional_pad_2d_signed(torch.ones(1, 1, 2, 2), 1, 0, 0, 1, N.PaddingMode.Zeros if hasattr(N.PaddingMode, "Zeros") else "zeros", 5.0).shape == (1, 1, 3, 3)
    g1, g2 = torch.Generator().manual_seed(1), torch.Generator().manual_seed(1)
    p1, p2 = torch.nn.Parameter(torch.empty(8, 4)), torch.nn.Parameter(torch.empty(8, 4))
    N.kaiming_uniform_with_fan_mode_and_generator(p1, "relu", "fan_out", g1)
    torch.nn.init.kaiming_uniform_(p2, mode="fan_out", nonlinearity="relu", generator=g2)
    assert torch.equal(p1, p2)
    N.trunc_normal_with_generator(p1, 0.0, 1.0, -0.5, 0.5, g1)
    assert float(p1.detach().abs().max()) <= 0.5 and float(N.log_sigmoid(torch.zeros(1))) == pytest.approx(-0.6931, abs=1e-4)
    torch.testing.assert_close(N.gelu_with(seq, "tanh"), torch.nn.functional.gelu(seq, approximate="tanh"))
    torch.testing.assert_close(N.softplus_with(seq, 2.0, 3.0), torch.nn.functional.softplus(seq, 2.0, 3.0))
    # distributions
    assert Dn.open_interval(0.0, 1.0).check(torch.tensor([0.0, 0.5, 1.0])).tolist() == [False, True, False]
    assert Dn.closed_interval(0.0, 1.0).check(torch.tensor([0.0, 0.5, 1.0])).all() and bool(Dn.positive.check(torch.tensor(1.0)))
    pn, qn = Dn.Normal(0.0, 1.0), Dn.Normal(1.0, 2.0)
    torch.testing.assert_close(Dn.kl_divergence_dyn(pn, qn), Dn.kl_divergence(pn, qn))
    torch.testing.assert_close(Dn.try_kl_expfamily(pn, qn), Dn.kl_divergence(pn, qn))
    assert Dn.try_kl_expfamily(pn, Dn.Gamma(1.0, 1.0)) is None
    assert Pf.estimate("matmul", [[4, 5], [5, 6]]) == 240 and Pf.estimate("my_custom_op", [[3, 4]]) is None


def test_jit_lowering_functions_onnx_dynamic_dims_and_nccl_named_helpers():
    # ferrotorch-jit/src/{codegen_ir,dag_fusion,codegen_jit}.rs; ferrotorch-serialize/src/onnx_export.rs:336-370;
    # ferrotorch-optim/src/foreach_utils.rs; ferrotorch-distributed/src/{nccl_sys,nccl_backend,nccl_collective}.rs
    import multiprocessing as mp
    import socket

    from ferrotorch_b200 import jit as J
    from ferrotorch_b200 import parallel as Pl
    from ferrotorch_b200 import serialize as S
    from ferrotorch_b200.serialize import onnx as X

    assert J.is_elementwise("relu") and J.is_binary_elementwise("add") and J.is_reduction("sum") and not J.is_elementwise("matmul")
    assert J.ir_op_to_unary("exp") is J.UnaryOpKind.Exp and J.ir_op_to_binary("relu") is None
    a, b = torch.randn(4), torch.randn(4)
    loops = J.lower_to_loops([("mul_c", 2.0), "relu", "add", "sum"], 2)
    assert loops[-1] == ("reduce", "sum") and J.jit_supports(loops)
    torch.testing.assert_close(J.CpuCodegen().compile(loops[0], "t")(a, b), torch.relu(a * 2) + b)
    with pytest.raises(J.JitError):
        J.lower_to_loops(["add"], 1)
    with pytest.raises(J.JitError):
        J.lower_to_loops(["sum", "relu"], 1)
    mm = J.lower_matmul(2, 3, 4)
    assert mm.flops() == 48 and mm.run(torch.ones(2, 3), torch.ones(3, 4)).shape == (2, 4) and "acc +=" in mm.source()
    assert J.jit_supports([mm]) and not J.jit_supports([mm, "something else"])
    e = J.apply_binary_op_expr("mul", J.apply_op_expr("exp", J.Expr.var(1)), J.Expr.var(0))
    torch.testing.assert_close(J.CpuCodegen().compile(J.LoopIR(2, e), "u")(a, b), torch.exp(b) * a)

    def f(x, y):
        return torch.relu(x * 2 + y).exp()

    compiled = J.compile(f, (a, b))
    groups = J.find_fusion_groups(compiled.graph)
    assert len(groups) == 1 and isinstance(J.fuse_dag(groups, compiled.graph)[0][0], J.LoopIR)
    raw = J.trace(f, (a, b))
    assert len(J.find_fusion_groups(raw)) == 1 and raw.count("fused_elementwise") == 0          # the caller's graph is untouched
    with pytest.raises(J.JitError):
        J.apply_fused_gpu(["relu"], a)
    w1 = X.encode_value_info("x", torch.float32, (1, 3), {0: "batch"}).finish()
    assert w1 == S.encode_value_info_dynamic("x", torch.float32, ["batch", 3]).finish() == S.encode_value_info_dynamic("x", 1, ["batch", 3]).finish()
    assert S.encode_dim_param("n").finish() == b"\x12\x01n" and len(S.encode_shape_with_dynamic([2, "n"]).finish()) == 9
    assert O.elemwise_max(torch.tensor([1.0, 5.0]), torch.tensor([3.0, 2.0])).tolist() == [3.0, 5.0]
    assert O.f64_scalar_on(0.1, "cpu").dim() == 0 and O.scalar_on(2, "cpu", torch.int64).dtype == torch.int64
    import torch.distributed as dist

    assert Pl.reduce_op_to_nccl(Pl.ReduceOp.Mean) == dist.ReduceOp.AVG and Pl.reduce_op_to_nccl("sum") == dist.ReduceOp.SUM
    assert Pl.is_available() == (torch.cuda.is_available() and dist.is_nccl_available()) and len(Pl.get_unique_id()) == 128
    Pl.group_start()
    Pl.group_end()
    with pytest.raises(Pl.DistributedError):
        Pl.group_end()
    # two processes join a communicator by id and reduce over it
    from dist_workers import comm_init_rank_worker

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    uid = bytes(Pl.get_unique_id())
    procs = [ctx.Process(target=comm_init_rank_worker, args=(r, 2, port, uid, q)) for r in range(2)]
    [p.start() for p in procs]
    got = sorted(q.get(timeout=120) for _ in procs)
    [p.join(60) for p in procs]
    assert got == [(0, 2, 3.0), (1, 2, 3.0)] and all(p.exitcode == 0 for p in procs)
