"""Learner, callbacks, metrics, TensorBoard writer, profiler, memory guard, data utilities."""
import json
import os
import struct
import time

import pytest
import torch
from torch import nn

from ferrotorch_b200 import data as D
from ferrotorch_b200 import profiler as P
from ferrotorch_b200 import train as T
from ferrotorch_b200.train import tensorboard as TB
from ferrotorch_b200.utils.memory_guard import MemoryBudgetExceeded, MemoryGuard, OomPolicy


def _loaders():
    torch.manual_seed(0)
    x = torch.randn(96, 8)
    y = (x[:, 0] + x[:, 1] > 0).long()
    ds = D.TensorDataset(x, y)
    return D.DataLoader(ds, batch_size=16, shuffle=False), D.DataLoader(ds, batch_size=32)


def test_learner_fit_checkpoint_resume_and_callbacks(tmp_path):
    tr, va = _loaders()
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    opt = torch.optim.Adam(model.parameters(), lr=5e-2)
    logs = []
    learner = T.Learner(model, opt, nn.CrossEntropyLoss(), scheduler=torch.optim.lr_scheduler.StepLR(opt, 2, 0.5),
                        metrics=[T.LossMetric(), T.AccuracyMetric(), T.TopKAccuracy(2), T.RunningAverage()],
                        callbacks=[T.ProgressLogger(3, logs.append), T.EMACallback(0.9),
                                   T.TensorBoardCallback(str(tmp_path / "tb")), T.EarlyStopping("accuracy", 50, "max")],
                        max_grad_norm=1.0, checkpoint_dir=str(tmp_path / "ck"))
    hist = learner.fit(tr, va, epochs=4)
    assert len(hist.epochs) == 4 and hist.epochs[-1].train["loss"] < hist.epochs[0].train["loss"]
    assert hist.epochs[-1].val["accuracy"] > 0.8 and hist.epochs[-1].val["top2_accuracy"] == 1.0
    assert hist.epochs[2].lr == pytest.approx(5e-2 * 0.5) and hist.best("accuracy", "val", "max") is not None
    assert logs and os.path.exists(str(tmp_path / "ck" / "checkpoint_epoch_3.ftc"))
    recs = TB.read_records(learner.callbacks[2].w.path)
    assert b"brain.Event:2" in recs[0] and any(b"train/loss" in r for r in recs)
    # resume into a fresh learner: same weights, epoch counter continues
    model2 = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 2))
    l2 = T.Learner(model2, torch.optim.Adam(model2.parameters(), lr=5e-2), nn.CrossEntropyLoss())
    l2.load_checkpoint(str(tmp_path / "ck" / "checkpoint_epoch_3.ftc"))
    assert l2.epoch == 4 and l2.global_step == learner.global_step
    for a, b in zip(model.parameters(), model2.parameters()):
        assert torch.equal(a, b)
    assert l2.evaluate(va)["loss"] == pytest.approx(hist.epochs[-1].val["loss"], rel=1e-5)


def test_early_stopping_and_checkpoint_sequential():
    tr, va = _loaders()
    model = nn.Linear(8, 2)
    learner = T.Learner(model, torch.optim.SGD(model.parameters(), lr=0.0), nn.CrossEntropyLoss(),
                        callbacks=[T.EarlyStopping("loss", patience=2)])
    assert len(learner.fit(tr, va, epochs=10).epochs) == 3
    layers = [nn.Linear(4, 4) for _ in range(5)]
    x = torch.randn(3, 4, requires_grad=True)
    y = T.checkpoint_sequential(layers, 2, x)
    ref = x
    for l in layers:
        ref = l(ref)
    assert torch.allclose(y, ref)
    y.sum().backward()
    assert x.grad is not None


def test_tensorboard_record_format():
    assert TB.crc32c(b"123456789") == 0xE3069283
    ev = TB.encode_scalar_event("loss", 1.5, 7, 100.0)
    rec = TB.record(ev)
    (n,) = struct.unpack_from("<Q", rec, 0)
    assert n == len(ev) and struct.unpack_from("<I", rec, 8)[0] == TB.masked_crc(rec[:8])
    assert b"loss" in ev and struct.pack("<f", 1.5) in ev


def test_profiler_scopes_schedule_and_reports(tmp_path):
    ready = []
    sched = P.ProfileSchedule(wait=1, warmup=1, active=2, repeat=1, on_trace_ready=lambda p: ready.append(len(p.events)))

    def work(p):
        for _ in range(5):
            with P.profile_op_scope("matmul", shapes=((8, 16), (16, 4))):
                torch.randn(8, 16) @ torch.randn(16, 4)
            p.step()
        p.record("manual", 12.0)
        p.record_memory("after", 1024)
        return 42

    r, prof = P.with_profiler(work, P.ProfileConfig(), sched)
    assert r == 42 and ready and sched.state() == "done"
    s = prof.summary()[("matmul", "cpu")]
    assert s["count"] == 2 and s["flops"] == 2 * (2.0 * 8 * 16 * 4)   # only the two active steps
    assert "matmul" in prof.table()
    trace = json.loads(prof.chrome_trace_json())
    assert any(e["name"] == "matmul" and e["ph"] == "X" for e in trace["traceEvents"])
    prof.export_chrome_trace(str(tmp_path / "t.json"))
    prof.export_tensorboard(str(tmp_path / "tb"))
    assert P.estimate_flops("attention", ((2, 128, 8, 64), (2, 256, 2, 64))) == 4.0 * 2 * 8 * 128 * 256 * 64
    with P.profile_op_scope("nothing installed"):
        pass


class _FakeAlloc:
    def __init__(self, total):
        self.total, self.used, self.cache = total, 0, 0

    def used_bytes(self):
        return self.used + self.cache

    def total_bytes(self):
        return self.total

    def empty_cache(self):
        self.cache = 0


def test_memory_guard_policies_hooks_watchdog():
    a = _FakeAlloc(1000)
    g = MemoryGuard(a, reserve_bytes=100, policy=OomPolicy.RUN_HOOKS_THEN_FAIL, pressure_threshold=0.8)
    a.used, a.cache = 500, 200
    assert g.available() == 200
    order = []
    g.add_pre_oom_hook(lambda need: order.append("low") or 0, priority=1)

    def free_acts(need):
        if "high" in order:
            return 0
        order.append("high")
        a.used -= 150
        return 150

    g.add_pre_oom_hook(free_acts, priority=10)
    g.ensure(300)                       # high-priority hook frees enough
    assert order == ["high"] and g.stats["freed_by_hooks"] == 150
    g.ensure(500)                       # hooks not enough, empty_cache makes room
    assert a.cache == 0
    called = []
    g.set_emergency_checkpoint(lambda: called.append(1))
    with pytest.raises(MemoryBudgetExceeded):
        g.ensure(5000)
    assert called and g.stats["failures"] == 1
    with pytest.raises(MemoryBudgetExceeded):
        MemoryGuard(a, policy=OomPolicy.FAIL).ensure(10_000)
    seen = []
    g.add_pressure_listener(seen.append)
    a.used = 850
    g.start_watchdog(0.01)
    import time

    time.sleep(0.15)
    assert not g.wait_if_paused(0.2) and seen and g.stats["pauses"] >= 1
    a.used = 100
    assert g.wait_if_paused(1.0)
    g.stop_watchdog()
    w = MemoryGuard(a, policy=OomPolicy.WAIT, wait_timeout_s=0.05)
    with pytest.raises(MemoryBudgetExceeded):
        w.ensure(10_000)


def test_data_utilities():
    ds = D.SyntheticTokens(100, 16, 10, seed=3)
    x, y = ds[4]
    x2, _ = ds[4]
    assert x.shape == (16,) and torch.equal(x[1:], y[:-1]) and torch.equal(x, x2)
    img, label = D.SyntheticImages(4, num_classes=10, size=8)[1]
    assert img.shape == (3, 8, 8) and 0 <= label < 10
    assert sorted(D.shuffle_with_seed(10, 1)) == list(range(10)) and D.shuffle_with_seed(10, 1) == D.shuffle_with_seed(10, 1)
    s0 = list(D.DistributedSampler(ds, num_replicas=2, rank=0, shuffle=False))
    s1 = list(D.DistributedSampler(ds, num_replicas=2, rank=1, shuffle=False))
    assert sorted(s0 + s1) == list(range(10))
    batches = list(D.DevicePrefetcher(D.DataLoader(ds, batch_size=4), "cpu"))
    assert len(batches) == 3 and batches[0][0].shape == (4, 16)


def test_observers_fake_quant_and_qat():
    import torch
    from torch import nn

    from ferrotorch_b200.nn import fake_quant as qat

    obs = qat.MinMaxObserver(8, symmetric=False)
    obs(torch.tensor([-1.0, 0.5, 3.0]))
    obs(torch.tensor([-2.0, 1.0]))
    scale, zero, qmin, qmax = obs.qparams()
    assert (qmin, qmax) == (0, 255) and float(scale) == pytest.approx(5.0 / 255) and float(zero) == round(2.0 / (5.0 / 255))
    pc = qat.MinMaxObserver(8, True, ch_axis=0)
    pc(torch.tensor([[1.0, -4.0], [0.5, 0.25]]))
    assert pc.qparams()[0].tolist() == pytest.approx([4.0 / 127, 0.5 / 127])
    ma = qat.MovingAverageObserver(momentum=0.5)
    ma(torch.tensor([0.0, 2.0]))
    ma(torch.tensor([0.0, 4.0]))
    assert float(ma.max_val) == pytest.approx(3.0)

    # straight-through gradient: 1 inside the range, 0 where the value was clipped
    fq = qat.FakeQuantize(4, True)
    fq.observer(torch.tensor([-1.0, 1.0]))
    fq.observe = False
    x = torch.tensor([0.3, 5.0, -0.7], requires_grad=True)
    y = fq(x)
    y.sum().backward()
    assert x.grad.tolist() == [1.0, 0.0, 1.0]
    assert float((y[0] - 0.3).abs()) <= float(fq.observer.qparams()[0]) / 2 + 1e-6

    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 4))
    ref = [p.detach().clone() for p in net.parameters()]
    qat.prepare_qat(net)
    assert isinstance(net[0], qat.QatLinear) and isinstance(net[2], qat.QatLinear)
    assert all(torch.equal(a, b) for a, b in zip(ref, [net[0].weight, net[0].bias, net[2].weight, net[2].bias]))
    opt = torch.optim.SGD(net.parameters(), 0.05)
    xs, ys = torch.randn(64, 16), torch.randint(0, 4, (64,))
    first = None
    for _ in range(40):
        loss = nn.functional.cross_entropy(net(xs), ys)
        first = first if first is not None else float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < first
    ints = qat.convert(net)
    q, sc, b = ints["0"]
    assert q.dtype == torch.int8 and q.shape == (32, 16)
    assert float((q.float() * sc[:, None] - net[0].weight).abs().max()) <= float(sc.max()) / 2 + 1e-6


def test_parity_sweep_harness_cpu():
    from ferrotorch_b200.utils import parity

    rows = parity.sweep(["rmsnorm", "swiglu", "attention"], "cpu")
    assert [r["op"] for r in rows] == ["rmsnorm", "swiglu", "attention"]
    assert all(r["ok"] and r["shapes"] >= 2 for r in rows)


def test_resume_after_the_trainer_process_dies(tmp_path):
    """Kill the training process between steps (os._exit, no clean-up); a new process resumes from
    the last asynchronously written checkpoint and ends with the same weights as an unbroken run."""
    import subprocess
    import sys
    import textwrap

    script = tmp_path / "train.py"
    script.write_text(textwrap.dedent('''
        import os, sys
        sys.path.insert(0, %r)
        import torch
        from ferrotorch_b200.serialize.state import AsyncCheckpointer, load_checkpoint

        ckpt, die_at, total = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 1))
        opt = torch.optim.AdamW(model.parameters(), lr=0.05)
        step = 0
        if os.path.exists(ckpt):
            ck = load_checkpoint(ckpt)
            model.load_state_dict(ck["model"])
            opt.load_state_dict(ck["optimizer"])
            step = ck["step"]
        writer = AsyncCheckpointer()
        g = torch.Generator().manual_seed(123)
        data = [(torch.randn(32, 8, generator=g), torch.randn(32, 1, generator=g)) for _ in range(total)]
        while step < total:
            x, y = data[step]
            loss = torch.nn.functional.mse_loss(model(x), y)
            opt.zero_grad(); loss.backward(); opt.step()
            step += 1
            writer.save_async(ckpt, model.state_dict(), opt.state_dict(), step=step).wait()
            if step == die_at:
                os._exit(17)
        torch.save([p.detach() for p in model.parameters()], ckpt + ".final")
    ''') % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    run = lambda ck, die: subprocess.run([sys.executable, str(script), str(ck), str(die), "8"], timeout=120).returncode  # noqa: E731
    assert run(tmp_path / "a.ckpt", 5) == 17          # died after step 5
    assert run(tmp_path / "a.ckpt", -1) == 0          # resumed at step 5, ran to 8
    assert run(tmp_path / "b.ckpt", -1) == 0          # unbroken reference
    wa, wb = torch.load(str(tmp_path / "a.ckpt") + ".final"), torch.load(str(tmp_path / "b.ckpt") + ".final")
    assert all(torch.equal(x, y) for x, y in zip(wa, wb))


def test_native_token_loader(tmp_path):
    from ferrotorch_b200.data import TokenFileLoader, write_token_file

    S, B = 16, 4
    n_samples = 50
    ids = torch.arange(n_samples * S + 1) % 60000
    path = str(tmp_path / "tokens.bin")
    assert write_token_file(path, ids) == 2

    def epoch_samples(loader):
        out = []
        for x, y in loader:
            assert x.shape == (B, S) and y.shape == (B, S) and x.dtype == torch.int64
            assert torch.equal(x[:, 1:], y[:, :-1])                       # labels are the inputs shifted by one
            assert torch.equal(x, (x[:, :1] + torch.arange(S)) % 60000)   # a window of the file
            out += (x[:, 0] // S).tolist()
        return out

    a = TokenFileLoader(path, S, B, num_workers=1, prefetch=2, seed=7)
    b = TokenFileLoader(path, S, B, num_workers=6, prefetch=5, seed=7)
    assert a.num_samples == n_samples and len(a) == n_samples // B
    e0a, e0b = epoch_samples(a), epoch_samples(b)
    assert e0a == e0b                                   # thread count does not change the order
    assert len(set(e0a)) == len(e0a) == (n_samples // B) * B and set(e0a) <= set(range(n_samples))
    e1a, e1b = epoch_samples(a), epoch_samples(b)
    assert e1a == e1b and e1a != e0a and a.epoch == 1   # a new permutation every epoch
    assert epoch_samples(TokenFileLoader(path, S, B, seed=8)) != e0a
    assert epoch_samples(TokenFileLoader(path, S, B, shuffle=False)) == list(range((n_samples // B) * B))

    # rank sharding: disjoint, and together one permutation prefix
    r0 = epoch_samples(TokenFileLoader(path, S, B, seed=7, rank=0, world_size=2))
    r1 = epoch_samples(TokenFileLoader(path, S, B, seed=7, rank=1, world_size=2))
    assert not set(r0) & set(r1) and len(r0) == len(r1) == (n_samples // (2 * B)) * B

    # uint32 ids and errors
    big = torch.tensor([70000, 1, 2, 3, 4, 5, 6, 7, 8], dtype=torch.int64)
    p2 = str(tmp_path / "big.bin")
    assert write_token_file(p2, big) == 4
    x, y = TokenFileLoader(p2, 4, 2, dtype_bytes=4, shuffle=False).next_batch()
    assert x.tolist() == [[70000, 1, 2, 3], [4, 5, 6, 7]] and y.tolist() == [[1, 2, 3, 4], [5, 6, 7, 8]]
    with pytest.raises(ValueError):
        TokenFileLoader(p2, 4, 64, dtype_bytes=4)
    with pytest.raises(ValueError):
        TokenFileLoader(str(tmp_path / "missing.bin"), 4, 2)


def test_arrow_and_dataframe_interop():
    pa = pytest.importorskip("pyarrow")
    pd = pytest.importorskip("pandas")
    from ferrotorch_b200 import data as D

    t = torch.arange(5, dtype=torch.float64)
    arr = D.tensor_to_arrow_array(t)
    assert str(arr.type) == "double" and arr.to_pylist() == [0.0, 1.0, 2.0, 3.0, 4.0]
    back = D.tensor_from_arrow_array(arr)
    assert back.dtype == torch.float64 and torch.equal(back, t)
    assert D.tensor_from_arrow_array(pa.chunked_array([[1, 2], [3]]), torch.float32).tolist() == [1.0, 2.0, 3.0]
    with pytest.raises(ValueError, match="nulls"):
        D.tensor_from_arrow_array(pa.array([1.0, None]))
    with pytest.raises(ValueError, match="unsupported"):
        D.tensor_from_arrow_array(pa.array(["a"]))
    with pytest.raises(ValueError):
        D.tensor_to_arrow_array(torch.zeros(2, 2))
    rb = pa.record_batch({"a": [1, 2, 3], "b": [0.5, 1.5, 2.5]})
    assert D.record_batch_to_tensor(rb).tolist() == [[1.0, 0.5], [2.0, 1.5], [3.0, 2.5]]
    assert D.record_batch_to_tensor(pa.Table.from_batches([rb, rb])).shape == (6, 2)
    df = pd.DataFrame({"x": [1, 2], "y": [0.25, 0.75]})
    assert D.dataframe_to_tensor(df, torch.float64).tolist() == [[1.0, 0.25], [2.0, 0.75]]
    with pytest.raises(ValueError, match="non-numeric"):
        D.dataframe_to_tensor(pd.DataFrame({"x": ["a"]}))
    with pytest.raises(ValueError, match="missing"):
        D.dataframe_to_tensor(pd.DataFrame({"x": [1.0, None]}))


def test_name_level_parity_helpers(tmp_path):
    """Small pieces that exist so that every public name of the reference's train / profiler /
    serialize / optim crates has a counterpart."""
    import ferrotorch_b200.optim as O
    import ferrotorch_b200.serialize as S

    # train
    assert T.EmaCallback is T.EMACallback and T.EvalResult({"loss": 0.5}, 3).get("loss") == 0.5
    lin = nn.Linear(3, 3)
    x = torch.randn(2, 3, requires_grad=True)
    T.checkpoint(lambda t: lin(t).relu(), x).sum().backward()
    assert x.grad is not None and float(T.clip_grad_norm_(lin.parameters(), 1e-3)) > 0
    T.clip_grad_value_(lin.parameters(), 1e-4)
    assert float(lin.weight.grad.abs().max()) <= 1e-4
    # profiler
    prof = P.Profiler()
    with P.CudaKernelScope(prof, "step", "kernel"):
        torch.randn(64, 64) @ torch.randn(64, 64)
    prof.record("copy", 12.0)
    prof.record_memory(P.MemoryCategory.ACTIVATIONS, 1024)
    rep = prof.report()
    names = [o.name for o in rep.ops()]
    assert set(names) == {"step", "copy"} and rep.top(1)[0].count == 1 and rep.total_us() >= 12.0
    assert "step" in rep.table() and json.loads(rep.chrome_trace_json())["traceEvents"]
    rep.save_chrome_trace(str(tmp_path / "t.json"))
    assert P.SchedulePhase.ACTIVE == P.ProfileSchedule(0, 0, 1).state() and P.OpSummary("a", "cpu", 2, 10.0).avg_us == 5.0
    # serialize
    sd = {"a.w": torch.randn(2, 2), "b.w": torch.randn(3)}
    S.save_safetensors_sharded(sd, str(tmp_path / "ck"), max_shard_bytes=16)
    idx = str(tmp_path / "ck" / "model.safetensors.index.json")
    seen = []
    full = S.load_safetensors_sharded_with_progress(idx, seen.append)
    assert set(full) == set(sd) and seen[-1].tensors_loaded == 2 and seen[-1].shard_count == len(seen) == 2
    assert list(S.load_safetensors_sharded_filtered(idx, lambda k: k.startswith("b."))) == ["b.w"]
    assert set(S.load_safetensors_auto(str(tmp_path / "ck"))) == set(sd) and set(S.load_safetensors_auto(idx)) == set(sd)
    S.save_safetensors(sd, str(tmp_path / "one.safetensors"))
    assert torch.equal(S.load_safetensors_auto(str(tmp_path / "one.safetensors"))["b.w"], sd["b.w"])
    assert torch.equal(S.load_safetensors_mmap(str(tmp_path / "one.safetensors"))["a.w"], sd["a.w"])
    with pytest.raises(FileNotFoundError):
        S.load_safetensors_auto(str(tmp_path))
    S.save_pytorch(sd, str(tmp_path / "m.pt"))
    assert S.validate_checkpoint(str(tmp_path / "m.pt")) == {"tensors": 2, "parameters": 7, "dtypes": ["torch.float32"]}
    torch.save({"evil": object()}, str(tmp_path / "bad.pt"))
    with pytest.raises(Exception):
        S.validate_checkpoint(str(tmp_path / "bad.pt"))                # arbitrary pickled objects are refused
    assert S.OnnxExportConfig(opset_version=17).opset_version == 17
    # optim: differentiable steps let an outer loss see through the update
    assert O.ExponentialMovingAverage is O.EMA and O.Kfac is not O.NaturalGradient      # Kronecker-factored vs its diagonal reduction
    w = torch.tensor([1.0, -2.0], requires_grad=True)
    lr = torch.tensor(0.1, requires_grad=True)
    (g,) = torch.autograd.grad((w ** 2).sum(), w, create_graph=True)
    (w1,) = O.diff_sgd_step([w], [g], lr)
    (w1 ** 2).sum().backward()
    assert lr.grad.item() == pytest.approx(-2 * (1 - 0.2) * 2 * 5.0, rel=1e-5)      # d/dlr sum((w (1 - 2 lr))^2)
    (w2,), (b2,) = O.diff_sgd_momentum_step([w.detach()], [g.detach()], [torch.ones(2)], 0.1, 0.5)
    assert torch.allclose(b2, 0.5 + g.detach()) and torch.allclose(w2, w.detach() - 0.1 * b2)


def test_memory_guard_builder_levels_hooks_and_safe_alloc():
    from ferrotorch_b200.utils.memory_guard import (MemoryBudgetExceeded, MemoryGuardBuilder, OomPolicy, PressureLevel)

    class Fake:
        used = 0

        def used_bytes(self):
            return self.used

        def total_bytes(self):
            return 1000

        def empty_cache(self):
            pass

    a = Fake()
    g = MemoryGuardBuilder().budget_bytes(1000).reserve_bytes(200).oom_policy(OomPolicy.RetryAfterFree).build(a)
    assert g.has_reservation() and g.reserved_bytes() == 200 and g.available() == 800
    assert [PressureLevel.of(p) for p in (0.1, 0.5, 0.7, 0.85, 0.95)] == list(PressureLevel)
    moves = []
    g.add_level_listener(lambda old, new: moves.append((old.name, new.name)))
    a.used = 600                                        # 600 / 800 usable = 75 %
    assert g.notify_pressure_change() == PressureLevel.MEDIUM and g.notify_pressure_change() == PressureLevel.MEDIUM
    a.used = 790
    g.notify_pressure_change()
    assert moves == [("NONE", "MEDIUM"), ("MEDIUM", "CRITICAL")]
    freed = []

    def drop_cache(need):
        freed.append(need)
        a.used -= 500
        return 500

    hid = g.register_hook(drop_cache, priority=5, name="cache")
    t = g.safe_alloc((50,), torch.float32)              # 200 bytes: needs the hook (only 10 available)
    assert t.shape == (50,) and freed == [190] and a.used == 290
    st = g.memory_stats()
    assert st["peak_bytes"] >= 290 and st["level"] == "NONE" and st["hook_runs"] == 1 and st["budget_bytes"] == 1000
    assert g.remove_hook(hid) and not g.remove_hook(hid)
    with pytest.raises(MemoryBudgetExceeded):
        g.safe_alloc((1000,), torch.float32)
    g.release_reservation()
    assert not g.has_reservation() and g.available() == 710
    g.set_budget(2000)
    g.set_oom_policy(OomPolicy.Fail)
    assert g.available() == 1710 and g.policy is OomPolicy.FAIL
    g.reset_peak_stats()
    assert g.memory_stats()["peak_bytes"] == 290
    with pytest.raises(ValueError):
        MemoryGuardBuilder().budget_bytes(100).reserve_bytes(100).build(a)


def test_cuda_vocabulary_degrades_cleanly_without_a_gpu():
    from ferrotorch_b200 import cuda as C

    assert [C.round_len(n) for n in (0, 1, 512, 513, (1 << 20) - 1, 1 << 20, (2 << 20) + 1)] == \
        [512, 512, 512, 1024, 1 << 20, 2 << 20, 4 << 20]
    assert C.MemoryGuardBuilder is not None and C.PressureLevel.CRITICAL == 4
    a = torch.rand(3)
    with C.fork_rng():
        torch.manual_seed(5)
        inside = torch.rand(3)
    after = torch.rand(3)
    torch.manual_seed(5)
    assert torch.equal(inside, torch.rand(3)) and not torch.equal(after, inside) and a is not None
    if not C.is_available():
        assert C.cached_bytes() == 0 and not C.is_stream_capturing()
        C.empty_cache()
        for call in (lambda: C.GpuDevice(0), lambda: C.cuda(a), lambda: C.alloc_zeros((2,)), C.graph_pool_handle,
                     lambda: C.make_graphed_callable(lambda t: t, (a,))):
            with pytest.raises(C.GpuError):
                call()
    assert torch.equal(C.tensor_to_cpu(a), a)


def test_parity_sweep_extended_cases_and_audit_file(tmp_path):
    import subprocess
    import sys

    from ferrotorch_b200.utils import parity

    rows = parity.sweep(["linear_bwd", "rope", "q4_0_linear", "linear_cross_entropy"], "cpu", random_shapes=1)
    assert [r["op"] for r in rows] == ["linear_bwd", "rope", "q4_0_linear", "linear_cross_entropy"] and all(r["ok"] for r in rows)
    assert rows[0]["shapes"] == 3 and rows[2]["shapes"] == 2            # tile-edge shapes only where the op takes any size
    assert len(parity.sweep(None, "cpu")) == 5 and len(parity.sweep(None, "cpu", extended=True)) == 14
    with pytest.raises(KeyError):
        parity.sweep(["nope"], "cpu")
    shapes = parity._edge_shapes((300, 264, 16), 5, seed=1)
    assert all(s[2] == 16 and s[1] % 8 == 0 and abs((s[0] + 3) % 128 - 3) <= 3 for s in shapes)
    out = tmp_path / "audit.json"
    proc = subprocess.run([sys.executable, "-m", "ferrotorch_b200.utils.parity", "--device", "cpu", "--ops", "swiglu_bwd",
                           "--out", str(out)], capture_output=True, text=True, timeout=300,
                          cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert proc.returncode == 0, proc.stderr[-2000:]
    audit = json.loads(out.read_text())
    assert audit["rows"][0]["op"] == "swiglu_bwd" and audit["rows"][0]["ok"]


def test_learner_drives_a_flat_trainer(tmp_path):
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.train.engine import FlatTrainer

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                      num_key_value_heads=1)
    model = LlamaForCausalLM(cfg)
    trainer = FlatTrainer(model, lr=5e-3, weight_decay=0.0, max_grad_norm=1.0)
    g = torch.Generator().manual_seed(1)
    batches = [torch.randint(0, 64, (4, 9), generator=g) for _ in range(4)]
    data = [(b[:, :-1], b[:, 1:]) for b in batches]
    seen = []

    class Spy(T.Callback):
        def on_batch_end(self, learner, epoch, batch, loss):
            seen.append(float(loss))

    lr = T.Learner(model, None, None, trainer=trainer, callbacks=[Spy()], checkpoint_dir=str(tmp_path))
    hist = lr.fit(data, val_data=data, epochs=3)
    assert len(seen) == 12 and lr.global_step == 12 and len(hist.epochs) == 3
    assert hist.epochs[-1].train["loss"] < hist.epochs[0].train["loss"] and hist.epochs[-1].val["loss"] < hist.epochs[0].val["loss"]
    assert hist.epochs[0].lr == 5e-3 and (tmp_path / "checkpoint_epoch_2.ftc").exists()
    # resume: a fresh model + trainer continue from the checkpoint with the same next-step loss
    torch.manual_seed(0)
    model2 = LlamaForCausalLM(cfg)
    trainer2 = FlatTrainer(model2, lr=5e-3, weight_decay=0.0, max_grad_norm=1.0)
    lr2 = T.Learner(model2, None, None, trainer=trainer2)
    lr2.load_checkpoint(str(tmp_path / "checkpoint_epoch_2.ftc"))
    assert lr2.epoch == 3 and lr2.global_step == 12
    a = float(trainer.step(*data[0]))
    b = float(trainer2.step(*data[0]))
    assert a == pytest.approx(b, rel=1e-5)


# --------------------------------------------------------------------------- run metrics (JSON lines per rank)
def test_metrics_logger_reports_job_rate_from_the_slowest_rank(tmp_path):
    import threading

    from ferrotorch_b200.parallel.backend import SimulatedGroup
    from ferrotorch_b200.train import MetricsLogger, read_metrics

    groups = SimulatedGroup.create_group(2)
    out = {}

    def rank(r):
        log = MetricsLogger(str(tmp_path), group=groups[r], unit="tokens", every=4, flops_per_item=100.0, peak_flops=1e6)
        for _ in range(8):
            log.begin_step()
            time.sleep(0.004 * (1 + r))                  # rank 1 is twice as slow
            log.end_step(items=1000, loss=torch.tensor(2.5), exposed_comm_ms=1.0)
        log.close()
        out[r] = log.reports

    ts = [threading.Thread(target=rank, args=(r,)) for r in range(2)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert len(out[0]) == len(out[1]) == 2
    for a, b in zip(out[0], out[1]):
        # both ranks report the same job: the slowest rank's step time, the sum of the items
        assert a.ms_per_step_max_over_ranks == b.ms_per_step_max_over_ranks == max(a.ms_per_step, b.ms_per_step)
        assert a.items_per_s == b.items_per_s
        assert abs(a.items_per_s - 2 * 4 * 1000 / (4 * a.ms_per_step_max_over_ranks / 1e3)) < 1e-6 * a.items_per_s
        assert a.ms_per_step < b.ms_per_step
        assert abs(a.flop_utilisation - a.items_per_s * 100.0 / 2e6) < 1e-12
        assert 0 < b.exposed_comm_frac < a.exposed_comm_frac < 1
    for r in range(2):
        rows = read_metrics(str(tmp_path / ("metrics_rank%d.jsonl" % r)))
        assert [row["step"] for row in rows] == [4, 8] and rows[0]["rank"] == r and rows[0]["unit"] == "tokens/s"
        assert rows[0]["loss"] == 2.5 and rows[0]["world_size"] == 2


def test_metrics_callback_logs_learner_batches_and_tensorboard_scalars(tmp_path):
    from ferrotorch_b200.train import Learner, MetricsCallback, MetricsLogger, TensorBoardWriter, read_metrics

    torch.manual_seed(0)
    model = torch.nn.Linear(6, 3)
    data = [(torch.randn(5, 6), torch.randint(0, 3, (5,))) for _ in range(6)]
    tb = TensorBoardWriter(str(tmp_path / "tb"))
    log = MetricsLogger(str(tmp_path), unit="samples", every=3, tensorboard=tb)
    Learner(model, torch.optim.SGD(model.parameters(), lr=0.1), torch.nn.functional.cross_entropy, callbacks=[MetricsCallback(log)],
            device="cpu").fit(data, epochs=2)
    tb.close()
    rows = read_metrics(log.path)
    assert [r["step"] for r in rows] == [3, 6, 9, 12] and all(r["steps_in_window"] == 3 for r in rows)
    assert all(r["items_per_s"] > 0 and r["ms_per_step"] == r["ms_per_step_max_over_ranks"] for r in rows)
    assert {r["epoch"] for r in rows} == {0, 1} and "exposed_comm_frac" not in rows[0]
    blob = b"".join(open(os.path.join(tmp_path / "tb", f), "rb").read() for f in os.listdir(tmp_path / "tb"))
    assert b"throughput/samples_per_s" in blob and b"train/loss" in blob
