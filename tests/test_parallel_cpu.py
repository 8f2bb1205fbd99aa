"""Mesh / DTensor / pipeline / FSDP / SyncBatchNorm on simulated CPU ranks, and the optimizers."""
import copy

import pytest
import torch
from torch import nn

from ferrotorch_b200 import optim as O
from ferrotorch_b200.parallel import (DDP, FSDP, DeviceMesh, DTensor, InvalidRank, Partial, Pipeline, Replicate, Shard,
                                      ShardingStrategy, SyncBatchNorm2d, run_simulated)


def test_device_mesh_maps():
    m = DeviceMesh((2, 4), ("dp", "tp"))
    assert m.size == 8 and m.coords(5) == (1, 1) and m.rank_of((1, 1)) == 5
    assert m.ranks_along_dim(5, "tp") == [4, 5, 6, 7] and m.ranks_along_dim(5, "dp") == [1, 5]
    assert m.groups_along_dim("dp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    with pytest.raises(InvalidRank):
        m.coords(8)
    with pytest.raises(InvalidRank):
        m.rank_of((2, 0))


def test_dtensor_redistribute_moves_data():
    full = torch.arange(24, dtype=torch.float32).view(4, 6)

    def body(g):
        d = DTensor.from_global(full, g, Shard(0))
        assert d.local.shape == (2, 6)
        rep = d.redistribute(Replicate())
        col = d.redistribute(Shard(1))
        part = DTensor(torch.full((2, 2), float(g.rank + 1)), g, Partial("sum"))
        return rep.local, col.local, part.redistribute(Replicate()).local, part.redistribute(Shard(0)).local, \
            rep.redistribute(Shard(0)).local

    res = run_simulated(2, body)
    for r, (rep, col, ar, rs, back) in enumerate(res):
        assert torch.equal(rep, full) and torch.equal(col, full[:, r * 3:(r + 1) * 3])
        assert torch.equal(ar, torch.full((2, 2), 3.0)) and torch.equal(rs, torch.full((1, 2), 3.0))
        assert torch.equal(back, full[r * 2:(r + 1) * 2])


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_pipeline_matches_single_process(schedule):
    torch.manual_seed(0)
    stages = [nn.Sequential(nn.Linear(6, 8), nn.Tanh()), nn.Sequential(nn.Linear(8, 8), nn.Tanh()), nn.Linear(8, 3)]
    x, y = torch.randn(8, 6), torch.randn(8, 3)
    ref = copy.deepcopy(nn.Sequential(*stages))
    loss_ref = nn.functional.mse_loss(ref(x), y)
    loss_ref.backward()

    def body(g):
        m = copy.deepcopy(stages[g.rank])
        p = Pipeline(m, g, n_micro=4, schedule=schedule, loss_fn=nn.functional.mse_loss)
        loss = p.train_step(x if g.rank == 0 else None, y if g.rank == 2 else None)
        return loss, [q.grad.clone() for q in m.parameters()]

    res = run_simulated(3, body)
    assert abs(float(res[2][0]) - float(loss_ref)) < 1e-6
    for s in range(3):
        for got, want in zip(res[s][1], [q.grad for q in ref[s].parameters()]):
            assert torch.allclose(got, want, atol=1e-6), "stage %d input gradients must be real, not zeros" % s


@pytest.mark.parametrize("strategy,intra", [(ShardingStrategy.FULL_SHARD, None), (ShardingStrategy.SHARD_GRAD_OP, None),
                                            (ShardingStrategy.NO_SHARD, None), (ShardingStrategy.HYBRID_SHARD, 2)])
def test_fsdp_matches_ddp(strategy, intra):
    torch.manual_seed(1)
    base = nn.Sequential(nn.Linear(5, 7), nn.ReLU(), nn.Linear(7, 3))
    xs = torch.randn(4, 6, 5)

    def run(g, use_fsdp):
        m = copy.deepcopy(base)
        if use_fsdp:
            w = FSDP(m, g, strategy, intra_node_size=intra)
            opt = torch.optim.SGD(w.shard_parameters(), lr=0.1)
        else:
            w = DDP(m, g)
            opt = torch.optim.SGD(m.parameters(), lr=0.1)
        for _ in range(2):
            opt.zero_grad()
            w(xs[g.rank]).pow(2).mean().backward()
            w.sync_gradients()
            opt.step()
        return w.full_state_dict() if use_fsdp else {k: v.clone() for k, v in m.state_dict().items()}

    a, b = run_simulated(4, run, True), run_simulated(4, run, False)
    for r in range(4):
        for k in b[0]:
            assert torch.allclose(a[r][k], b[0][k], atol=1e-6), (strategy, k)


def test_sync_batch_norm_equals_big_batch():
    torch.manual_seed(2)
    x = torch.randn(8, 3, 4, 4)
    bn = nn.BatchNorm2d(3)
    xr = x.clone().requires_grad_()
    want = bn(xr)
    want.square().sum().backward()

    def body(g):
        m = SyncBatchNorm2d(3, g)
        xi = x[g.rank * 4:(g.rank + 1) * 4].clone().requires_grad_()
        out = m(xi)
        out.square().sum().backward()
        return out.detach(), xi.grad, m.running_mean.clone(), m.running_var.clone(), m.weight.grad

    res = run_simulated(2, body)
    out = torch.cat([r[0] for r in res])
    assert torch.allclose(out, want.detach(), atol=1e-5)
    assert torch.allclose(torch.cat([r[1] for r in res]), xr.grad, atol=1e-4)
    assert torch.allclose(res[0][2], bn.running_mean, atol=1e-6) and torch.allclose(res[0][3], bn.running_var, atol=1e-5)
    assert torch.allclose(res[0][4] + res[1][4], bn.weight.grad, atol=1e-4)


def test_fused_optimizers_match_torch_on_cpu():
    torch.manual_seed(3)
    for ours, theirs in [(lambda p: O.FusedAdamW(p, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1),
                          lambda p: torch.optim.AdamW(p, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)),
                         (lambda p: O.FusedSGD(p, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True),
                          lambda p: torch.optim.SGD(p, lr=0.1, momentum=0.9, weight_decay=1e-4, nesterov=True))]:
        a = nn.Sequential(nn.Linear(4, 5), nn.Linear(5, 2))
        b = copy.deepcopy(a)
        oa, ob = ours(a.parameters()), theirs(b.parameters())
        for _ in range(3):
            x = torch.randn(6, 4)
            for m, o in ((a, oa), (b, ob)):
                o.zero_grad()
                m(x).square().mean().backward()
                o.step()
        for p, q in zip(a.parameters(), b.parameters()):
            assert torch.allclose(p, q, atol=1e-6)
        sd = oa.state_dict()
        oa.load_state_dict(sd)


def test_extra_optimizers_and_schedules_reduce_loss():
    torch.manual_seed(4)
    x, y = torch.randn(64, 8), torch.randn(64, 1)
    for make in (lambda p: O.Muon(p, lr=0.02), lambda p: O.Adafactor(p, lr=1e-2), lambda p: O.NaturalGradient(p, lr=1e-2)):
        m = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))
        opt = make(m.parameters())
        first = None
        for _ in range(60):
            opt.zero_grad()
            loss = nn.functional.mse_loss(m(x), y)
            loss.backward()
            opt.step()
            first = first if first is not None else float(loss)
        assert float(loss) < first
    m = nn.Linear(2, 2)
    opt = torch.optim.SGD(m.parameters(), lr=1.0)
    sch = O.cosine_warmup_scheduler(opt, warmup_steps=2, total_steps=6, min_ratio=0.1)
    lrs = []
    for _ in range(7):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        sch.step()
    assert lrs[0] == 0.0 and lrs[2] == 1.0 and abs(lrs[6] - 0.1) < 1e-6 and lrs[3] > lrs[4] > lrs[5]
    ema = O.EMA(m, decay=0.5)
    with torch.no_grad():
        m.weight.add_(2.0)
    ema.update()
    ema.apply()
    applied = m.weight.detach().clone()
    ema.restore()
    assert torch.allclose(applied + 1.0, m.weight)
    acc = O.GradientAccumulator(3)
    assert [acc.backward(m(torch.ones(1, 2)).sum()) for _ in range(3)] == [False, False, True]
    assert O.StepLR is torch.optim.lr_scheduler.StepLR and O.GradScaler is not None


def test_p2p_verbs_probes_and_aliases():
    import ferrotorch_b200.parallel as P
    from ferrotorch_b200.parallel.backend import SelfSend, UnsupportedOp, run_simulated

    def body(g):
        peer = 1 - g.rank
        got = P.sendrecv(g, torch.full((3,), float(g.rank)), peer)
        if g.rank == 0:
            P.send(g, torch.arange(4.0), 1)
            extra = None
        else:
            extra = P.recv(g, (4,), 0)
        rs = P.async_reduce_scatter(g, torch.arange(4.0) * (g.rank + 1)).wait(10)
        try:
            P.send(g, torch.zeros(1), g.rank)
            own = "sent"
        except SelfSend:
            own = "refused"
        return got, extra, rs, own

    r0, r1 = run_simulated(2, body)
    assert r0[0].tolist() == [1.0] * 3 and r1[0].tolist() == [0.0] * 3 and r1[1].tolist() == [0.0, 1.0, 2.0, 3.0]
    assert r0[2].tolist() == [0.0, 3.0] and r1[2].tolist() == [6.0, 9.0] and r0[3] == r1[3] == "refused"
    assert P.is_gloo_available() and isinstance(P.is_nccl_available(), bool) and isinstance(P.is_ucc_available(), bool)
    assert isinstance(P.is_mpi_available(), bool)
    assert P.PipelineSchedule.OneFOneB.value == "1f1b" and P.Placement.Shard is P.Shard and P.async_all_gather is P.all_gather_async
    for fn in (P.gpu_allreduce, P.gpu_broadcast):
        with pytest.raises(UnsupportedOp):
            fn(torch.zeros(2))                      # host tensors are not silently bounced through the CPU path


@pytest.mark.parametrize("world", [2, 3, 5])
def test_portable_ring_algorithms_on_simulated_ranks(world):
    from ferrotorch_b200.parallel import ring
    from ferrotorch_b200.parallel.backend import InvalidRank, run_simulated

    def body(g):
        t = torch.arange(11, dtype=torch.float64) * (g.rank + 1)
        s = ring.ring_all_reduce(g, t.clone(), "sum")
        m = ring.ring_all_reduce(g, t.clone().view(11, 1), "mean")
        outs = []
        for root in range(g.world_size):
            b = torch.full((4,), float(g.rank))
            outs.append(ring.tree_broadcast(g, b, root).tolist())
        ring.ring_barrier(g)
        try:
            ring.tree_broadcast(g, torch.zeros(1), g.world_size)
            bad = "accepted"
        except InvalidRank:
            bad = "refused"
        return s, m, outs, bad

    tot = world * (world + 1) / 2
    for s, m, outs, bad in run_simulated(world, body):
        assert torch.allclose(s, torch.arange(11, dtype=torch.float64) * tot)
        assert torch.allclose(m.view(-1), torch.arange(11, dtype=torch.float64) * tot / world) and m.shape == (11, 1)
        assert outs == [[float(root)] * 4 for root in range(world)] and bad == "refused"


def test_fsdp_prefetch_overlaps_the_gather():
    from ferrotorch_b200.parallel.backend import run_simulated
    from ferrotorch_b200.parallel.fsdp import FSDP, ShardingStrategy

    import copy

    torch.manual_seed(0)
    proto = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))

    def body(g):
        m = copy.deepcopy(proto)                                     # every rank starts from the same weights
        ref = [p.detach().clone() for p in m.parameters()]
        f = FSDP(m, g, ShardingStrategy.FULL_SHARD)
        assert all(p.numel() == 0 for p in m.parameters())           # sharded: the full weights are gone
        h = f.prefetch_forward_params()
        x = torch.randn(4, 6, generator=torch.Generator().manual_seed(g.rank))
        y = f(x)                                                     # waits for the handle, gathers nothing itself
        assert h.is_done() and f._prefetch is None
        want = torch.nn.functional.linear(torch.tanh(torch.nn.functional.linear(x, ref[0], ref[1])), ref[2], ref[3])
        y.sum().backward()
        f.sync_gradients()
        return torch.allclose(y, want, atol=1e-6), all(s.grad is not None for s in f.shard_parameters())

    assert all(a and b for a, b in run_simulated(2, body))


@pytest.mark.parametrize("world,causal", [(2, True), (4, True), (4, False), (3, True)])
def test_ring_and_ulysses_attention_equal_full_attention(world, causal):
    from ferrotorch_b200.ops import reference as R
    from ferrotorch_b200.parallel import context_parallel as CP
    from ferrotorch_b200.parallel.backend import run_simulated

    torch.manual_seed(0)
    B, S_loc, Hq, Hkv, D = 2, 5, 12, 12 if world == 3 else 4, 8
    S = world * S_loc
    q, k, v = torch.randn(B, S, Hq, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    want, _ = R.attention(q, k, v, causal=causal)

    def body(g):
        sl = slice(g.rank * S_loc, (g.rank + 1) * S_loc)
        ring = CP.ring_attention(q[:, sl], k[:, sl], v[:, sl], g, causal)
        uly = CP.ulysses_attention(q[:, sl], k[:, sl], v[:, sl], g, causal) if Hkv % g.world_size == 0 else None
        return ring, uly

    for r, (ring, uly) in enumerate(run_simulated(world, body)):
        sl = slice(r * S_loc, (r + 1) * S_loc)
        assert torch.allclose(ring, want[:, sl], atol=1e-5), (r, (ring - want[:, sl]).abs().max())
        if uly is not None:
            assert torch.allclose(uly, want[:, sl], atol=1e-5), (r, (uly - want[:, sl]).abs().max())
    o1, l1 = R.attention(q, k[:, :7], v[:, :7], causal=False)
    o2, l2 = R.attention(q, k[:, 7:], v[:, 7:], causal=False)
    merged, _ = CP.merge_attention(o1, l1, o2, l2)
    assert torch.allclose(merged, R.attention(q, k, v, causal=False)[0], atol=1e-5)
    with pytest.raises(ValueError):
        run_simulated(2, lambda g: CP.ulysses_attention(q[:, :2, :3], k[:, :2, :1], v[:, :2, :1], g))


@pytest.mark.parametrize("world,causal", [(2, True), (4, True), (4, False), (3, True)])
def test_ring_and_ulysses_attention_gradients_equal_full_attention(world, causal):
    # backward of both schemes on simulated ranks against autograd through full attention:
    # dq of the local queries, dk / dv of the local keys (GQA: summed over the query group)
    from ferrotorch_b200.ops import reference as R
    from ferrotorch_b200.parallel import context_parallel as CP
    from ferrotorch_b200.parallel.backend import run_simulated

    torch.manual_seed(1)
    B, S_loc, Hq, Hkv, D = 2, 6, 12, 12 if world == 3 else 4, 8
    S = world * S_loc
    q, k, v = (torch.randn(B, S, h, D, requires_grad=True) for h in (Hq, Hkv, Hkv))
    go = torch.randn(B, S, Hq, D)
    R.attention(q, k, v, causal=causal)[0].backward(go)

    def body(g):
        sl = slice(g.rank * S_loc, (g.rank + 1) * S_loc)
        res = []
        for fn in (CP.ring_attention, CP.ulysses_attention):
            if fn is CP.ulysses_attention and Hkv % g.world_size:
                res.append(None)
                continue
            ql, kl, vl = (t[:, sl].detach().clone().requires_grad_() for t in (q, k, v))
            fn(ql, kl, vl, g, causal).backward(go[:, sl])
            res.append((ql.grad, kl.grad, vl.grad))
        return res

    for r, per_fn in enumerate(run_simulated(world, body)):
        sl = slice(r * S_loc, (r + 1) * S_loc)
        for name, grads in zip(("ring", "ulysses"), per_fn):
            if grads is None:
                continue
            for got, want, what in zip(grads, (q.grad, k.grad, v.grad), "qkv"):
                assert torch.allclose(got, want[:, sl], atol=2e-5), (name, r, what, (got - want[:, sl]).abs().max())


def test_attention_block_backward_pieces_add_up():
    # two key blocks with the statistics of the whole row: dq pieces add to the full dq, dk / dv are the blocks' own
    from ferrotorch_b200.ops import reference as R
    from ferrotorch_b200.ops.attention import attention_block_backward

    torch.manual_seed(2)
    q, k, v = (torch.randn(1, 7, h, 8, requires_grad=True) for h in (4, 2, 2))
    go = torch.randn(1, 7, 4, 8)
    out, lse = R.attention(q, k, v, causal=False)
    out.backward(go)
    dq1, dk1, dv1 = attention_block_backward(q.detach(), k.detach()[:, :3], v.detach()[:, :3], out.detach(), lse.detach(), go, False)
    dq2, dk2, dv2 = attention_block_backward(q.detach(), k.detach()[:, 3:], v.detach()[:, 3:], out.detach(), lse.detach(), go, False)
    assert torch.allclose(dq1 + dq2, q.grad, atol=1e-5)
    assert torch.allclose(torch.cat([dk1, dk2], 1), k.grad, atol=1e-5)
    assert torch.allclose(torch.cat([dv1, dv2], 1), v.grad, atol=1e-5)


def test_hybrid_group_routes_by_device_and_checks_ranks():
    from ferrotorch_b200.parallel import backend as B

    class Recorder(B.Group):
        def __init__(self, rank, world):
            self.rank, self.world_size, self.calls = rank, world, []

        def send(self, t, dst):
            self.calls.append(("send", dst))

        def recv(self, t, src, timeout=None):
            self.calls.append(("recv", src))

        def barrier(self):
            self.calls.append(("barrier",))

        def all_reduce(self, t, op="sum"):
            self.calls.append(("all_reduce", op))
            return t

    ctl, dat = Recorder(1, 4), Recorder(1, 4)
    h = B.HybridGroup(ctl, dat)
    assert (h.rank, h.world_size) == (1, 4) and h.tcp() is ctl and h.nccl() is dat
    x = torch.ones(3)
    h.send(x, 0), h.recv(x, 2), h.barrier(), h.all_reduce(x, "mean")
    assert ctl.calls == [("send", 0), ("recv", 2), ("barrier",), ("all_reduce", "mean")] and dat.calls == []

    class FakeCuda(torch.Tensor):
        is_cuda = True

    h.all_reduce(torch.ones(2).as_subclass(FakeCuda))
    assert dat.calls == [("all_reduce", "sum")]
    h.synchronize_data()
    with pytest.raises(B.InvalidRank):
        B.HybridGroup(Recorder(0, 2), Recorder(1, 2))
    with pytest.raises(B.BackendUnavailable):
        B.init_group("ucc")


def test_hybrid_group_over_simulated_transports():
    from ferrotorch_b200.parallel import backend as B

    ctl, dat = B.SimulatedGroup.create_group(3), B.SimulatedGroup.create_group(3)
    out = [None] * 3

    def work(r):
        h = B.HybridGroup(ctl[r], dat[r])
        t = torch.full((4,), float(r + 1))
        h.all_reduce(t, "sum")
        h.barrier()
        out[r] = t

    import threading
    ts = [threading.Thread(target=work, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    assert all(o is not None and torch.equal(o, torch.full((4,), 6.0)) for o in out)


def test_function_style_collectives_and_reference_names(tmp_path):
    import ferrotorch_b200.parallel as P

    def work(g):
        r, w = g.rank, g.world_size
        x = torch.full((4,), float(r + 1))
        s = P.allreduce(x, g, P.ReduceOp.Sum)
        m = P.allreduce_with_timeout(x, g, P.ReduceOp.Mean, timeout=20.0)
        assert torch.equal(x, torch.full((4,), float(r + 1)))            # input untouched
        gathered = P.all_gather_with_timeout(x[:1], g, timeout=20.0)
        rs = P.reduce_scatter(torch.arange(2.0 * w), g)
        b = P.broadcast(x, g, root=1)
        a2a = P.all_to_all(torch.arange(float(w)) + 10 * r, g)
        send = [1] * w
        un = P.all_to_all_single_uneven(torch.arange(float(w)) + 10 * r, send, send, g)
        P.barrier(g)
        assert g.timeout == 30.0                                          # restored after the bounded calls
        with pytest.raises(P.SizeMismatch):
            P.reduce_scatter(torch.ones(w + 1), g)
        return s, m, gathered, rs, b, a2a, un

    outs = P.run_simulated(3, work)
    for r, (s, m, gathered, rs, b, a2a, un) in enumerate(outs):
        assert torch.equal(s, torch.full((4,), 6.0)) and torch.equal(m, torch.full((4,), 2.0))
        assert torch.equal(gathered, torch.tensor([1.0, 2.0, 3.0])) and torch.equal(rs, torch.tensor([3.0 * 2 * r, 3.0 * (2 * r + 1)]))
        assert torch.equal(b, torch.full((4,), 2.0)) and torch.equal(a2a, torch.tensor([r, 10.0 + r, 20.0 + r])) and torch.equal(un, a2a)
    assert P.Backend is P.Group and P.TcpBackend is P.TcpGroup and P.HybridBackend is P.HybridGroup and P.DEFAULT_COLLECTIVE_TIMEOUT == 60.0
    for ctor in (P.MpiBackend, P.UccBackend, P.NcclBackend, P.GlooBackend):
        with pytest.raises(P.BackendUnavailable):
            ctor()
    with pytest.raises(P.UnsupportedOp):
        P.nccl_allreduce(torch.ones(2), None)
    # checkpoint types: flat shards written by 2 ranks, read back by 1 and by 3
    full = {"w": torch.arange(12.0)}
    meta = P.flat_shard_metadata({"w": full["w"][:6]}, 2)
    assert meta.tensor_specs["w"].full_shape == [12] and meta.to_json()["num_ranks"] == 2
    from ferrotorch_b200.parallel.dist_checkpoint import save_reference_distributed
    for r in range(2):
        save_reference_distributed(str(tmp_path), {"w": full["w"][6 * r:6 * r + 6]}, {"w": 0}, {"w": [6, 6]}, r, 2)
    ck = P.DistributedCheckpoint.open(str(tmp_path))
    assert ck.shard_metadata.num_ranks == 2 and torch.equal(ck.load(0, 1)["w"], full["w"])
    parts = [P.reshard(str(tmp_path), 2, 3, r)["w"] for r in range(3)]
    assert torch.equal(torch.cat(parts), full["w"]) and [p.numel() for p in parts] == [4, 4, 4]
    with pytest.raises(P.DistCheckpointError):
        P.DistributedCheckpoint.open(str(tmp_path / "nope"))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_vocabulary_parallel_sampling_equals_single_device_sampling(world):
    # temperature / top-k / top-p on logits sharded over the vocabulary pick exactly the tokens the
    # single-device procedure picks from the full logits with the same uniform numbers; the last shard
    # is padded; a nucleus wider than the first candidate list makes the call widen it
    from ferrotorch_b200.parallel import vocab_sampling as VS
    from ferrotorch_b200.parallel.backend import run_simulated

    torch.manual_seed(0)
    B, V = 64, 1000
    Vl = (V + world - 1) // world
    logits = torch.randn(B, V) * 3.0
    logits[:8] *= 0.05                      # nearly flat rows: very wide nuclei
    logits[8:16, :300] += 6.0               # rows whose probable tokens all sit in the first shard
    padded = torch.cat([logits, torch.zeros(B, Vl * world - V)], 1)
    cases = [(1.0, 0, 1.0), (0.7, 50, 1.0), (1.3, 0, 0.9), (1.0, 40, 0.8), (0.0, 0, 1.0), (1.0, 0, 0.999), (2.0, 5, 0.5)]

    def body(g):
        out = []
        for step, (temp, k, p) in enumerate(cases):
            u = VS.shared_uniform(B, 7, step)
            lo = g.rank * Vl
            out.append(VS.sample_vocab_parallel(padded[:, lo:lo + Vl], g, lo, u, temp, k, p, candidates=16, valid=max(0, min(Vl, V - lo))))
        return out

    res = run_simulated(world, body)
    for step, (temp, k, p) in enumerate(cases):
        u = VS.shared_uniform(B, 7, step)
        want = logits.argmax(-1) if temp == 0.0 else VS.sample_reference(logits, u, temp, k, p)
        for r in range(world):
            assert torch.equal(res[r][step], want), (world, step, (res[r][step] != want).sum())
        assert int(want.max()) < V
    # the draws follow the distribution: frequencies of a small vocabulary against its softmax
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).expand(4000, 4).contiguous()
    g1 = run_simulated(2, lambda g: VS.sample_vocab_parallel(small[:, g.rank * 2:(g.rank + 1) * 2], g, g.rank * 2,
                                                             VS.shared_uniform(4000, 3, 0)))[0]
    freq = torch.bincount(g1, minlength=4).float() / 4000
    assert torch.allclose(freq, small[0].softmax(-1), atol=0.03)


# --------------------------------------------------------------------------- FSDP with one flat buffer per unit
@pytest.mark.parametrize("prefetch,overlap,intra", [(True, True, None), (False, False, None), (True, True, 2)],
                         ids=["overlapped", "inline", "hybrid-2x2"])
def test_flat_fsdp_units_train_like_one_process_and_release_their_buffers(prefetch, overlap, intra):
    import threading

    from torch import nn

    from ferrotorch_b200.parallel.backend import SimulatedGroup
    from ferrotorch_b200.parallel.fsdp_flat import FsdpUnit, auto_wrap

    class Block(nn.Module):
        def __init__(self, d):
            super().__init__()
            self.a, self.b = nn.Linear(d, 2 * d), nn.Linear(2 * d, d)

        def forward(self, x):
            return x + self.b(torch.tanh(self.a(x)))

    def make():
        torch.manual_seed(0)
        return nn.Sequential(nn.Linear(6, 8), Block(8), Block(8), Block(8), nn.Linear(8, 3))

    W, steps = 4, 4
    torch.manual_seed(1)
    X, Y = torch.randn(16, 6), torch.randn(16, 3)
    ref = make()
    opt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    ref_losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = nn.functional.mse_loss(ref(X), Y)
        loss.backward()
        opt.step()
        ref_losses.append(float(loss.detach()))
    groups = SimulatedGroup.create_group(W)
    out = {}
    protos = [make() for _ in range(W)]           # built here: the global generator is not thread-safe

    def rank(r):
        model = auto_wrap(protos[r], groups[r], (Block,), reshard_after_forward=True, prefetch=prefetch, overlap_grad_sync=overlap,
                          intra_node_size=intra)
        ps = model.sharded_parameters()
        o = torch.optim.SGD(ps, lr=0.1, momentum=0.9)
        xs, ys = X.chunk(W)[r], Y.chunk(W)[r]
        losses, freed = [], None
        for _ in range(steps):
            o.zero_grad()
            loss = nn.functional.mse_loss(model(xs), ys)
            freed = [u.full.untyped_storage().size() for u in model.units]        # between forward and backward
            loss.backward()
            model.sync_gradients()
            o.step()
            losses.append(float(loss.detach()))
        stats = [dict(u.stats) for u in model.units]
        out[r] = (losses, model.full_state_dict(), freed, stats, sum(p.numel() for p in ps))

    ts = [threading.Thread(target=rank, args=(r,)) for r in range(W)]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    assert len(out) == W
    sd_ref = ref.state_dict()
    for r in range(W):
        losses, sd, freed, stats, held = out[r]
        assert set(sd) == set(sd_ref)
        for k in sd_ref:
            torch.testing.assert_close(sd[k], sd_ref[k], rtol=1e-5, atol=1e-6)
        assert freed == [0, 0, 0]                                               # every unit gave its full buffer back
        # per step and unit: one all-gather before forward, one before backward, one reduce-scatter
        assert all(s == {"all_gathers": 2 * steps, "reduce_scatters": steps} for s in stats)
        shard_ways = intra or W
        assert held <= (sum(p.numel() for p in ref.parameters()) + 3 * W * 5) // shard_ways + 1      # about 1 / ways of the model
    mean_losses = [sum(out[r][0][i] for r in range(W)) / W for i in range(steps)]
    torch.testing.assert_close(torch.tensor(mean_losses), torch.tensor(ref_losses), rtol=1e-5, atol=1e-6)
    one = SimulatedGroup.create_group(1)[0]
    with pytest.raises(ValueError):
        FsdpUnit(nn.ReLU(), one)
    net = nn.Linear(3, 3)
    u = FsdpUnit(net, one, reshard_after_forward=False)
    with torch.no_grad():
        assert u(torch.ones(1, 3)).shape == (1, 3) and u.full.untyped_storage().size() > 0     # kept when asked to


# --------------------------------------------------------------------------- rank-addressed RPC over a group
def test_group_rpc_agent_buffers_out_of_order_responses_and_serves_while_waiting():
    import threading
    import time

    from ferrotorch_b200.parallel.backend import InvalidRank, SimulatedGroup
    from ferrotorch_b200.parallel.dist_checkpoint import GroupRpcAgent

    w = SimulatedGroup.create_group(2)
    res, errs = {}, []

    def r0():
        try:
            a = GroupRpcAgent(w[0])
            a.register("who", lambda: "rank0")
            slow = a.rpc_async(1, "work", 0.3, "slow")
            time.sleep(0.05)
            fast = a.rpc_async(1, "work", 0.0, "fast")
            res["fast"], res["t_fast"] = fast.wait(10), time.time()
            res["slow"], res["t_slow"] = slow.wait(10), time.time()
            res["tensor"] = a.rpc_sync(1, "double", torch.arange(3.0), scale=3)
            try:
                a.rpc_sync(1, "boom")
            except RuntimeError as e:
                res["err"] = str(e)
            res["mutual0"] = a.rpc_sync(1, "who")                 # rank 1 calls "who" here at the same time
            with pytest.raises(InvalidRank):
                a.rpc_sync(0, "who")
            assert (a.rank(), a.world_size()) == (0, 2)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)

    def r1():
        try:
            a = GroupRpcAgent(w[1])

            def work(delay, tag):
                time.sleep(delay)
                return tag

            a.register("work", work)
            a.register("double", lambda t, scale=2: t * scale)
            a.register("boom", lambda: 1 / 0)
            a.register("who", lambda: "rank1")
            a.serve(0, 2, concurrent=True)                         # the two overlapping calls
            a.serve(0, 2)                                          # double, boom
            res["mutual1"] = a.rpc_sync(0, "who")                  # serves rank 0's request while waiting for its own answer
        except BaseException as e:  # noqa: BLE001
            errs.append(e)

    ts = [threading.Thread(target=f) for f in (r0, r1)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert not errs, errs
    assert res["fast"] == "fast" and res["slow"] == "slow" and res["t_fast"] < res["t_slow"]       # answered out of order
    assert res["tensor"].tolist() == [0.0, 3.0, 6.0] and "ZeroDivisionError" in res["err"]
    assert res["mutual0"] == "rank1" and res["mutual1"] == "rank0"
