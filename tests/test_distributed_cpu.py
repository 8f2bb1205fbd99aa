"""Host-side communication: simulated in-process ranks, loopback TCP between processes,
timeouts / size mismatches / a rank that leaves, and the CPU plumbing config (tiny Llama,
DDP world 2, bitwise-equal losses and reduced gradients).  No GPU involved."""
import multiprocessing as mp
import socket

import pytest
import torch

from ferrotorch_b200.parallel import backend as B
from ferrotorch_b200.parallel.host_ddp import DDP, compute_buckets

import dist_workers as W


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _spawn(fn, world, *extra, timeout=180):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port, q) + extra) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(world):
        r, v = q.get(timeout=timeout)
        out[r] = v
    for p in procs:
        p.join(30)
    for v in out.values():
        assert not (isinstance(v, str) and v.startswith("ERR")), v
    return out


# ----------------------------------------------------------------------------- simulated group
def test_simulated_collectives_four_ranks():
    def body(g):
        r, w = g.rank, g.world_size
        s = g.all_reduce(torch.full((3,), float(r + 1)), "sum")
        m = g.all_reduce(torch.full((3,), float(r + 1)), "mean")
        b = g.broadcast(torch.full((2,), float(r)), 2)
        ag = g.all_gather(torch.tensor([float(r)]))
        rs = g.reduce_scatter(torch.arange(w, dtype=torch.float32))
        a2a = g.all_to_all(torch.arange(w, dtype=torch.float32) + 10 * r)
        un = g.all_to_all(torch.arange(sum(range(1, w + 1)), dtype=torch.float32) + 100 * r,
                          send_counts=[p + 1 for p in range(w)], recv_counts=[r + 1] * w)
        g.barrier()
        return s, m, b, ag, rs, a2a, un

    res = B.run_simulated(4, body)
    for r, (s, m, b, ag, rs, a2a, un) in enumerate(res):
        assert s.tolist() == [10.0] * 3 and m.tolist() == [2.5] * 3
        assert b.tolist() == [2.0, 2.0]
        assert ag.tolist() == [0.0, 1.0, 2.0, 3.0]
        assert rs.tolist() == [4.0 * r]
        assert a2a.tolist() == [r + 10.0 * p for p in range(4)]
        assert un.numel() == 4 * (r + 1)


def test_simulated_errors():
    gs = B.SimulatedGroup.create_group(2, timeout=0.2)
    with pytest.raises(B.SelfSend):
        gs[0].send(torch.zeros(1), 0)
    with pytest.raises(B.InvalidRank):
        gs[0].send(torch.zeros(1), 5)
    with pytest.raises(B.Timeout):
        gs[0].recv(torch.zeros(1), 1)
    gs[1].send(torch.zeros(8), 0)
    with pytest.raises(B.SizeMismatch):
        gs[0].recv(torch.zeros(4), 1)
    with pytest.raises(B.InvalidWorldSize):
        B.SimulatedGroup.create_group(0)
    with pytest.raises(B.SizeMismatch):
        B.run_simulated(2, lambda g: g.reduce_scatter(torch.zeros(3)))
    with pytest.raises(B.BackendUnavailable):
        B.init_group("mpi")


def test_subgroup_maps_ranks():
    def body(g):
        if g.rank in (1, 3):
            sg = B.SubGroup(g, [3, 1, 3])
            v = sg.all_reduce(torch.tensor([float(g.rank)]), "sum")
            return sg.rank, sg.world_size, sg.global_rank(1), v.item()
        return None

    res = B.run_simulated(4, body)
    assert res[1] == (0, 2, 3, 4.0) and res[3] == (1, 2, 3, 4.0)
    gs = B.SimulatedGroup.create_group(2)
    with pytest.raises(B.InvalidRank):
        B.SubGroup(gs[0], [1])


def test_ddp_buckets_and_sync_simulated():
    p = [torch.nn.Parameter(torch.zeros(n)) for n in (10, 20, 30, 40)]
    assert compute_buckets(p, 50 * 4) == [[3], [2, 1], [0]]  # reverse order, <= 200 bytes each

    def body(g):
        torch.manual_seed(g.rank)
        m = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.ReLU(), torch.nn.Linear(8, 2))
        d = DDP(m, g, bucket_size_bytes=64)
        d.broadcast_parameters(0)
        x = torch.full((3, 4), float(g.rank + 1))
        d(x).sum().backward()
        local = [q.grad.clone() for q in m.parameters()]
        d.sync_gradients()
        return [q.detach().clone() for q in m.parameters()], local, [q.grad.clone() for q in m.parameters()]

    res = B.run_simulated(3, body)
    for k in range(4):
        want = (res[0][1][k] + res[1][1][k] + res[2][1][k]) / 3
        for r in range(3):
            assert torch.equal(res[r][0][k], res[0][0][k])          # broadcast parameters
            assert torch.equal(res[r][2][k], res[0][2][k])          # bitwise-equal reduced grads
            assert torch.allclose(res[r][2][k], want, atol=1e-6)


def test_ddp_overlapped_buckets_equal_the_sequential_form():
    # buckets reduced on a worker thread while backward still runs: same result bit for bit, also with
    # a parameter that gets no gradient, over several steps, and with accumulation under no_sync()
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b, self.c = torch.nn.Linear(6, 16), torch.nn.Linear(16, 16), torch.nn.Linear(16, 3)
            self.unused = torch.nn.Linear(4, 4)

        def forward(self, x):
            return self.c(torch.tanh(self.b(torch.tanh(self.a(x)))))

    import copy

    torch.manual_seed(7)
    proto = Net()                                             # ranks are threads: one initialisation, copied

    def body(g, overlap):
        m = copy.deepcopy(proto)
        d = DDP(m, g, bucket_size_bytes=300, overlap=overlap)
        assert len(d.buckets) > 3
        out = []
        gen = torch.Generator().manual_seed(100 + g.rank)
        for step in range(3):
            m.zero_grad(set_to_none=True)
            with d.no_sync():
                d(torch.randn(5, 6, generator=gen)).square().sum().backward()      # accumulated, not exchanged
            d(torch.randn(5, 6, generator=gen)).square().sum().backward()
            d.sync_gradients()
            out.append([None if q.grad is None else q.grad.clone() for q in m.parameters()])
            with torch.no_grad():
                for q in m.parameters():
                    if q.grad is not None:
                        q -= 0.1 * q.grad
        return out

    seq = B.run_simulated(3, body, False)
    ovl = B.run_simulated(3, body, True)
    for r in range(3):
        for s_step, o_step in zip(seq[r], ovl[r]):
            for a, b in zip(s_step, o_step):
                assert (a is None and b is None) or torch.equal(a, b)
    for step in range(3):                                   # and every rank holds the same reduced gradients
        for a, b in zip(ovl[0][step], ovl[2][step]):
            assert torch.equal(a, b)


# ----------------------------------------------------------------------------- loopback TCP
@pytest.mark.parametrize("world", [2, 3, 5])
def test_tcp_collectives(world):
    out = _spawn(W.collectives, world)
    tot = float(sum(range(1, world + 1)))
    for r in range(world):
        o = out[r]
        assert o["sum"] == [tot] * 5
        assert o["mean"] == [i * tot / world for i in range(4)]
        assert o["bcast"] == [1.0] * 3
        assert o["gather"] == [[float(k), 1.0] for k in range(world)]
        assert o["rs"] == [world * (2.0 * r), world * (2.0 * r + 1)]
        assert o["a2a"] == [r + 10.0 * p for p in range(world)]
        assert o["ring"] == [tot, 999 * tot]
        assert o["f64"] == [0.5 * tot] * 3
        for root in range(world):                      # binary-tree broadcast from every root
            assert o["tree%d" % root] == [float(root * 10 + root)] * 7
        assert o["bad_root"] == "InvalidRank"
    assert out[world - 1]["p2p"] == 42.0


def test_tcp_recv_timeout_is_an_error_not_a_hang():
    out = _spawn(W.timeout_case, 2)
    assert out[0].startswith("timeout") and float(out[0].split()[1]) < 2.0


def test_tcp_size_mismatch():
    out = _spawn(W.size_mismatch_case, 2)
    assert out[0] == "size mismatch"


def test_tcp_rank_that_leaves_is_detected():
    out = _spawn(W.dead_peer_case, 2)
    assert out[1] == "left" and out[0].startswith("error")


def _hostile_peer(port, announce, frames, close_after=None):
    """A raw socket that plays rank 1 badly: sends ``announce`` as its rank, then ``frames``."""
    import struct
    import threading
    import time

    def run():
        deadline = time.time() + 20
        while True:
            try:
                s = socket.create_connection(("127.0.0.1", port), timeout=1)
                break
            except OSError:
                if time.time() > deadline:
                    return
                time.sleep(0.05)
        s.sendall(struct.pack("<Q", announce))
        for f in frames:
            s.sendall(f)
        time.sleep(close_after if close_after is not None else 3.0)
        s.close()

    t = threading.Thread(target=run, daemon=True)
    t.start()
    return t


def test_tcp_hostile_peer_is_rejected_with_typed_errors():
    import struct
    import time

    # a peer that announces a rank outside the world never gets into the group
    port = _free_port()
    _hostile_peer(port, 99, [])
    with pytest.raises(B.InvalidRank):
        B.TcpGroup(0, 2, "127.0.0.1", port, timeout=10)
    # a length prefix that disagrees with what the receiver expects (here: 2^60 bytes) is an
    # error at once, not an allocation or a long read
    port = _free_port()
    _hostile_peer(port, 1, [struct.pack("<Q", 1 << 60) + b"junk"])
    g = B.TcpGroup(0, 2, "127.0.0.1", port, timeout=10)
    t0 = time.perf_counter()
    with pytest.raises(B.SizeMismatch):
        g.recv(torch.zeros(4), 1, timeout=5.0)
    assert time.perf_counter() - t0 < 2.0
    g.close()
    # a peer that hangs up in the middle of a payload: an error, not a hang
    port = _free_port()
    _hostile_peer(port, 1, [struct.pack("<Q", 16) + b"only8byt"], close_after=0.2)
    g = B.TcpGroup(0, 2, "127.0.0.1", port, timeout=10)
    t0 = time.perf_counter()
    with pytest.raises(B.DistributedError):
        g.recv(torch.zeros(4), 1, timeout=5.0)
    assert time.perf_counter() - t0 < 4.0
    g.close()


# ----------------------------------------------------------------------------- config 0
@pytest.mark.parametrize("backend", ["tcp", "gloo"])
def test_config0_tiny_llama_ddp_bitwise(backend):
    steps = 20 if backend == "tcp" else 4
    out = _spawn(W.config0, 2, steps, backend, timeout=600)
    a, b = out[0], out[1]
    assert a["losses"] == b["losses"], "rank losses differ bitwise"
    assert a["grads"] == b["grads"], "post-all-reduce gradients differ bitwise"
    assert a["last"] < a["first"]


@pytest.mark.parametrize("backend,schedule", [("tcp", "1f1b"), ("gloo", "1f1b"), ("gloo", "gpipe")])
def test_pipeline_stages_as_processes_with_posted_transfers(backend, schedule):
    out = _spawn(W.pipeline_case, 3, backend, schedule)
    assert all(v == "ok" for v in out.values()), out


def test_plain_torch_tensor_parallel_baseline_is_a_correct_model():
    # the baseline that the tensor-parallel benchmarks are compared with must itself compute the right thing
    out = _spawn(W.torch_tp_baseline_case, 2)
    assert all(v == "ok" for v in out.values()), out


def test_vocab_parallel_embedding_and_cross_entropy_gloo():
    out = _spawn(W.vocab_parallel_case, 2)
    assert all(v == "ok" for v in out.values()), out


def test_heartbeat_detects_a_dead_rank_and_survivors_reshard(tmp_path):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=W.elastic_case, args=(r, 3, 0, q, str(tmp_path))) for r in range(3)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in range(2))           # rank 2 never reports
    for p in procs:
        p.join(30)
    assert set(out) == {0, 1}, out
    for r, v in out.items():
        assert not isinstance(v, str), v
        detected, new_rank, new_world, rows = v
        assert detected == [2] and new_world == 2 and new_rank == r
    # global vector after 3 steps at world 3 (rows of rank k start at 100 k) and 3 more at world 2
    full = out[0][3] + out[1][3]
    assert full == [6.0] * 4 + [106.0] * 4 + [206.0] * 4


def test_heartbeat_clean_leave_and_store_barrier(tmp_path):
    from ferrotorch_b200.parallel.elastic import FileStore, Heartbeat, RankFailure, barrier, survivors

    store = FileStore(str(tmp_path))
    a, b = Heartbeat(store, 0, 2, interval=0.02, timeout=0.3), Heartbeat(store, 1, 2, interval=0.02, timeout=0.3)
    a.wait_for_all(5.0)
    a.check()
    b.check()
    b.leave()
    with pytest.raises(RankFailure) as e:
        a.check()
    assert e.value.left == [1] and e.value.ranks == [] and survivors(2, e.value) == [0]
    a.stop()
    barrier(store, "solo", 0, [0], limit=1.0)
    with pytest.raises(RankFailure):
        barrier(store, "pair", 0, [0, 1], limit=0.2)


def test_hybrid_mesh_groups_and_data_parallel_trainer_gloo():
    out = _spawn(W.hybrid_case, 4)
    want = {0: (1.0, 2.0), 1: (1.0, 4.0), 2: (5.0, 2.0), 3: (5.0, 4.0)}
    for r in range(4):
        (tp_sum, dp_sum, tp_n, dp_n), diff, losses = out[r]
        assert (tp_sum, dp_sum) == want[r] and (tp_n, dp_n) == (2, 2)
        assert diff < 2e-5, diff                       # two half-batch replicas == one full-batch process
        assert losses[-1] < losses[0]


def test_rendezvous_config_from_launcher_environments():
    R = B.RendezvousConfig
    c = R.from_env({"RANK": "1", "WORLD_SIZE": "4", "MASTER_ADDR": "10.0.0.1", "MASTER_PORT": "1234"})
    assert (c.master_addr, c.master_port, c.rank, c.world_size) == ("10.0.0.1", 1234, 1, 4)
    c = R.from_env({"OMPI_COMM_WORLD_RANK": "2", "OMPI_COMM_WORLD_SIZE": "3"})          # started by mpirun
    assert (c.rank, c.world_size, c.master_addr, c.master_port) == (2, 3, "127.0.0.1", 29500)
    assert R.from_env({"PMI_RANK": "0", "PMI_SIZE": "1"}).world_size == 1
    assert R.from_env({"RANK": "0", "OMPI_COMM_WORLD_RANK": "5", "WORLD_SIZE": "2"}).rank == 0   # torchrun's names win
    for env, err in (({}, B.NoConnection), ({"RANK": "0"}, B.NoConnection), ({"RANK": "x", "WORLD_SIZE": "2"}, B.InvalidRank),
                     ({"RANK": "2", "WORLD_SIZE": "2"}, B.InvalidRank), ({"RANK": "0", "WORLD_SIZE": "0"}, B.InvalidWorldSize),
                     ({"RANK": "0", "WORLD_SIZE": "1", "MASTER_PORT": "http"}, B.NoConnection)):
        with pytest.raises(err):
            R.from_env(env)
