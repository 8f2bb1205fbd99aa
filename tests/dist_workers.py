"""Process entry points for the loopback-TCP tests (spawned with multiprocessing)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _group(rank, world, port, timeout=20.0):
    from ferrotorch_b200.parallel.backend import TcpGroup

    return TcpGroup(rank, world, "127.0.0.1", port, timeout=timeout)


def collectives(rank, world, port, q):
    import torch

    try:
        g = _group(rank, world, port)
        out = {}
        t = torch.full((5,), float(rank + 1))
        g.all_reduce(t, "sum")
        out["sum"] = t.tolist()
        t = torch.arange(4, dtype=torch.float32) * (rank + 1)
        g.all_reduce(t, "mean")
        out["mean"] = t.tolist()
        b = torch.full((3,), float(rank))
        g.broadcast(b, 1)
        out["bcast"] = b.tolist()
        out["gather"] = g.all_gather(torch.tensor([[float(rank), 1.0]])).tolist()
        out["rs"] = g.reduce_scatter(torch.arange(world * 2, dtype=torch.float32)).tolist()
        out["a2a"] = g.all_to_all(torch.arange(world, dtype=torch.float32) + 10 * rank).tolist()
        r = torch.arange(1000, dtype=torch.float32) * (rank + 1)
        g.all_reduce(r, "sum", algorithm="ring")
        out["ring"] = [float(r[1]), float(r[999])]
        d = torch.full((3,), 0.5 * (rank + 1), dtype=torch.float64)
        g.all_reduce(d, "sum")
        out["f64"] = d.tolist()
        if rank == 0:
            g.send(torch.tensor([42.0]), world - 1)
        if rank == world - 1:
            x = torch.zeros(1)
            g.recv(x, 0)
            out["p2p"] = x.item()
        for root in range(world):
            tb = torch.full((7,), float(rank * 10 + root))
            g.broadcast(tb, root, algorithm="tree")
            out["tree%d" % root] = tb.tolist()
        g.barrier(algorithm="ring")
        try:
            g.broadcast(torch.zeros(1), world, algorithm="tree")
            out["bad_root"] = "accepted"
        except Exception as e:  # noqa: BLE001
            out["bad_root"] = type(e).__name__
        g.barrier()
        g.close()
        q.put((rank, out))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "ERR %r" % (e,)))


def timeout_case(rank, world, port, q):
    """Rank 1 never sends: rank 0's receive must raise Timeout, not hang."""
    import torch

    from ferrotorch_b200.parallel.backend import Timeout

    try:
        g = _group(rank, world, port, timeout=30.0)      # generous rendezvous: a cold process start is slow
        if rank == 0:
            t0 = time.time()
            try:
                g.recv(torch.zeros(4), 1, timeout=0.5)
                q.put((rank, "no error"))
            except Timeout:
                q.put((rank, "timeout %.2f" % (time.time() - t0)))
        else:
            time.sleep(1.5)
            q.put((rank, "idle"))
        g.close()
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "ERR %r" % (e,)))


def size_mismatch_case(rank, world, port, q):
    import torch

    from ferrotorch_b200.parallel.backend import SizeMismatch

    try:
        g = _group(rank, world, port, timeout=5.0)
        if rank == 1:
            g.send(torch.zeros(8), 0)
            q.put((rank, "sent"))
        else:
            try:
                g.recv(torch.zeros(4), 1)
                q.put((rank, "no error"))
            except SizeMismatch:
                q.put((rank, "size mismatch"))
        g.close()
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "ERR %r" % (e,)))


def dead_peer_case(rank, world, port, q):
    """Rank 1 exits between steps; rank 0's next collective fails with an error, it does not hang."""
    import torch

    from ferrotorch_b200.parallel.backend import DistributedError

    try:
        g = _group(rank, world, port, timeout=3.0)
        t = torch.ones(4)
        g.all_reduce(t)
        if rank == 1:
            g.close()
            q.put((rank, "left"))
            return
        time.sleep(0.3)
        try:
            g.all_reduce(t)
            q.put((rank, "no error"))
        except DistributedError as e:
            q.put((rank, "error %s" % type(e).__name__))
        g.close()
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "ERR %r" % (e,)))


def config0(rank, world, port, q, steps=20, backend="tcp"):
    """BASELINE config 0: tiny Llama, fp32 CPU, AdamW, clip 1.0, DDP world 2 over loopback TCP."""
    import torch

    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.parallel.host_ddp import DDP

    try:
        torch.set_num_threads(2)
        if backend == "tcp":
            g = _group(rank, world, port, timeout=60.0)
        else:
            import torch.distributed as dist

            from ferrotorch_b200.parallel.backend import TorchGroup

            dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
            g = TorchGroup()
        torch.manual_seed(1000 + rank)  # different init per rank: broadcast must fix it
        model = LlamaForCausalLM(LlamaConfig.tiny())
        ddp = DDP(model, g)
        ddp.broadcast_parameters(0)
        opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
        gen = torch.Generator().manual_seed(0)  # seed 0 on every rank (config 0)
        losses, grad_sums = [], []
        t0 = time.time()
        for _ in range(steps):
            ids = torch.randint(0, 4096, (8, 129), generator=gen)
            loss = model(ids[:, :-1], labels=ids[:, 1:])
            opt.zero_grad(set_to_none=True)
            loss.backward()
            ddp.sync_gradients()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            grad_sums.append(torch.cat([p.grad.reshape(-1) for p in model.parameters()]).double().sum().item().hex())
            opt.step()
            losses.append(loss.item().hex())
        q.put((rank, {"losses": losses, "grads": grad_sums, "first": float.fromhex(losses[0]),
                      "last": float.fromhex(losses[-1]), "s_per_step": (time.time() - t0) / steps}))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR %r %s" % (e, traceback.format_exc())))


def vocab_parallel_case(rank, world, port, q):
    """Vocabulary-parallel embedding + cross-entropy over gloo against the unsharded math."""
    try:
        import os

        import torch
        import torch.distributed as dist

        from ferrotorch_b200.parallel.tp_layers import (VocabParallelEmbedding, all_reduce_replicated_grads,
                                                        vocab_parallel_cross_entropy)

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        g = torch.Generator().manual_seed(4)
        V, H, M = 32, 8, 12
        table = torch.randn(V, H, generator=g)
        ids = torch.randint(0, V, (M,), generator=g)
        upstream = torch.randn(M, H, generator=g)
        logits = torch.randn(M, V, generator=g) * 3
        tgt = torch.randint(0, V, (M,), generator=g)
        tgt[3] = -100
        vl, ms = V // world, M // world
        errs = []

        # ---- embedding: rows of the unsharded lookup, and the table gradient of this shard
        t_ref = table.clone().requires_grad_()
        (torch.nn.functional.embedding(ids, t_ref) * upstream).sum().backward()
        emb = VocabParallelEmbedding(vl, H, dist.group.WORLD, rank, world, dtype=torch.float32)
        with torch.no_grad():
            emb.weight.copy_(table[rank * vl:(rank + 1) * vl])
        rows = emb(ids)
        if not torch.allclose(rows, table[ids][rank * ms:(rank + 1) * ms], atol=1e-6):
            errs.append("embedding rows")
        (rows * upstream[rank * ms:(rank + 1) * ms]).sum().backward()
        if not torch.allclose(emb.weight.grad, t_ref.grad[rank * vl:(rank + 1) * vl], atol=1e-5):
            errs.append("embedding grad")

        # ---- cross-entropy over vocabulary shards
        l_ref = logits.clone().requires_grad_()
        loss_ref = torch.nn.functional.cross_entropy(l_ref, tgt, ignore_index=-100)
        loss_ref.backward()
        l_loc = logits[:, rank * vl:(rank + 1) * vl].clone().requires_grad_()
        loss = vocab_parallel_cross_entropy(l_loc, tgt, dist.group.WORLD, rank, world)
        (loss * 2.0).backward()
        if abs(float(loss) - float(loss_ref)) > 1e-5:
            errs.append("loss %g vs %g" % (float(loss), float(loss_ref)))
        if not torch.allclose(l_loc.grad, 2.0 * l_ref.grad[:, rank * vl:(rank + 1) * vl], atol=1e-6):
            errs.append("logit grad")

        # ---- replicated-parameter reduction
        p = torch.nn.Parameter(torch.zeros(4))
        p.main_grad = torch.full((4,), float(rank + 1))
        all_reduce_replicated_grads([p], dist.group.WORLD)
        if p.main_grad.tolist() != [float(sum(range(1, world + 1)))] * 4:
            errs.append("replicated grads")
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok" if not errs else "ERR " + ", ".join(errs)))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR " + traceback.format_exc()[-1500:]))


def elastic_case(rank, world, port, q, root):
    """Three ranks train a row-sharded vector and checkpoint every step; rank 2 dies without a
    word after step 3.  The others notice through the heartbeat before their next step, regroup
    as a world of two, reload the last complete checkpoint resharded 3 -> 2 and finish."""
    try:
        import os

        import torch

        from ferrotorch_b200.parallel import dist_checkpoint as dc
        from ferrotorch_b200.parallel.elastic import FileStore, Heartbeat, RankFailure, barrier, survivors

        store = FileStore(os.path.join(root, "store"))
        hb = Heartbeat(store, rank, world, interval=0.05, timeout=0.5)
        hb.wait_for_all(30.0)
        w = torch.zeros(12 // world) + 100.0 * rank            # this rank's rows
        step, detected, my_rank, my_world = 0, None, rank, world
        total_steps = 6
        while step < total_steps:
            try:
                if my_world == world:
                    hb.check()
            except RankFailure as f:
                detected = f.ranks
                alive = survivors(world, f)
                barrier(store, "regroup", rank, alive, limit=20.0)
                my_rank, my_world = alive.index(rank), len(alive)
                last = max(s for s in range(step + 1) if all(
                    os.path.exists(os.path.join(root, "ckpt_%d" % s, "shard_%d.safetensors" % r)) for r in range(world)))
                state, extra = dc.load_distributed(os.path.join(root, "ckpt_%d" % last), my_rank, my_world)
                w, step = state["w"], extra["step"]
                continue
            w = w + 1.0
            step += 1
            if my_world == world:
                dc.save_distributed(os.path.join(root, "ckpt_%d" % step), {"w": w}, {"w": 0}, rank=rank,
                                    world_size=world, extra={"step": step})
                if rank == 2 and step == 3:
                    os._exit(0)                                 # no leave(), no clean-up
                time.sleep(0.4)                                 # a step takes a while
        hb.stop()
        q.put((rank, (detected, my_rank, my_world, w.tolist())))
    except BaseException:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR " + traceback.format_exc()[-1500:]))


def hybrid_case(rank, world, port, q):
    """dp x tp process groups over gloo, and data parallelism added to a flat trainer: two replicas
    with half the batch each follow the same trajectory as one process with the whole batch."""
    try:
        import os

        import torch
        import torch.distributed as dist

        from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
        from ferrotorch_b200.models.llama_tp import add_data_parallel, hybrid_groups
        from ferrotorch_b200.train.engine import FlatTrainer

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        tp, dp = hybrid_groups(2)
        a = torch.tensor([float(rank)])
        b = a.clone()
        dist.all_reduce(a, group=tp)                  # world 4, tp 2: tp groups {0,1} {2,3}, dp groups {0,2} {1,3}
        dist.all_reduce(b, group=dp)
        sums = (a.item(), b.item(), dist.get_world_size(tp), dist.get_world_size(dp))
        cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                          num_attention_heads=2, num_key_value_heads=1)
        torch.manual_seed(0)
        model = LlamaForCausalLM(cfg)
        tr = add_data_parallel(FlatTrainer(model, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0), dp)
        g = torch.Generator().manual_seed(5)
        tokens = torch.randint(0, 64, (4, 9), generator=g)            # the global batch of the dp group
        k = dist.get_rank(dp)
        mine = tokens[2 * k:2 * k + 2]
        losses = [float(tr.step(mine[:, :-1], mine[:, 1:])) for _ in range(3)]
        torch.manual_seed(0)
        ref_model = LlamaForCausalLM(cfg)
        ref = FlatTrainer(ref_model, lr=1e-2, weight_decay=0.0, max_grad_norm=1.0)
        for _ in range(3):
            ref.step(tokens[:, :-1], tokens[:, 1:])
        diff = max(float((p - r).abs().max()) for p, r in zip(model.parameters(), ref_model.parameters()))
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, (sums, diff, losses)))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR %r %s" % (e, traceback.format_exc())))


def pipeline_case(rank, world, port, q, backend="tcp", schedule="1f1b"):
    """Three pipeline stages as processes: loss and every gradient against the one-process model;
    posted sends keep their order; the next micro-batch's receive is posted ahead of its use."""
    import copy

    import torch
    from torch import nn

    from ferrotorch_b200.parallel import Pipeline

    try:
        torch.set_num_threads(1)
        if backend == "tcp":
            g = _group(rank, world, port, timeout=30.0)
            g.connect_mesh()
        else:
            import torch.distributed as dist

            from ferrotorch_b200.parallel.backend import TorchGroup

            dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
            g = TorchGroup()
        # ordered non-blocking transfers: eight posted messages arrive in posting order
        if rank == 0:
            ops = [g.isend(torch.full((3,), float(i)), 1) for i in range(8)]
            for op in ops:
                op.wait()
        elif rank == 1:
            bufs = [torch.empty(3) for _ in range(8)]
            ops = [g.irecv(b, 0) for b in bufs]
            for op in ops:
                op.wait()
            assert [float(b[0]) for b in bufs] == [float(i) for i in range(8)], bufs
        torch.manual_seed(0)
        stages = [nn.Sequential(nn.Linear(6, 8), nn.Tanh()), nn.Sequential(nn.Linear(8, 8), nn.Tanh()), nn.Linear(8, 3)]
        x, y = torch.randn(8, 6), torch.randn(8, 3)
        ref = copy.deepcopy(nn.Sequential(*stages))
        loss_ref = nn.functional.mse_loss(ref(x), y)
        loss_ref.backward()
        m = copy.deepcopy(stages[rank])
        p = Pipeline(m, g, n_micro=4, schedule=schedule, loss_fn=nn.functional.mse_loss)
        for step in range(2):                                   # second step: a fresh header, same shapes
            m.zero_grad(set_to_none=True)
            loss = p.train_step(x if rank == 0 else None, y if rank == world - 1 else None)
        if rank == world - 1:
            assert abs(float(loss) - float(loss_ref)) < 1e-6
        for got, want in zip(m.parameters(), ref[rank].parameters()):
            assert torch.allclose(got.grad, want.grad, atol=1e-6)
        if rank > 0:
            assert p.stats["prefetched_recvs"] >= 2 * 3, p.stats
        if rank < world - 1:
            assert p.stats["posted_sends"] >= 2 * 4, p.stats
        g.barrier()
        q.put((rank, "ok"))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR %r %s" % (e, traceback.format_exc())))


def torch_tp_baseline_case(rank, world, port, q):
    """The plain-torch tensor-parallel baseline model on two gloo ranks: its sharded loss equals
    the loss of the assembled unsharded weights, replicated parameters stay equal while training,
    the loss falls, greedy decoding gives the same tokens on both ranks."""
    import importlib.util

    import torch
    import torch.distributed as dist

    try:
        torch.set_num_threads(1)
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks", "bench_torch_tp.py")
        spec = importlib.util.spec_from_file_location("bench_torch_tp", path)
        B = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(B)
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
        solo = [dist.new_group([r]) for r in range(world)]
        s = dict(B.SHAPES["tiny"])
        torch.manual_seed(1234 + rank)
        dev, dt = torch.device("cpu"), torch.float32
        m = B.TPLlama(s, world, rank, dt, dev, 64)
        for p in [m.embed, m.norm] + [t for b in m.blocks for t in (b.n1, b.n2)]:
            dist.broadcast(p.data, 0)
        ids = torch.randint(0, s["vocab"], (3, 17), generator=torch.Generator().manual_seed(5))
        loss = m.loss(ids[:, :-1], ids[:, 1:], dist.group.WORLD)

        def gather(t):
            out = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(out, t.detach().contiguous())
            return out

        full = B.TPLlama(s, 1, 0, dt, dev, 64)
        with torch.no_grad():
            full.embed.copy_(m.embed), full.norm.copy_(m.norm)
            full.lm_head.copy_(torch.cat(gather(m.lm_head))[: full.lm_head.shape[0]])
            for fb, b in zip(full.blocks, m.blocks):
                d = b.d
                parts = [t.split([b.hq * d, b.hkv * d, b.hkv * d]) for t in gather(b.qkv)]
                fb.qkv.copy_(torch.cat([torch.cat([p[i] for p in parts]) for i in range(3)]))
                gu = [t.chunk(2) for t in gather(b.gate_up)]
                fb.gate_up.copy_(torch.cat([torch.cat([p[i] for p in gu]) for i in range(2)]))
                fb.o.copy_(torch.cat(gather(b.o), 1)), fb.down.copy_(torch.cat(gather(b.down), 1))
                fb.n1.copy_(b.n1), fb.n2.copy_(b.n2)
        want = full.loss(ids[:, :-1], ids[:, 1:], solo[rank])
        assert abs(float(loss) - float(want)) < 1e-4, (float(loss), float(want))
        # gradients of a replicated parameter agree with the unsharded model
        loss.backward(), want.backward()
        assert torch.allclose(m.embed.grad, full.embed.grad, atol=1e-5) and torch.allclose(m.blocks[0].n1.grad, full.blocks[0].n1.grad, atol=1e-5)
        assert torch.allclose(m.blocks[0].o.grad, full.blocks[0].o.grad.chunk(world, 1)[rank], atol=1e-5)
        opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
        first = last = None
        for _ in range(6):
            opt.zero_grad()
            l = m.loss(ids[:, :-1], ids[:, 1:], dist.group.WORLD)
            l.backward()
            opt.step()
            first, last = (float(l) if first is None else first), float(l)
        assert last < first
        for t in gather(m.embed):
            assert torch.equal(t, m.embed.detach())
        a = argparse_like(batch=2, prompt=9, new=4, prefill_seqs=1, warmup=0)
        out = B.run_decode(a, s, m, dist.group.WORLD, dev, world)
        assert out["decode_ms_per_step"] > 0 and out["new_tokens"] == 4
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except BaseException as e:  # noqa: BLE001
        import traceback

        q.put((rank, "ERR %r %s" % (e, traceback.format_exc())))


def argparse_like(**kw):
    import types

    return types.SimpleNamespace(**kw)


def comm_init_rank_worker(rank: int, world: int, port: int, uid: bytes, q) -> None:
    """Join a communicator by id (the reference's ``comm_init_rank``) and all-reduce over it."""
    import torch

    from ferrotorch_b200 import parallel as P

    g = P.comm_init_rank(world, uid, rank, "127.0.0.1", port)
    t = torch.tensor([float(rank + 1)])
    total = P.allreduce(t, g, P.ReduceOp.Sum)          # returns a new tensor
    q.put((rank, g.world_size, float(total)))
    import torch.distributed as dist

    dist.barrier()
    dist.destroy_process_group()
