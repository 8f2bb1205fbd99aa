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
        g = _group(rank, world, port, timeout=1.0)
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
