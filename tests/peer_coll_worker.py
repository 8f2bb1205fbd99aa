"""Worker for the peer-memory collective tests (torch.distributed.run): all-gather, even and
uneven all-to-all, all-reduce and reduce-scatter of ``PeerCollectives`` against torch.distributed,
several calls in a row on the same buffers."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200.parallel.peer_collectives import PeerCollectives  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pc = PeerCollectives(dist.group.WORLD, dev, max_bytes=32 << 20, timeout_ms=8000)
    g = torch.Generator().manual_seed(100 + rank)
    for it in range(3):
        # all-gather (one aligned size, one that needs padding)
        for shape, dt in (((1024, 64), torch.bfloat16), ((7, 3), torch.float32)):
            x = torch.randn(*shape, generator=g).to(dt).to(dev)
            want = torch.empty((world * shape[0],) + shape[1:], device=dev, dtype=dt)
            dist.all_gather_into_tensor(want, x)
            got = pc.all_gather(x)
            assert torch.equal(got, want), "all_gather %s it %d" % (shape, it)
        # even all-to-all
        x = torch.randn(world * 96, 40, generator=g).to(torch.bfloat16).to(dev)
        want = torch.empty_like(x)
        dist.all_to_all_single(want, x)
        assert torch.equal(pc.all_to_all(x), want), "all_to_all it %d" % it
        # uneven: rank r sends (r + d + 1) rows to rank d
        send = [rank + d + 1 for d in range(world)]
        recv = [s + rank + 1 for s in range(world)]
        x = torch.randn(sum(send), 5, generator=g).to(dev)
        want = torch.empty(sum(recv), 5, device=dev)
        dist.all_to_all_single(want, x, output_split_sizes=recv, input_split_sizes=send)
        assert torch.equal(pc.all_to_all(x, send, recv), want), "uneven all_to_all it %d" % it
        # all-reduce: every rank must end with the same bits; value matches NCCL within rounding
        for dt, n in ((torch.float32, 100003), (torch.bfloat16, 1 << 20)):
            x = torch.randn(n, generator=g).to(dt).to(dev)
            want = x.clone().float()
            dist.all_reduce(want)
            got = pc.all_reduce_(x.clone())
            tol = 1e-5 if dt == torch.float32 else 2e-2
            assert (got.float() - want).abs().max() <= tol * max(1.0, float(want.abs().max())), "all_reduce %s" % dt
            ref = got.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(ref, got), "ranks disagree bitwise after all_reduce"
        x = torch.randn(world * 33, 8, generator=g).to(dev)
        want = x.clone()
        dist.all_reduce(want)
        got = pc.reduce_scatter(x)
        assert torch.allclose(got, want[rank * 33:(rank + 1) * 33], atol=1e-5), "reduce_scatter"
    torch.cuda.synchronize()
    pc.check_status()
    if rank == 0:
        print("peer collectives world=%d ok" % world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
