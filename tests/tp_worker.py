"""Worker for the tensor-parallel kernel tests (torch.distributed.run, or plain python for world 1).

Checks ft_tp_ag_gemm against all_gather + matmul and ft_tp_gemm_rs against matmul +
reduce_scatter (fp32 references), for a large-M (prefill / training) and a small-M (decode)
shape, twice in a row on the same slot (epoch handling, counter reset)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import _native  # noqa: E402
from ferrotorch_b200.parallel.tensor_parallel import TPContext  # noqa: E402


def main():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    ctx = TPContext(group, dev, timeout_ms=20000)
    g = torch.Generator(device="cpu").manual_seed(5)

    def rnd(*s, scale=1.0):
        return (torch.randn(*s, generator=g) * scale).to(torch.bfloat16).to(dev)

    for (M, K, N) in [(1024, 512, 768), (64, 1024, 512), (300 * world, 256, 264)]:
        ms = ctx.rows_per_rank(M)
        for it in range(2):
            # ---- AG -> GEMM (column parallel): every rank has the full X to build the reference
            X = rnd(M, K)
            Wfull = rnd(N * world, K, scale=0.05)
            Wloc = Wfull[rank * N:(rank + 1) * N].contiguous()
            ctx.wait_gather_buffer_free(0)
            ctx.my_rows(0, M, K).copy_(X[rank * ms:min(M, (rank + 1) * ms)])
            y = ctx.ag_gemm(0, M, Wloc)
            torch.cuda.synchronize()
            ctx.check_status()
            want = X.float() @ Wloc.float().t()
            err = (y.float() - want).abs().max().item()
            assert err < 0.05 * (K ** 0.5) * 0.05 + 0.05, "ag_gemm M=%d it=%d rank %d err %g" % (M, it, rank, err)
            # ---- GEMM -> RS (row parallel): X sharded on K
            Xk = rnd(M, K * world)
            Wk = rnd(N, K * world, scale=0.05)
            xl = Xk[:, rank * K:(rank + 1) * K].contiguous()
            wl = Wk[:, rank * K:(rank + 1) * K].contiguous()
            res = rnd(M, N)
            lo, hi = rank * ms, min(M, (rank + 1) * ms)
            out = ctx.gemm_rs(1, xl, wl, residual=res[lo:hi].contiguous())
            torch.cuda.synchronize()
            ctx.check_status()
            want = (Xk.float() @ Wk.float().t() + res.float())[lo:hi]
            err = (out.float() - want).abs().max().item()
            tol = 0.05 + 0.02 * want.abs().max().item()
            assert err < tol, "gemm_rs M=%d it=%d rank %d err %g (tol %g)" % (M, it, rank, err, tol)
    if world > 1:
        dist.barrier()
    if rank == 0:
        print("tp kernels world=%d ok, launches %d" % (world, _native.launch_count()))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
