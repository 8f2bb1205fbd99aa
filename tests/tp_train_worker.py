"""Worker for the tensor-parallel *training* tests (torch.distributed.run, or plain python for
world 1).

1. The backward forms of the fused kernels against fp32 references: ``allgather(X) @ W`` with the
   weight stored ``[K, N]``, ``reduce_scatter(X @ W)`` likewise, and the gather-only launch.
2. A sharded Llama against the unsharded model with the same weights: loss and every gradient.
3. A few optimizer steps through the flat-arena trainer on the shards.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.models.llama_tp import TPLlamaForCausalLM, make_tp_trainer  # noqa: E402
from ferrotorch_b200.parallel.tensor_parallel import TPContext  # noqa: E402


def rel(a, b):
    a, b = a.float(), b.float()
    return float((a - b).norm() / b.norm().clamp_min(1e-6))


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
    tp = TPContext(group, dev, timeout_ms=int(os.environ.get("FT_COMM_TIMEOUT_MS", "10000")))
    g = torch.Generator(device="cpu").manual_seed(11)

    def rnd(*s, scale=1.0):
        return (torch.randn(*s, generator=g) * scale).to(torch.bfloat16).to(dev)

    # ------------------------------------------------------------------ 1. kernel forms
    for (M, K, N) in [(1024, 512, 384), (256 * world, 320, 200)]:
        ms = tp.rows_per_rank(M)
        lo, hi = rank * ms, min(M, (rank + 1) * ms)
        for it in range(2):
            X = rnd(M, K)
            Wkn = rnd(K, N, scale=0.05)                    # stored [K, N]
            tp.wait_gather_buffer_free(13)
            tp.my_rows(13, M, K).copy_(X[lo:hi])
            y = tp.ag_gemm(13, M, Wkn, w_is_kn=True)
            torch.cuda.synchronize()
            tp.check_status()
            e = rel(y, X.float() @ Wkn.float())
            assert e < 2e-2, "ag_gemm[kn] M=%d it=%d rank %d rel %g" % (M, it, rank, e)
            assert torch.equal(tp.gather_buffer(13, M, K), X), "gather buffer incomplete after ag_gemm"

            Xl = rnd(M, K)                                 # this rank's partial operand
            xs = [torch.empty_like(Xl) for _ in range(world)]
            if world > 1:
                dist.all_gather(xs, Xl)
            else:
                xs = [Xl]
            out = tp.gemm_rs(14, Xl, Wkn, w_is_kn=True)
            torch.cuda.synchronize()
            tp.check_status()
            want = sum(x.float() for x in xs) @ Wkn.float()
            e = rel(out, want[lo:hi])
            assert e < 2e-2, "gemm_rs[kn] M=%d it=%d rank %d rel %g" % (M, it, rank, e)

            tp.wait_gather_buffer_free(15)
            tp.my_rows(15, M, K).copy_(X[lo:hi])
            full = tp.all_gather_rows(15, M, K)
            torch.cuda.synchronize()
            tp.check_status()
            assert torch.equal(full, X), "all_gather_rows M=%d it=%d rank %d" % (M, it, rank)

    # ------------------------------------------------------------------ 2. model equivalence
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=16, num_key_value_heads=8, head_dim=64, max_position_embeddings=512)
    torch.manual_seed(0)
    full_model = LlamaForCausalLM(cfg).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        for n, p in full_model.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)        # norm weights away from 1 so their grads matter
    B, S = 2, 256
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=g).to(dev)
    labels = torch.randint(0, cfg.vocab_size, (B, S), generator=g).to(dev)
    loss_ref = full_model(ids, labels=labels)
    loss_ref.backward()

    tp_model = TPLlamaForCausalLM(cfg, tp).load_full(full_model)
    for use_ckpt in (False, True):
        tp_model.checkpoint_layers = use_ckpt
        tp_model.zero_grad(set_to_none=True)
        loss = tp_model(ids, labels=labels)
        loss.backward()
        tp_model.sync_replicated_grads()
        torch.cuda.synchronize()
        tp.check_status()
        assert abs(float(loss) - float(loss_ref)) < 2e-2 * abs(float(loss_ref)), (float(loss), float(loss_ref))
        for name, mine, ref in tp_model.full_grad_slices(full_model):
            e = rel(mine, ref)
            assert e < 6e-2, "grad %s (ckpt=%s) rank %d rel %g" % (name, use_ckpt, rank, e)

    # ------------------------------------------------------------------ 3. optimizer steps
    tp_model.checkpoint_layers = False
    tp_model.zero_grad(set_to_none=True)
    tr = make_tp_trainer(tp_model, lr=1e-3, weight_decay=0.1, max_grad_norm=1.0, micro_batches=2)
    losses = [float(tr.step(ids, labels)) for _ in range(6)]
    torch.cuda.synchronize()
    tp.check_status()
    assert losses[-1] < losses[0], losses
    if world > 1:
        t = torch.tensor(losses, device=dev)
        ts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(ts, t)
        assert all(torch.equal(ts[0], x) for x in ts), "ranks disagree on the loss"
        # replicated weights stay identical on every rank
        w = tp_model.norm.weight.detach().clone()
        ws = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(ws, w)
        assert all(torch.equal(ws[0], x) for x in ws), "replicated weights diverged"
    if rank == 0:
        print("ok losses", losses)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
