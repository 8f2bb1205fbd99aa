"""Worker for the multi-GPU data-parallel tests (launched with torch.distributed.run).

Trains a small Llama with FusedDDP on WORLD_SIZE GPUs and checks that (a) replicas are bitwise
identical after every step, (b) the weights match a single-process run on the concatenated
batch (rank 0 recomputes it), for mode fused and mode nccl.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import _native  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.parallel.ddp import FusedDDP  # noqa: E402
from ferrotorch_b200.train.engine import FlatTrainer  # noqa: E402


def make_model(cfg, device):
    torch.manual_seed(7)
    return LlamaForCausalLM(cfg).to(device, torch.bfloat16)


def main():
    mode = sys.argv[1] if len(sys.argv) > 1 else "fused"
    clip = None
    if mode == "fused_clip":
        # gradient clipping: reduce-only bucket kernels, then the norm and the clipped update
        mode, clip = "fused", 0.05
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512, intermediate_size=1408, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=256)
    hp = dict(optimizer="adamw", lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=clip)
    B, S, steps = 2, 128, 3
    g = torch.Generator().manual_seed(0)
    data = torch.randint(0, cfg.vocab_size, (steps, world * B, S + 1), generator=g).to(device)

    ddp = FusedDDP(dist.group.WORLD, mode=mode, bucket_mb=2.0, timeout_ms=20000)
    tr = FlatTrainer(make_model(cfg, device), micro_batches=2, ddp=ddp, allocator=ddp.allocator, **hp)
    ddp.broadcast_parameters(tr)
    for s in range(steps):
        t = data[s, rank * B:(rank + 1) * B]
        loss = tr.step(t[:, :-1], t[:, 1:])
        torch.cuda.synchronize()
        ddp.check_status()
        # (a) bitwise-identical replicas
        mine = tr.arena.params.clone()
        ref = mine.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(mine, ref), "rank %d diverged from rank 0 at step %d (%s)" % (rank, s, mode)
    # (b) single-process oracle on the concatenated batch
    if rank == 0:
        tr1 = FlatTrainer(make_model(cfg, device), micro_batches=2 * world, **hp)
        for s in range(steps):
            t = data[s]
            tr1.step(t[:, :-1], t[:, 1:])
        torch.cuda.synchronize()
        a, b = tr.master[: tr.arena.numel], tr1.master[: tr1.arena.numel]
        err = (a - b).abs().max().item()
        assert err < 5e-3, "DDP(%s) weights differ from the single-process run: max err %g" % (mode, err)
        print("ddp %s world=%d ok: loss %.4f, max |dW| vs single process %.2e, launches %d" %
              (mode, world, float(loss), err, _native.launch_count()))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
