"""Worker: LlamaEngine (paged KV, fused TP kernels) against a full-recompute oracle."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import _native  # noqa: E402
from ferrotorch_b200.models.engine import LlamaEngine  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
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
    # every rank needs at least one KV head: more heads (and a wider model) at 8 ranks
    kvh = 4 if world <= 4 else 8
    cfg = LlamaConfig(vocab_size=2048, hidden_size=512 if world <= 4 else 1024,
                      intermediate_size=1024 if world <= 4 else 2048, num_hidden_layers=2,
                      num_attention_heads=2 * kvh, num_key_value_heads=kvh, head_dim=64, max_position_embeddings=256,
                      initializer_range=0.08)
    torch.manual_seed(3)
    model = LlamaForCausalLM(cfg).to(dev, torch.bfloat16).eval()
    fmt = os.environ.get("FT_TEST_WEIGHTS", "bf16")
    if fmt == "q4_0":
        # the oracle gets the same rounding: every linear weight goes through Q4_0 and back (twice:
        # the second pass sees bf16 inputs like the engine does, and is a fixed point)
        from ferrotorch_b200.ops.quant import dequant_q4_0_planes, quantize_q4_0_planes
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() == 2 and "embed_tokens" not in name:
                    for _ in range(2):
                        p.copy_(dequant_q4_0_planes(*quantize_q4_0_planes(p)).to(p.dtype))
    sd = model.hf_state_dict()
    eng = LlamaEngine(cfg, TPContext(group, dev), max_batch=4, max_seq_len=128, weights=sd,
                      prefill_chunk_tokens=96, cuda_graph=os.environ.get("FT_TEST_GRAPH") == "1",
                      weight_format=fmt)
    B, S, new = 4, 48, 8
    prompts = torch.randint(0, cfg.vocab_size, (B, S), generator=torch.Generator().manual_seed(1)).to(dev)
    got = eng.generate(prompts, new)
    torch.cuda.synchronize()
    eng.tp.check_status()
    # oracle: recompute the whole prefix every step with the training model
    ids = prompts.clone()
    want = []
    with torch.no_grad():
        for _ in range(new):
            logits = model(ids, last_token_only=True)[:, -1].float()
            nxt = logits.argmax(-1)
            want.append(nxt)
            ids = torch.cat([ids, nxt[:, None]], 1)
    want = torch.stack(want, 1)
    agree = (got == want).float().mean().item()
    first = (got[:, 0] == want[:, 0]).float().mean().item()
    assert first == 1.0, "prefill tokens differ: %s vs %s" % (got[:, 0].tolist(), want[:, 0].tolist())
    assert agree >= 0.8, "decode disagreement %.2f\n%s\n%s" % (agree, got.tolist(), want.tolist())
    if world > 1:
        dist.barrier()
    if rank == 0:
        print("engine world=%d ok, agreement %.2f, launches %d" % (world, agree, _native.launch_count()))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
