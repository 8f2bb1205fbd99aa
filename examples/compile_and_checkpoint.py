#!/usr/bin/env python
"""Trace-and-fuse JIT, SafeTensors / GGUF round trips and a training checkpoint.

    python examples/compile_and_checkpoint.py [--device cuda]
"""
import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrotorch_b200 import jit, serialize  # noqa: E402
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.serialize.gguf import load_gguf_state_dict, write_gguf  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args()

    def gated(x, y):
        return torch.nn.functional.silu(x * 1.5 + y) * y - torch.tanh(x)

    x, y = torch.randn(1 << 16, device=a.device), torch.randn(1 << 16, device=a.device)
    fn = jit.compile(gated, (x, y))
    print("fused into %d kernel(s): %s" % (fn.graph.count("fused_elementwise"), fn.graph.ops()))
    assert torch.allclose(fn(x, y), gated(x, y), atol=1e-5)

    model = LlamaForCausalLM(LlamaConfig.tiny())
    with tempfile.TemporaryDirectory() as d:
        st = os.path.join(d, "model.safetensors")
        serialize.save_safetensors(model.hf_state_dict(), st)
        other = LlamaForCausalLM(LlamaConfig.tiny())
        other.load_hf_state_dict(serialize.load_safetensors(st))
        assert all(torch.equal(p, q) for p, q in zip(model.parameters(), other.parameters()))
        gg = os.path.join(d, "model.gguf")
        emb = model.model.embed_tokens.weight.detach().float()
        write_gguf(gg, {"token_embd.weight": (0, tuple(emb.shape), emb.numpy().tobytes())},      # ggml type 0 = F32
                   {"general.architecture": "llama"})
        back = load_gguf_state_dict(gg)
        print("gguf tensors:", {k: tuple(v.shape) for k, v in back.items()})
        ck = os.path.join(d, "train.ckpt")
        opt = torch.optim.AdamW(model.parameters())
        serialize.AsyncCheckpointer().save_async(ck, model.state_dict(), opt.state_dict(), step=7).wait()
        print("checkpoint step:", serialize.load_checkpoint(ck)["step"])
    return True


if __name__ == "__main__":
    main()
