#!/usr/bin/env python
"""Same-box baselines for the Llama inference benchmark (``bench_inference.py``): the same model
shape, batch, prompt and generation length through two library stacks on one GPU.

    python benchmarks/bench_inference_baselines.py --impl hf      # transformers generate(), SDPA, eager
    python benchmarks/bench_inference_baselines.py --impl vllm    # vLLM offline engine, dummy weights

Random-init (``hf``) / dummy (``vllm``) bf16 weights, uniform-random prompt ids, greedy sampling with
the end-of-sequence token ignored, so every sequence produces exactly ``--new`` tokens.  Decode
time per step = (time of prompt + ``--new`` tokens - time of prompt + 1 token) / (``--new`` - 1),
both measured after one untimed run of the same call.  None of this library's kernels run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time

LLAMA = {
    "llama3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5),
    "small": dict(vocab_size=32000, hidden_size=2048, intermediate_size=8192, num_hidden_layers=8,
                  num_attention_heads=16, num_key_value_heads=8, rope_theta=500000.0, rms_norm_eps=1e-5),
}


def run_hf(a, shape):
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(max_position_embeddings=a.prompt + a.new + 32, tie_word_embeddings=False,
                      attn_implementation="sdpa", **shape)
    with torch.device("cuda"):
        model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), device="cuda")

    def gen(n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        with torch.no_grad():
            # the default (dynamic) cache: the static one routes generate() through torch.compile
            out = model.generate(ids, max_new_tokens=n, min_new_tokens=n, do_sample=False, pad_token_id=0)
        e1.record()
        torch.cuda.synchronize()
        assert out.shape[1] == a.prompt + n
        return e0.elapsed_time(e1)

    gen(4)
    ms1 = gen(1)
    msn = gen(a.new)
    return ms1, msn, "transformers generate(): SDPA attention, dynamic KV cache, eager"


def run_vllm(a, shape):
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    import numpy as np
    from vllm import LLM, SamplingParams

    d = tempfile.mkdtemp(prefix="ft_vllm_cfg_")
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", torch_dtype="bfloat16",
               max_position_embeddings=a.prompt + a.new + 32, tie_word_embeddings=False, bos_token_id=1, eos_token_id=2,
               head_dim=shape["hidden_size"] // shape["num_attention_heads"], **shape)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", tensor_parallel_size=1,
              max_model_len=a.prompt + a.new + 32, max_num_seqs=a.batch, gpu_memory_utilization=0.6,
              enable_prefix_caching=False, seed=0)
    rng = np.random.default_rng(0)
    prompts = [{"prompt_token_ids": rng.integers(3, shape["vocab_size"], a.prompt).tolist()} for _ in range(a.batch)]

    def gen(n):
        sp = SamplingParams(max_tokens=n, min_tokens=n, temperature=0.0, ignore_eos=True, detokenize=False)
        t0 = time.perf_counter()
        outs = llm.generate(prompts, sp, use_tqdm=False)
        ms = (time.perf_counter() - t0) * 1e3
        assert all(len(o.outputs[0].token_ids) == n for o in outs)
        return ms

    gen(4)
    ms1 = gen(1)
    msn = gen(a.new)
    return ms1, msn, "vLLM offline engine, dummy weights, default CUDA-graph decode; host wall clock around generate()"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="hf", choices=["hf", "vllm"])
    ap.add_argument("--model", default="llama3-8b", choices=sorted(LLAMA))
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    a = ap.parse_args()
    shape = LLAMA[a.model]
    try:
        ms1, msn, how = (run_hf if a.impl == "hf" else run_vllm)(a, shape)
    except Exception as e:  # noqa: BLE001  (a baseline that cannot start is reported, not fatal)
        print(json.dumps({"metric": "llama_decode_tokens_per_s", "impl": a.impl, "unavailable": "%s: %s" % (type(e).__name__, str(e)[:300])}))
        return 0
    step = (msn - ms1) / max(1, a.new - 1)
    print(json.dumps({
        "metric": "llama_decode_tokens_per_s", "impl": a.impl, "model": a.model, "tp": 1, "batch": a.batch,
        "prompt": a.prompt, "new_tokens": a.new, "prefill_ms": ms1, "prefill_tokens_per_s": a.batch * a.prompt / (ms1 / 1e3),
        "decode_ms_per_step": step, "decode_tokens_per_s": a.batch / (step / 1e3), "total_ms": msn, "how": how,
        "dtype": "bf16", "data": "synthetic"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
