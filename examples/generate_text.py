#!/usr/bin/env python
"""Sampling, beam search, speculative decoding and JSON-constrained decoding with a random tiny
Llama (the calls are the same for a loaded checkpoint: ``model.load_hf_state_dict(...)``).

    python examples/generate_text.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from ferrotorch_b200.models.generation import (GenerationConfig, GrammarLogitsProcessor, beam_search, generate,  # noqa: E402
                                               speculative_decode)
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM  # noqa: E402
from ferrotorch_b200.utils.text import JsonGrammar  # noqa: E402


def main():
    torch.manual_seed(0)
    vocab = ["{", "}", '"k"', ":", ",", "1", "2", "[", "]", "true", "null", " ", "<eos>"] + ["w%d" % i for i in range(51)]
    cfg = LlamaConfig(vocab_size=len(vocab), hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=256)
    model, draft = LlamaForCausalLM(cfg).eval(), LlamaForCausalLM(cfg).eval()
    prompt = torch.tensor([[13, 14, 15]])
    eos = vocab.index("<eos>")
    out = generate(model, prompt, GenerationConfig(max_new_tokens=12, do_sample=True, top_k=20, top_p=0.9,
                                                   temperature=0.8, repetition_penalty=1.1, seed=1))
    print("sampled      :", out[0].tolist())
    print("beam search  :", beam_search(model, prompt, num_beams=3, max_new_tokens=8)[0].tolist())
    spec, stats = speculative_decode(model, draft, prompt, max_new_tokens=12, gamma=3)
    print("speculative  :", spec[0].tolist(), stats)
    js = generate(model, prompt, GenerationConfig(max_new_tokens=24, do_sample=True, seed=3, eos_token_id=eos),
                  logits_processor=GrammarLogitsProcessor(JsonGrammar(), vocab, eos))
    text = "".join(vocab[t] for t in js[0, 3:].tolist() if t != eos)
    print("json-masked  :", text)
    assert JsonGrammar().accepts_prefix(text)
    return text


if __name__ == "__main__":
    main()
