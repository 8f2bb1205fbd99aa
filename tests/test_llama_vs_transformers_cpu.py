"""The Llama stack against Hugging Face ``transformers`` on shared random weights (CPU, fp32): logits,
RoPE scaling variants, tied embeddings, KV-cache generation, and the state-dict round trip.  The
reference checks itself the same way against pinned PyTorch runs
(ferrotorch-llama/tests/conformance_pretrained_causal_lm.rs, scripts/verify_*_inference.py)."""
import pytest
import torch

from ferrotorch_b200.models.generation import GenerationConfig, generate
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM

tr = pytest.importorskip("transformers")

BASE = dict(vocab_size=128, hidden_size=64, intermediate_size=112, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0)


def _pair(**over):
    kw = dict(BASE, **over)
    torch.manual_seed(0)
    hf_kw = dict(kw)
    hf = tr.LlamaForCausalLM(tr.LlamaConfig(**hf_kw, attention_bias=False, mlp_bias=False)).eval()
    ours = LlamaForCausalLM(LlamaConfig.from_hf(hf.config.to_dict())).eval()
    ours.load_hf_state_dict(hf.state_dict())
    return hf, ours


@pytest.mark.parametrize("over", [
    {},                                                               # GQA, plain RoPE
    {"num_key_value_heads": 4},                                      # multi-head
    {"num_key_value_heads": 1, "rope_theta": 500000.0},              # multi-query
    {"tie_word_embeddings": True},
    {"rope_scaling": {"rope_type": "linear", "factor": 2.0}},
    {"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 64}},
], ids=["gqa", "mha", "mqa", "tied", "linear", "llama3"])
def test_logits_match_transformers(over):
    hf, ours = _pair(**over)
    ids = torch.randint(0, 128, (2, 37), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = ours(ids).float()
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max()


def test_greedy_generation_with_kv_cache_matches_transformers():
    hf, ours = _pair()
    ids = torch.randint(0, 128, (2, 9), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        want = hf.generate(ids, max_new_tokens=12, do_sample=False, pad_token_id=0)
    got = generate(ours, ids, GenerationConfig.greedy(12))
    assert torch.equal(got, want)


def test_state_dict_round_trip_keeps_hf_names():
    hf, ours = _pair()
    back = ours.hf_state_dict()
    ref = hf.state_dict()
    assert set(back) == set(ref)
    for k in ref:
        assert torch.equal(back[k], ref[k]), k
