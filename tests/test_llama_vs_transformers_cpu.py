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


def test_from_pretrained_reads_a_transformers_directory_and_round_trips(tmp_path):
    hf, _ = _pair(tie_word_embeddings=True)
    hf.save_pretrained(str(tmp_path / "hf"), safe_serialization=True)
    ours = LlamaForCausalLM.from_pretrained(str(tmp_path / "hf"), dtype=torch.float32).eval()
    ids = torch.randint(0, 128, (2, 11), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        assert torch.allclose(ours(ids).float(), hf(input_ids=ids).logits, atol=2e-4)
    assert ours.lm_head.weight is ours.model.embed_tokens.weight              # tied, as the config says
    ours.save_pretrained(str(tmp_path / "back"))
    again = tr.LlamaForCausalLM.from_pretrained(str(tmp_path / "back")).eval()   # and transformers reads ours
    with torch.no_grad():
        assert torch.allclose(again(input_ids=ids).logits, hf(input_ids=ids).logits, atol=1e-5)
    ours.save_pretrained(str(tmp_path / "sharded"), max_shard_bytes=64 << 10)
    sharded = LlamaForCausalLM.from_pretrained(str(tmp_path / "sharded"), dtype=torch.float32).eval()
    with torch.no_grad():
        assert torch.equal(sharded(ids), ours(ids))
    with pytest.raises(FileNotFoundError):
        (tmp_path / "empty").mkdir()
        (tmp_path / "empty" / "config.json").write_text((tmp_path / "back" / "config.json").read_text())
        LlamaForCausalLM.from_pretrained(str(tmp_path / "empty"))


def test_from_gguf_builds_the_model_the_file_describes(tmp_path):
    from ferrotorch_b200.serialize import gguf as G

    hf, ours = _pair()
    sd = ours.hf_state_dict()
    inv = {"model.embed_tokens": "token_embd", "model.norm": "output_norm", "lm_head": "output"}
    layer = {v: k for k, v in G._LAYER_MAP.items()}
    tensors = {}
    for k, v in sd.items():
        base, kind = k.rsplit(".", 1)
        if base in inv:
            name = "%s.%s" % (inv[base], kind)
        else:
            _, _, i, rest = base.split(".", 3)
            name = "blk.%s.%s.%s" % (i, layer[rest], kind)
        if v.dim() == 2 and "token_embd" not in name:
            tensors[name] = (G.GGML_F16, tuple(v.shape), v.to(torch.float16).numpy().tobytes())
        else:
            tensors[name] = (G.GGML_F32, tuple(v.shape), v.float().numpy().tobytes())
    md = {"general.architecture": "llama", "llama.embedding_length": 64, "llama.feed_forward_length": 112, "llama.block_count": 2,
          "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.context_length": 256,
          "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0, "llama.vocab_size": 128}
    path = str(tmp_path / "m.gguf")
    G.write_gguf(path, tensors, md)
    model = LlamaForCausalLM.from_gguf(path, dtype=torch.float32).eval()
    assert (model.config.num_key_value_heads, model.config.intermediate_size, model.config.tie_word_embeddings) == (2, 112, False)
    ids = torch.randint(0, 128, (1, 9), generator=torch.Generator().manual_seed(4))
    with torch.no_grad():
        assert torch.allclose(model(ids).float(), ours(ids).float(), atol=5e-3)       # weights went through fp16


def test_inferencer_logits_and_sparsity_profile_match_hooks_on_transformers():
    """``LlamaGpuInferencer`` (on the host here): last-position and all-position logits, and the
    profiled forward's per-head / per-block magnitudes and bootstrap state against the same
    quantities tapped from the ``transformers`` twin with hooks on ``o_proj`` / ``down_proj``."""
    from ferrotorch_b200.models.inferencer import GraphedDecoder, LlamaGpuInferencer

    hf, ours = _pair()
    inf = LlamaGpuInferencer(ours, device="cpu")
    ids = torch.randint(0, 128, (11,), generator=torch.Generator().manual_seed(4)).tolist()
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([ids])).logits[0]
    assert torch.allclose(inf.forward_logits_from_ids_all(ids), want, atol=2e-4, rtol=1e-4)
    assert torch.allclose(inf.forward_from_ids(ids), want[-1], atol=2e-4, rtol=1e-4)
    # taps on the twin
    S, Hq, D, I = len(ids), 4, 16, 112
    attn_in, mlp_in, layer_out = [], [], []
    hs = []
    for layer in hf.model.layers:
        hs.append(layer.self_attn.o_proj.register_forward_pre_hook(lambda m, a: attn_in.append(a[0].detach())))
        hs.append(layer.mlp.down_proj.register_forward_pre_hook(lambda m, a: mlp_in.append(a[0].detach())))
        hs.append(layer.register_forward_hook(lambda m, a, o: layer_out.append((o[0] if isinstance(o, tuple) else o).detach())))
    with torch.no_grad():
        hf(input_ids=torch.tensor([ids]))
    for h in hs:
        h.remove()
    block, nb = 16, 7
    prof = inf.forward_from_ids_profiled_with_bootstrap(ids, block, nb, bootstrap_k=1)
    assert prof.seq_len == S and prof.hidden_size == 64 and prof.bootstrap_k == 1
    assert prof.attn_magnitudes.shape == (S, 2, Hq) and prof.mlp_magnitudes.shape == (S, 2, nb)
    for li in range(2):
        a = attn_in[li].reshape(S, Hq, D).abs().amax(-1)
        m = mlp_in[li].reshape(S, nb, block).abs().amax(-1)
        assert torch.allclose(prof.attn_magnitudes[:, li], a, atol=1e-4, rtol=1e-4)
        assert torch.allclose(prof.mlp_magnitudes[:, li], m, atol=1e-4, rtol=1e-4)
    assert torch.allclose(prof.bootstrap_hidden, layer_out[0].reshape(S, 64), atol=1e-4, rtol=1e-4)
    assert prof.attn_at(3, 1, 2) == float(prof.attn_magnitudes[3, 1, 2])
    # the local plain-act variant: |gated * (y @ W_down)| per block, y the layer's output
    pl = inf.forward_from_ids_profiled_with_bootstrap(ids, block, nb, None, True)
    for li, layer in enumerate(hf.model.layers):
        z = layer_out[li].reshape(S, 64) @ layer.mlp.down_proj.weight.detach()
        m = (mlp_in[li].reshape(S, I) * z).reshape(S, nb, block).abs().amax(-1)
        assert torch.allclose(pl.mlp_magnitudes[:, li], m, atol=1e-4, rtol=1e-3)
    assert pl.bootstrap_hidden is None and torch.equal(pl.attn_magnitudes, prof.attn_magnitudes)
    assert inf.forward_from_ids_profiled(ids, block, nb).bootstrap_hidden is None
    for bad in ((0, 7), (16, 6), (16, 0)):
        with pytest.raises(ValueError):
            inf.forward_from_ids_profiled(ids, *bad)
    with pytest.raises(ValueError):
        inf.forward_from_ids_profiled_with_bootstrap(ids, block, nb, 3)
    with pytest.raises(ValueError):
        inf.forward_from_ids([128])
    # the decoder object: same logits as the single-token forward, calls counted
    dec = GraphedDecoder.capture(inf, warmup_token=1)
    for i, tok in enumerate((5, 99, 5)):
        assert torch.equal(dec.decode_step(tok), inf.forward_from_ids([tok])) and dec.num_replays() == i + 1
    with pytest.raises(ValueError):
        dec.decode_step(1000)
    assert "num_replays=3" in repr(dec)
    # the value cache walks to the same logits, and the 4-bit HQQ container loads
    from ferrotorch_b200.models.llama_compat import LlamaKvCache

    cache = LlamaKvCache.empty()
    for i, tok in enumerate(ids[:5]):
        logits, cache = ours.forward_one_with_cache(tok, cache)
        assert torch.allclose(logits.float(), want[i], atol=2e-4, rtol=1e-4) and len(cache) == i + 1
    assert cache.layers[0].k.shape == (2, 5, 16)
    assert ours.forward_from_ids(ids).shape == (1, S, 128)
    with pytest.raises(ValueError):
        ours.forward_one_with_cache(1, LlamaKvCache.empty().extend([(torch.zeros(2, 1, 16), torch.zeros(2, 1, 16))] * 3))
