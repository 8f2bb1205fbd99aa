"""Model families on CPU: ResNet shapes / registry, Llama generation utilities (sampling filters,
cached generate == full recompute, beam search, speculative decoding == greedy)."""
import pytest
import torch

from ferrotorch_b200.models import generation as G
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
from ferrotorch_b200.models.resnet import create_model, list_models, resnet18, resnet50
from ferrotorch_b200.train import FlatTrainer


def test_resnet_shapes_registry_and_training_step():
    m = resnet50(num_classes=10)
    assert sum(p.numel() for p in m.parameters()) == 23_528_522
    assert m(torch.randn(2, 3, 64, 64)).shape == (2, 10)
    assert "resnet50" in list_models() and isinstance(create_model("resnet18", num_classes=3), type(resnet18()))
    with pytest.raises(KeyError):
        create_model("no_such_model")
    small = resnet18(num_classes=4)
    tr = FlatTrainer(small, optimizer="sgd", lr=0.05, momentum=0.9, weight_decay=1e-4,
                     loss_fn=lambda mod, x, y: torch.nn.functional.cross_entropy(mod(x), y))
    x, y = torch.randn(8, 3, 32, 32), torch.randint(0, 4, (8,))
    losses = [float(tr.step(x, y)) for _ in range(6)]
    assert losses[-1] < losses[0]


def _tiny():
    cfg = LlamaConfig.tiny()
    cfg.num_hidden_layers = 2
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).eval()


def test_sampling_filters():
    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0]])
    assert G.filter_top_k_top_p(logits, top_k=2).isinf().sum() == 2
    kept = G.filter_top_k_top_p(logits, top_p=0.7)
    assert not kept[0, 1].isinf() and not kept[0, 2].isinf() and kept[0, 3].isinf()
    pen = G.apply_repetition_penalty(torch.tensor([[2.0, -2.0, 1.0]]), torch.tensor([[0, 1]]), 2.0)
    assert pen.tolist() == [[1.0, -4.0, 1.0]]
    cfg = G.GenerationConfig(do_sample=True, temperature=0.7, top_k=3, seed=1)
    g = torch.Generator().manual_seed(1)
    t = G.sample_next(torch.randn(5, 50), cfg, generator=g)
    assert t.shape == (5,)


def test_cached_generate_matches_full_recompute_and_streams():
    m = _tiny()
    ids = torch.randint(0, 4096, (2, 7), generator=torch.Generator().manual_seed(3))
    seen = []
    out = G.generate(m, ids, G.GenerationConfig(max_new_tokens=5), streamer=seen.append)
    ref = ids
    with torch.no_grad():
        for _ in range(5):
            ref = torch.cat([ref, m(ref, last_token_only=True)[:, -1].argmax(-1)[:, None]], 1)
    assert torch.equal(out, ref) and len(seen) == 5
    eos = int(out[0, 8])
    stopped = G.generate(m, ids[:1], G.GenerationConfig(max_new_tokens=5, eos_token_id=eos))
    assert stopped.shape[1] <= 12 and int(stopped[0, -1]) == eos


def test_beam_search_and_speculative_decoding():
    m = _tiny()
    ids = torch.randint(0, 4096, (1, 5), generator=torch.Generator().manual_seed(4))
    greedy = G.generate(m, ids, G.GenerationConfig(max_new_tokens=6))
    beam1 = G.beam_search(m, ids, num_beams=1, max_new_tokens=6)
    assert torch.equal(beam1, greedy)
    beam4 = G.beam_search(m, ids, num_beams=4, max_new_tokens=6)

    def logp(seq):
        with torch.no_grad():
            lp = m(seq[:, :-1]).float().log_softmax(-1)
        return float(lp[0, 4:].gather(-1, seq[0, 5:, None]).sum())

    assert logp(beam4) >= logp(greedy) - 1e-4
    cfg2 = LlamaConfig.tiny()
    cfg2.num_hidden_layers = 1
    torch.manual_seed(9)
    draft = LlamaForCausalLM(cfg2).eval()
    out, stats = G.speculative_decode(m, draft, ids, max_new_tokens=6, gamma=3)
    assert torch.equal(out, greedy) and stats["proposed"] >= stats["accepted"] and stats["target_calls"] <= 6
    out2, stats2 = G.speculative_decode(m, m, ids, max_new_tokens=6, gamma=3)
    assert torch.equal(out2, greedy) and stats2["accepted"] == stats2["proposed"]


def test_grammar_constrained_generate_yields_valid_json():
    import json

    from ferrotorch_b200.models.generation import GenerationConfig, GrammarLogitsProcessor, generate
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.utils.text import JsonGrammar

    vocab = ["{", "}", '"a"', '"b"', ":", ",", "1", "2", "[", "]", "true", " ", "<eos>", "x", "y", "z"]
    cfg = LlamaConfig(vocab_size=len(vocab), hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=1, head_dim=16, max_position_embeddings=128)
    torch.manual_seed(3)
    model = LlamaForCausalLM(cfg).eval()
    eos = vocab.index("<eos>")
    proc = GrammarLogitsProcessor(JsonGrammar(), vocab, eos)
    g = JsonGrammar()
    for seed in range(4):
        out = generate(model, torch.tensor([[0, 4, 6]]), GenerationConfig(max_new_tokens=24, do_sample=True, seed=seed,
                                                                          temperature=1.5, eos_token_id=eos),
                       logits_processor=proc)
        text = "".join(vocab[t] for t in out[0, 3:].tolist() if t != eos)
        assert g.accepts_prefix(text), text
        if eos in out[0, 3:].tolist():
            json.loads(text)


def test_flat_trainer_trajectory_matches_torch_adamw_with_clipping():
    """Five optimizer steps of the flat-arena trainer (micro-batches, global-norm clipping, decay only
    on matrices) against the same loop written with torch.optim.AdamW + clip_grad_norm_."""
    import copy

    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.train.engine import FlatTrainer

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=8, max_position_embeddings=64)
    ours = LlamaForCausalLM(cfg)
    ref = copy.deepcopy(ours)
    hp = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    tr = FlatTrainer(ours, optimizer="adamw", weight_decay=0.1, max_grad_norm=0.5, micro_batches=2, **hp)
    decay = [p for p in ref.parameters() if p.dim() >= 2]
    no_decay = [p for p in ref.parameters() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}], **hp)
    g = torch.Generator().manual_seed(1)
    for step in range(5):
        t = torch.randint(0, cfg.vocab_size, (4, 17), generator=g)
        x, y = t[:, :-1], t[:, 1:]
        loss = tr.step(x, y)
        opt.zero_grad()
        total = 0.0
        for i in range(2):                                   # the same two micro-batches
            l = ref(x[2 * i:2 * i + 2], labels=y[2 * i:2 * i + 2], loss_denominator=y.numel())
            l.backward()
            total += float(l)
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
        assert abs(float(loss) - total) < 1e-5, (step, float(loss), total)
    for (n, p), q in zip(ours.named_parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=2e-5), (n, float((p - q).abs().max()))


def test_generation_primitives_and_loader_aliases():
    from ferrotorch_b200.models import generation as G
    from ferrotorch_b200.serialize import gguf, quant_loaders as Q

    logits = torch.tensor([[1.0, 3.0, 2.0, 0.0]])
    assert G.argmax(logits).tolist() == [1] and torch.equal(G.apply_temperature(logits, 2.0), logits / 2)
    assert torch.isinf(G.top_k_filter(logits, 2)).sum() == 2 and G.top_k_filter(logits, 2)[0, 1] == 3.0
    kept = G.top_p_filter(logits, 0.6)
    assert kept[0, 1] == 3.0 and torch.isinf(kept[0, 3]) and torch.isinf(kept[0, 0])
    assert G.sample_softmax(torch.tensor([[0.0, 50.0]])).tolist() == [1]
    with pytest.raises(ValueError):
        G.apply_temperature(logits, 0.0)
    out = G.SpecDecodeOutput(torch.zeros(1, 3), proposed=8, accepted=6, target_calls=2)
    assert out.acceptance_rate() == 0.75 and G.SpecDecodeConfig().gamma == 4
    sd = gguf.gguf_to_hf_state_dict({"blk.0.attn_q.weight": torch.zeros(1), "token_embd.weight": torch.zeros(1), "x": torch.zeros(1)})
    assert set(sd) == {"model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight", "x"}
    assert Q.dequantize_gptq_q4 is Q.dequantize_gptq and Q.dequantize_awq_q4 is Q.dequantize_awq
    w = torch.randn(8, 64)
    wq, scale, zero = Q.pack_hqq(w)[:3]
    dense = Q.hqq_state_dict_to_dense({"l.W_q": wq, "l.scale": scale, "l.zero": zero, "l.shape": torch.tensor([8, 64]),
                                       "norm.weight": torch.ones(3)})
    assert set(dense) == {"l.weight", "norm.weight"} and (dense["l.weight"] - w).abs().max() < 0.5


def test_resnet_folded_for_inference_matches_eval_model():
    from ferrotorch_b200.models import resnet as R

    torch.manual_seed(0)
    for ctor in (R.resnet18, R.resnet50):
        m = ctor(num_classes=7)
        for mod in m.modules():                                  # non-trivial running statistics and affine terms
            if isinstance(mod, torch.nn.BatchNorm2d):
                mod.running_mean.normal_(0, 0.1)
                mod.running_var.uniform_(0.5, 1.5)
                mod.weight.data.uniform_(0.5, 1.5)
                mod.bias.data.normal_(0, 0.1)
        with pytest.raises(ValueError):
            R.fuse_for_inference(m)
        m.eval()
        fused = R.fuse_for_inference(m)
        x = torch.randn(2, 3, 64, 64)
        with torch.no_grad():
            ref = m(x)
        torch.testing.assert_close(fused(x), ref, rtol=1e-3, atol=1e-3)
        assert not any(isinstance(mod, torch.nn.BatchNorm2d) for mod in fused.modules())
    conv, bn = torch.nn.Conv2d(4, 6, 3, bias=True), torch.nn.BatchNorm2d(6).eval()
    bn.running_mean.normal_()
    bn.running_var.uniform_(0.5, 2.0)
    w, b = R.fold_conv_bn(conv, bn)
    xx = torch.randn(1, 4, 5, 5)
    torch.testing.assert_close(torch.nn.functional.conv2d(xx, w, b), bn(conv(xx)), rtol=1e-4, atol=1e-5)


# --------------------------------------------------------------------------- speculative sampling (rejection step)
def test_speculative_sampling_keeps_the_target_distribution_and_repeats_by_seed():
    from ferrotorch_b200.models.spec_decode import (FunctionHandle, LlamaHandle, ModelHandle, SpecSamplingConfig,
                                                    residual_distribution, speculative_sample)

    V = 4
    g = torch.Generator().manual_seed(3)
    T, D = torch.randn(V, V, generator=g, dtype=torch.float64) * 1.5, torch.randn(V, V, generator=g, dtype=torch.float64) * 1.5
    target, draft = FunctionHandle(lambda ids: T[ids[-1]], V), FunctionHandle(lambda ids: D[ids[-1]], V)
    # exact joint distribution of two tokens sampled from the target after the prompt token 1
    P = torch.softmax(T, -1)
    joint = P[1][:, None] * P
    counts = torch.zeros(V, V, dtype=torch.float64)
    n, acc, prop = 6000, 0, 0
    for seed in range(n):
        o = speculative_sample(target, draft, [0, 1], SpecSamplingConfig(draft_k=2, max_new_tokens=2, seed=seed))
        assert len(o.tokens) == 2 and o.target_calls <= 2
        counts[o.tokens[0], o.tokens[1]] += 1
        acc, prop = acc + o.accepted_count, prop + o.proposed_count
    tv = 0.5 * (counts / n - joint).abs().sum()
    assert float(tv) < 0.035, float(tv)                  # sampling noise of 6000 draws over 16 cells is about 0.02
    assert 0.2 < acc / prop < 0.95                       # a different draft is sometimes rejected
    # the draft's own distribution is clearly different, so the match above is the rejection step's doing
    Q = torch.softmax(D, -1)
    assert float(0.5 * (Q[1][:, None] * Q - joint).abs().sum()) > 0.15
    # draft == target: everything is accepted
    o = speculative_sample(target, target, [2], SpecSamplingConfig(draft_k=3, max_new_tokens=9, seed=1))
    assert o.accepted_count == o.proposed_count and o.acceptance_rate() == 1.0 and len(o.tokens) == 9
    # same seed, same tokens; eos stops; validation
    a = speculative_sample(target, draft, [0], SpecSamplingConfig(draft_k=3, max_new_tokens=12, seed=5)).tokens
    assert a == speculative_sample(target, draft, [0], SpecSamplingConfig(draft_k=3, max_new_tokens=12, seed=5)).tokens
    assert a != speculative_sample(target, draft, [0], SpecSamplingConfig(draft_k=3, max_new_tokens=12, seed=6)).tokens
    e = speculative_sample(target, draft, [0], SpecSamplingConfig(draft_k=3, max_new_tokens=50, seed=5, eos_token_ids=[a[3]])).tokens
    assert e == a[:a.index(a[3]) + 1]
    with pytest.raises(ValueError):
        speculative_sample(target, draft, [0], SpecSamplingConfig(draft_k=0))
    with pytest.raises(ValueError):
        speculative_sample(target, FunctionHandle(lambda ids: torch.zeros(5), 5), [0])
    p, q = torch.tensor([0.5, 0.5, 0.0]), torch.tensor([0.2, 0.7, 0.1])
    assert torch.allclose(residual_distribution(p, q), torch.tensor([1.0, 0.0, 0.0]))
    assert torch.equal(residual_distribution(p, p), p)
    # the default all-positions path (one call per prefix) agrees with a single-pass handle
    class Slow(ModelHandle):
        def forward_ids(self, ids):
            return T[ids[-1]]

        def vocab_size(self):
            return V
    assert torch.equal(Slow().forward_ids_all_positions([0, 3, 2]), T[[0, 3, 2]])
    # a real model behind LlamaHandle: with the model as its own draft every token is accepted and the
    # handle's last-position logits equal the model's
    cfg = LlamaConfig.tiny()
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg).eval()
    h = LlamaHandle(m)
    ids = [5, 9, 2, 7]
    torch.testing.assert_close(h.forward_ids(ids), m(torch.tensor([ids]))[0, -1].double())
    o = speculative_sample(h, h, ids, SpecSamplingConfig(draft_k=3, max_new_tokens=7, seed=11))
    assert o.acceptance_rate() == 1.0 and len(o.tokens) == 7 and h.vocab_size() == cfg.vocab_size
