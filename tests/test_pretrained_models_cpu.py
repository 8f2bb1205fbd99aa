"""Checkpoint-compatible BERT / Whisper encoder / GCN / PPO policy: same numbers as the Hugging Face
implementations on shared random weights, published parameter counts, key names, loaders."""
import math

import pytest
import torch

from ferrotorch_b200.models import pretrained as P
from ferrotorch_b200.models import zoo

tr = pytest.importorskip("transformers")


def test_bert_matches_transformers_and_minilm_preset():
    cfg = P.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                       max_position_embeddings=20)
    hf = tr.BertModel(tr.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                    intermediate_size=64, max_position_embeddings=20)).eval()
    m = P.BertModel(cfg).eval()
    sd = {"bert." + k: v for k, v in hf.state_dict().items()}          # a task model's prefix
    sd["bert.embeddings.position_ids"] = torch.arange(20)[None]
    sd["cls.predictions.bias"] = torch.zeros(100)
    rep = m.load_hf_state_dict(sd)
    assert rep.missing == [] and sorted(rep.dropped) == ["cls.predictions.bias", "embeddings.position_ids"]
    ids = torch.randint(0, 100, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.long)
    mask[1, 6:] = 0
    tt = torch.zeros_like(ids)
    tt[:, 5:] = 1
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask, token_type_ids=tt)
        h, pooled = m(ids, mask, tt)
    assert torch.allclose(h[mask.bool()], want.last_hidden_state[mask.bool()], atol=1e-5)
    assert torch.allclose(pooled, want.pooler_output, atol=1e-5)
    st = P.SentenceTransformer(cfg).eval()
    st.load_hf_state_dict(hf.state_dict())
    e = st.encode(ids, mask)
    with torch.no_grad():
        plain = hf(input_ids=ids, attention_mask=mask).last_hidden_state      # token types all zero
    ref = (plain * mask[..., None]).sum(1) / mask.sum(1, keepdim=True)
    assert torch.allclose(e, torch.nn.functional.normalize(ref, dim=-1), atol=1e-5)
    assert torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-6)
    ids2 = ids.clone()
    ids2[1, 6:] = 3                                                     # padding content is invisible
    assert torch.allclose(st.encode(ids2, mask)[1], e[1], atol=1e-6)
    with torch.device("meta"):
        assert sum(p.numel() for p in P.BertModel(P.BertConfig.all_minilm_l6_v2()).parameters()) == 22_713_216
    c = P.BertConfig.from_hf({"vocab_size": 30522, "hidden_size": 384, "num_hidden_layers": 6, "num_attention_heads": 12,
                              "intermediate_size": 1536, "model_type": "bert"})
    assert c == P.BertConfig.all_minilm_l6_v2() and c.head_dim() == 32
    with pytest.raises(ValueError):
        P.BertConfig.from_hf({"hidden_size": 10})
    with pytest.raises(ValueError):
        P.BertConfig(hidden_size=10, num_attention_heads=3).validate()
    with pytest.raises(KeyError):
        P.BertModel(cfg).load_hf_state_dict({"embeddings.word_embeddings.weight": torch.zeros(100, 32)})
    with pytest.raises(ValueError, match="shape"):
        P.BertModel(cfg).load_hf_state_dict({"embeddings.word_embeddings.weight": torch.zeros(7, 32)}, strict=False)


def test_whisper_encoder_and_front_end_match_transformers():
    hc = tr.WhisperConfig(num_mel_bins=16, d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64,
                          max_source_positions=20, decoder_layers=1, decoder_attention_heads=4, decoder_ffn_dim=64,
                          vocab_size=60, max_target_positions=10, pad_token_id=0, bos_token_id=1, eos_token_id=2,
                          decoder_start_token_id=1)
    hf = tr.WhisperModel(hc).eval()
    m = P.WhisperEncoder(P.WhisperConfig(16, 32, 2, 4, 64, 20)).eval()
    assert torch.allclose(m.embed_positions.weight, hf.encoder.embed_positions.weight, atol=1e-6)   # the sinusoid table
    rep = m.load_hf_state_dict({"model." + k: v for k, v in hf.state_dict().items()})
    assert rep.missing == [] and rep.dropped and all(k.startswith("model.decoder.") for k in rep.dropped)
    mel = torch.randn(2, 16, 40)
    with torch.no_grad():
        assert torch.allclose(m(mel), hf.encoder(mel).last_hidden_state, atol=1e-5)
    with pytest.raises(ValueError):
        m(torch.randn(2, 16, 44))                                       # 22 frames > 20 positions
    with pytest.raises(ValueError):
        m(torch.randn(2, 8, 40))
    with torch.device("meta"):
        tiny = P.WhisperEncoder(P.WhisperConfig.whisper_tiny())
    assert sum(p.numel() for p in tiny.parameters()) == 8_208_384 and P.WhisperConfig.whisper_tiny().encoder_head_dim() == 64
    fe = tr.WhisperFeatureExtractor(feature_size=80)
    t = torch.arange(16000 * 2) / 16000
    audio = 0.3 * torch.sin(2 * math.pi * 440 * t) + 0.05 * torch.randn(t.shape, generator=torch.Generator().manual_seed(0))
    want = torch.from_numpy(fe(audio.numpy(), sampling_rate=16000, return_tensors="np").input_features[0])
    got = P.log_mel_spectrogram(audio)
    assert got.shape == (80, 3000) and torch.allclose(got, want, atol=1e-4)
    assert P.log_mel_spectrogram(audio, pad_to_chunk=False).shape == (80, 200)
    assert P.mel_filterbank(80).shape == (80, 201)


def test_gcn_follows_pyg_normalisation_and_trains():
    torch.manual_seed(0)
    x = torch.randn(5, 3)
    ei = torch.tensor([[0, 1, 1, 2, 3, 4], [1, 0, 2, 1, 4, 3]])
    conv = P.GcnConv(3, 4)
    adj = torch.zeros(5, 5)
    adj[ei[1], ei[0]] = 1
    want = zoo.GcnConv.normalize(adj) @ (x @ conv.lin.weight.t()) + conv.bias       # dense D^-1/2 (A + I) D^-1/2
    assert torch.allclose(conv(x, ei), want, atol=1e-6)
    assert torch.allclose(conv(x, ei.flatten().tolist()), want, atol=1e-6)           # a flat [2 * E] list works too
    iso = P.GcnConv(3, 4)                                                             # an isolated node keeps its own features
    assert torch.allclose(iso(x, torch.zeros(2, 0, dtype=torch.long)), x @ iso.lin.weight.t() + iso.bias, atol=1e-6)
    net = P.GcnNet(3, 8, 2, dropout=0.0)
    assert sorted(net.state_dict()) == ["conv1.bias", "conv1.lin.weight", "conv2.bias", "conv2.lin.weight"]
    assert (net.in_features(), net.hidden(), net.num_classes()) == (3, 8, 2)
    y = torch.tensor([0, 0, 0, 1, 1])
    opt = torch.optim.Adam(net.parameters(), lr=0.05)
    for _ in range(80):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(net(x, ei), y).backward()
        opt.step()
    assert (net.eval()(x, ei).argmax(-1) == y).all()
    other = P.GcnNet(3, 8, 2)
    assert other.load_hf_state_dict(net.state_dict()).missing == []
    assert torch.allclose(other.eval()(x, ei), net(x, ei))
    g = P.Graph(x, ei.flatten().tolist(), y)
    assert (g.num_nodes(), g.num_features(), g.num_edges(), g.edge_src(2), g.edge_dst(2)) == (5, 3, 6, 1, 2)
    with pytest.raises(ValueError):
        P.Graph(x, [[0], [9]])
    with pytest.raises(ValueError):
        conv(x, torch.tensor([[0], [5]]))


def test_sb3_policy_layout():
    torch.manual_seed(0)
    p = P.MlpPolicy(P.MlpPolicyConfig.cartpole_v1())
    keys = sorted(p.state_dict())
    assert len(keys) == 12 and "mlp_extractor.policy_net.2.weight" in keys and "mlp_extractor.value_net.0.bias" in keys
    assert p.state_dict()["action_net.weight"].shape == (2, 64) and p.state_dict()["value_net.weight"].shape == (1, 64)
    obs = torch.randn(3, 4)
    out = p(obs)
    assert out.action_logits.shape == (3, 2) and out.value.shape == (3,)
    want = p.action_net(torch.tanh(p.mlp_extractor.policy_net[2](torch.tanh(p.mlp_extractor.policy_net[0](obs)))))
    assert torch.allclose(out.action_logits, want)
    assert torch.equal(p.act(obs), out.action_logits.argmax(-1)) and p(obs[0]).value.shape == (1,)
    sd = {"policy." + k: v for k, v in p.state_dict().items()}
    sd["log_std"] = torch.zeros(2)
    q = P.MlpPolicy()
    rep = q.load_hf_state_dict(sd)
    assert rep.dropped == ["log_std"] and rep.missing == [] and torch.allclose(q(obs).value, out.value)
    assert (p.mlp_extractor.obs_dim(), p.mlp_extractor.hidden(), p.config().n_actions) == (4, 64, 2)
    with pytest.raises(ValueError):
        p(torch.randn(3, 5))


def test_loaders_read_model_directories_and_files(tmp_path):
    from ferrotorch_b200.serialize.state import save_pytorch, save_safetensors

    hf = tr.BertModel(tr.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                    intermediate_size=64, max_position_embeddings=20)).eval()
    hf.save_pretrained(str(tmp_path / "bert"), safe_serialization=True)
    model, rep = P.load_bert_model(str(tmp_path / "bert"))
    assert rep.missing == [] and model.config.hidden_size == 32
    ids = torch.randint(0, 100, (2, 7))
    with torch.no_grad():
        assert torch.allclose(model(ids)[0], hf(input_ids=ids).last_hidden_state, atol=1e-5)
    st, rep = P.load_sentence_transformer(str(tmp_path / "bert" / "model.safetensors"))       # file + neighbouring config
    assert rep.missing == [] and torch.allclose(st.encode(ids).norm(dim=-1), torch.ones(2), atol=1e-6)
    hc = tr.WhisperConfig(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64,
                          max_source_positions=20, decoder_layers=1, decoder_attention_heads=4, decoder_ffn_dim=64,
                          vocab_size=60, max_target_positions=10, pad_token_id=0, bos_token_id=1, eos_token_id=2,
                          decoder_start_token_id=1)
    wm = tr.WhisperModel(hc).eval()
    wm.save_pretrained(str(tmp_path / "whisper"), safe_serialization=True)
    enc, rep = P.load_whisper_encoder(str(tmp_path / "whisper"))
    mel = torch.randn(1, 16, 40)          # the HF encoder insists on exactly 2 * max_source_positions frames
    with torch.no_grad():
        assert rep.missing == [] and torch.allclose(enc(mel), wm.encoder(mel).last_hidden_state, atol=1e-5)
    g = P.GcnNet(7, 5, 3)
    save_safetensors(g.state_dict(), str(tmp_path / "gcn.safetensors"))
    g2, rep = P.load_gcn_net(str(tmp_path / "gcn.safetensors"))
    assert (g2.in_features(), g2.hidden(), g2.num_classes()) == (7, 5, 3) and rep.missing == []
    pol = P.MlpPolicy(P.MlpPolicyConfig(6, 16, 3))
    sd = {"policy." + k: v for k, v in pol.state_dict().items()}
    sd["policy.log_std"] = torch.zeros(3)
    save_pytorch(sd, str(tmp_path / "policy.pth"))
    p2, rep = P.load_ppo_policy(str(tmp_path / "policy.pth"))
    obs = torch.randn(2, 6)
    assert p2.config() == P.MlpPolicyConfig(6, 16, 3) and rep.dropped == ["log_std"] and torch.equal(p2(obs).value, pol.eval()(obs).value)
    with pytest.raises(FileNotFoundError):
        (tmp_path / "none").mkdir()
        P.load_bert_model(str(tmp_path / "none"))


def test_reference_names_of_small_models():
    from ferrotorch_b200.models import pretrained as P
    from ferrotorch_b200.utils import text

    assert P.N_FRAMES == 3000 and P.N_MELS == 80 and P.HfBertConfig is P.BertConfig and text.Tokenizer.__name__ == "Tokenizer"
    cfg = P.BertConfig(vocab_size=50, hidden_size=16, num_hidden_layers=1, num_attention_heads=2, intermediate_size=32,
                       max_position_embeddings=16)
    m = P.BertModel(cfg).eval()
    ids = torch.randint(0, 50, (2, 6))
    out = P.BertOutput.of(m, ids)
    assert out.last_hidden_state.shape == (2, 6, 16) and out.pooler_output.shape == (2, 16)
    wc = P.WhisperConfig(num_mel_bins=8, d_model=16, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=32,
                         max_source_positions=10)
    enc = P.WhisperEncoder(wc).eval()
    stem = P.WhisperConvStem(enc)
    mel = torch.randn(1, 8, 20)
    assert stem(mel).shape == (1, 10, 16) and isinstance(enc.layers[0].self_attn, P.WhisperEncoderSelfAttention)
    assert P.ValueHead(8).out_features == 1 and P.ActionNet(8, 3).out_features == 3
