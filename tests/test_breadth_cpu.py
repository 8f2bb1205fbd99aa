"""CPU tests: sharded checkpoints with resharding, async collectives, RPC, the small model zoo,
tokenizer / hub / grammar helpers, ML metrics and the distributions re-export."""
import json
import os

import pytest
import torch

from ferrotorch_b200.models import zoo
from ferrotorch_b200.parallel import dist_checkpoint as dc
from ferrotorch_b200.parallel.backend import SizeMismatch, run_simulated
from ferrotorch_b200.utils import ml, text


# --------------------------------------------------------------------------- distributed checkpoint
def _full_state():
    g = torch.Generator().manual_seed(3)
    return {"w": torch.randn(8, 6, generator=g), "b": torch.randn(6, generator=g), "col": torch.randn(4, 8, generator=g)}


DIMS = {"w": 0, "b": None, "col": 1}


def _save(tmp, world):
    full = _full_state()
    for r in range(world):
        local = {k: (v if DIMS[k] is None else v.chunk(world, dim=DIMS[k])[r].contiguous()) for k, v in full.items()}
        dc.save_distributed(str(tmp), local, DIMS, rank=r, world_size=world, extra={"step": 7})
    return full


def test_dist_checkpoint_same_world(tmp_path):
    full = _save(tmp_path, 2)
    for r in range(2):
        st, extra = dc.load_distributed(str(tmp_path), r, 2)
        assert extra == {"step": 7}
        assert torch.equal(st["w"], full["w"].chunk(2, 0)[r])
        assert torch.equal(st["col"], full["col"].chunk(2, 1)[r])
        assert torch.equal(st["b"], full["b"])


@pytest.mark.parametrize("new_world", [1, 4])
def test_dist_checkpoint_reshard(tmp_path, new_world):
    full = _save(tmp_path, 2)
    for r in range(new_world):
        st, _ = dc.load_distributed(str(tmp_path), r, new_world)
        assert torch.equal(st["w"], full["w"].chunk(new_world, 0)[r])
        assert torch.equal(st["col"], full["col"].chunk(new_world, 1)[r])
        assert torch.equal(st["b"], full["b"])


def test_dist_checkpoint_reshard_indivisible(tmp_path):
    _save(tmp_path, 2)
    with pytest.raises(SizeMismatch):
        dc.load_distributed(str(tmp_path), 0, 3)


def test_dist_checkpoint_uneven_world_changes_twice(tmp_path):
    # 4 ranks -> reload uneven on 3 -> save again from the uneven shards -> reload on 2: the second
    # save must record the real shard sizes, not rank 0's size times the world
    full = _save(tmp_path / "a", 4)
    three = [dc.load_distributed(str(tmp_path / "a"), r, 3, uneven=True)[0] for r in range(3)]
    assert [t["w"].shape[0] for t in three] == [3, 3, 2]
    for r in range(3):   # no group: every rank writes its own sizes beside its shard
        dc.save_distributed(str(tmp_path / "b"), three[r], DIMS, rank=r, world_size=3)
    for r in range(2):
        st, _ = dc.load_distributed(str(tmp_path / "b"), r, 2)
        assert torch.equal(st["w"], full["w"].chunk(2, 0)[r])
        assert torch.equal(st["col"], full["col"].chunk(2, 1)[r])
    # with the sizes known at save time the metadata itself carries them

    def body(g):
        dc.save_distributed(str(tmp_path / "c"), three[g.rank], DIMS, group=g)
        return True

    assert all(run_simulated(3, body))
    meta = json.load(open(tmp_path / "c" / "metadata.json"))
    assert meta["tensors"]["w"]["shard_sizes"] == [3, 3, 2] and meta["tensors"]["w"]["global_shape"] == [8, 6]
    assert meta["tensors"]["col"]["shard_sizes"] == [3, 3, 2]
    st, _ = dc.load_distributed(str(tmp_path / "c"), 1, 2)
    assert torch.equal(st["w"], full["w"].chunk(2, 0)[1])


def test_async_dist_checkpointer(tmp_path):
    full = _full_state()
    ck = dc.AsyncDistributedCheckpointer()
    local = dict(full)
    ck.save_async(str(tmp_path), local, {k: None for k in full}, 0, 1)
    local["w"].zero_()          # the snapshot was taken before the writer started
    ck.wait()
    assert ck.is_done()
    st, _ = dc.load_distributed(str(tmp_path), 0, 1)
    assert torch.equal(st["w"], _full_state()["w"])


def test_async_checkpointer_reports_errors(tmp_path):
    blocker = tmp_path / "file"
    blocker.write_text("x")
    ck = dc.AsyncDistributedCheckpointer()
    ck.save_async(str(blocker), {"a": torch.zeros(1)}, {"a": None}, 0, 1)
    with pytest.raises(OSError):
        ck.wait()


def test_pending_collective():
    p = dc.PendingCollective(lambda a, b: a + b, 2, 3)
    assert p.wait(5) == 5 and p.is_done()
    bad = dc.PendingCollective(lambda: 1 / 0)
    with pytest.raises(ZeroDivisionError):
        bad.wait(5)


def test_async_collectives_simulated():
    from ferrotorch_b200.parallel.backend import run_simulated

    def body(g):
        # one collective in flight per group at a time: their order across ranks must match
        red = dc.all_reduce_async(g, torch.full((4,), float(g.rank + 1))).wait(10)
        return red, dc.all_gather_async(g, torch.tensor([float(g.rank)])).wait(10)

    for red, gathered in run_simulated(3, body):
        assert torch.equal(red, torch.full((4,), 6.0))
        got = torch.cat(list(gathered)) if isinstance(gathered, (list, tuple)) else gathered.flatten()
        assert got.tolist() == [0.0, 1.0, 2.0]


def test_rpc_agent():
    a = dc.RpcAgent("worker0")
    try:
        a.register("add", lambda x, y=0: x + y)
        a.register("tensor", lambda t: t * 2)
        assert dc.RpcAgent.rpc_sync(a.address, "add", 2, y=5) == 7
        assert torch.equal(dc.RpcAgent.rpc_sync(a.address, "tensor", torch.ones(3)), torch.full((3,), 2.0))
        assert dc.RpcAgent.rpc_async(a.address, "add", 1, y=1).wait(10) == 2
        with pytest.raises(RuntimeError, match="no handler"):
            dc.RpcAgent.rpc_sync(a.address, "missing")
        a.register("boom", lambda: 1 / 0)
        with pytest.raises(RuntimeError, match="ZeroDivisionError"):
            dc.RpcAgent.rpc_sync(a.address, "boom")
        a.register("echo", lambda *xs, **kw: [list(xs), kw])
        nested = {"k": (1, 2.5, None, "s", b"\x00\xff"), "t": torch.arange(6, dtype=torch.int32).view(2, 3)}
        got = dc.RpcAgent.rpc_sync(a.address, "echo", nested, flag=True)
        assert got[1] == {"flag": True} and got[0][0]["k"] == nested["k"]
        assert torch.equal(got[0][0]["t"], nested["t"])
        # the wire carries data only: an object is refused on the sending side, and bytes that
        # are not a well-formed payload are an error reply, never executed
        with pytest.raises(TypeError):
            dc.RpcAgent.rpc_sync(a.address, "echo", object())
        import pickle
        import socket
        import struct
        evil = pickle.dumps((print, ("pwned",)))
        with socket.create_connection(a.address, timeout=10) as sk:
            sk.sendall(struct.pack("<QI", 9, 4) + b"echo" + struct.pack("<Q", len(evil)) + evil)
            req_id, ok, body = dc._recv_response(sk)
        assert req_id == 9 and not ok
    finally:
        a.shutdown()


# --------------------------------------------------------------------------- model zoo
def test_bert_and_sentence_embeddings():
    torch.manual_seed(0)
    bert = zoo.BertModel(vocab_size=100, hidden=32, layers=2, heads=4, intermediate=64, max_pos=16).eval()
    ids = torch.randint(0, 100, (2, 10))
    mask = torch.ones(2, 10, dtype=torch.long)
    mask[1, 6:] = 0
    h, pooled = bert(ids, mask)
    assert h.shape == (2, 10, 32) and pooled.shape == (2, 32)
    emb = zoo.SentenceTransformer(bert)(ids, mask)
    assert torch.allclose(emb.norm(dim=-1), torch.ones(2), atol=1e-5)
    ids2 = ids.clone()
    ids2[1, 6:] = 5          # padding content must not change the embedding
    assert torch.allclose(zoo.SentenceTransformer(bert)(ids2, mask)[1], emb[1], atol=1e-5)


def test_whisper_front_end_and_encoder():
    audio = torch.sin(torch.arange(16000) * 2 * torch.pi * 440 / 16000)[None]
    mel = zoo.log_mel_spectrogram(audio)
    assert mel.shape == (1, 80, 100)
    assert float(mel.max() - mel.min()) <= 2.0 + 1e-5       # 8 dB-decades clamp, divided by 4
    enc = zoo.WhisperEncoder(d_model=64, heads=4, layers=1, n_ctx=64).eval()
    assert enc(mel).shape == (1, 50, 64)


def test_gcn_normalisation_and_training_step():
    adj = torch.tensor([[0, 1, 0], [1, 0, 1], [0, 1, 0]], dtype=torch.float32)
    an = zoo.GcnConv.normalize(adj)
    assert torch.allclose(an, an.T)
    assert torch.allclose(an[0, 0], torch.tensor(0.5))
    assert torch.allclose(zoo.GcnConv.normalize(adj.to_sparse()), an)
    net = zoo.Gcn(5, 8, 2, dropout=0.0)
    x, y = torch.randn(3, 5), torch.tensor([0, 1, 0])
    opt = torch.optim.Adam(net.parameters(), 0.05)
    first = None
    for _ in range(30):
        loss = torch.nn.functional.cross_entropy(net(x, an), y)
        first = first or float(loss)
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert float(loss) < first


@pytest.mark.parametrize("discrete", [False, True])
def test_mlp_policy_and_ppo_loss(discrete):
    torch.manual_seed(0)
    pol = zoo.MlpPolicy(4, 3, discrete=discrete)
    obs = torch.randn(16, 4)
    act, val, logp = pol(obs)
    assert val.shape == (16,) and logp.shape == (16,)
    assert act.shape == ((16,) if discrete else (16, 3))
    det1, _, _ = pol(obs, deterministic=True)
    det2, _, _ = pol(obs, deterministic=True)
    assert torch.equal(det1, det2)
    loss = zoo.ppo_loss(pol, obs, act, logp.detach(), torch.randn(16), torch.randn(16), ent_coef=0.01)
    loss.backward()
    assert all(p.grad is not None for p in pol.actor.parameters())


def test_ddim_scheduler_and_unet():
    torch.manual_seed(0)
    sch = zoo.DDIMScheduler()
    x0, noise = torch.randn(2, 4, 8, 8), torch.randn(2, 4, 8, 8)
    sch.set_timesteps(10)
    t = int(sch.timesteps[0])
    xt = sch.add_noise(x0, noise, torch.tensor([t, t]))
    # with the true noise, stepping from the last-but-zero timestep chain recovers x0 at t=0
    x = xt
    for step_t in sch.timesteps.tolist():
        a = sch.alphas_cumprod[step_t]
        eps = (x - a.sqrt() * x0) / (1 - a).sqrt()
        x = sch.step(eps, step_t, x)
    assert torch.allclose(x, x0, atol=1e-4)
    unet = zoo.TinyUNet(channels=4, base=16, ctx_dim=12).eval()
    out = unet(xt, torch.tensor([t, t]), torch.randn(2, 5, 12))
    assert out.shape == xt.shape
    img = zoo.ddim_sample(zoo.TinyUNet(channels=4, base=16).eval(), sch, (1, 4, 8, 8), steps=3,
                          generator=torch.Generator().manual_seed(1))
    assert img.shape == (1, 4, 8, 8) and torch.isfinite(img).all()


# --------------------------------------------------------------------------- text utilities
def test_json_grammar_prefixes():
    g = text.JsonGrammar()
    for s in ["", "{", '{"a', '{"a":', '{"a": 1,', "[1,", "tr", "-", "-1.5e", '"abc', '{"a": {"b": null}}', "[[],[]]"]:
        assert g.accepts_prefix(s), s
    for s in ["}", "{1", '{"a" 1', "[,", '{"a":}', "01", "[1 2]", '{"a":1,}', "[]]", "1 2"]:
        assert not g.accepts_prefix(s), s
    assert g.is_complete('{"a": [1, 2]}') and not g.is_complete('{"a": [1, 2]')


def test_token_mask_drives_valid_json():
    g = text.JsonGrammar()
    vocab = ["{", "}", '"k"', ":", "1", ",", "[", "]", "x", "<eos>"]
    eos = 9
    m = text.token_mask(g, "", vocab, eos)
    assert m.tolist() == [True, False, True, False, True, False, True, False, False, False]
    m = text.token_mask(g, '{"k"', vocab, eos)
    assert [vocab[i] for i in m.nonzero().flatten().tolist()] == [":"]
    m = text.token_mask(g, '{"k":1}', vocab, eos)
    assert m.nonzero().flatten().tolist() == [eos]
    # greedy decode with adversarial logits still ends as valid JSON
    torch.manual_seed(0)
    out = ""
    for _ in range(40):
        logits = torch.randn(len(vocab))
        logits[eos] += 1.0
        tok = int(text.apply_token_mask(logits, text.token_mask(g, out, vocab, eos)).argmax())
        if tok == eos:
            break
        out += vocab[tok]
    if g.is_complete(out):
        json.loads(out)
    else:
        assert g.accepts_prefix(out)


def test_chat_templates():
    msgs = [{"role": "system", "content": "s"}, {"role": "user", "content": "hi"}]
    t = text.apply_chat_template(msgs)
    assert t.startswith("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\ns<|eot_id|>")
    assert t.endswith("<|start_header_id|>assistant<|end_header_id|>\n\n")
    c = text.apply_chat_template(msgs, "chatml", add_generation_prompt=False)
    assert c == "<|im_start|>system\ns<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n"
    assert text.apply_chat_template(msgs, "{{ messages | length }} turns") == "2 turns"    # any other string is a Jinja template


def test_tokenizer_round_trip(tmp_path):
    tokenizers = pytest.importorskip("tokenizers")
    from tokenizers import models, pre_tokenizers

    tok = tokenizers.Tokenizer(models.WordLevel({"hello": 0, "world": 1, "[UNK]": 2}, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    p = tmp_path / "tokenizer.json"
    tok.save(str(p))
    t = text.load_tokenizer(str(p))
    ids = text.encode(t, "hello world foo")
    assert ids == [0, 1, 2]
    assert text.decode(t, ids[:2]) == "hello world"


def test_hub_offline(tmp_path, monkeypatch):
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    with pytest.raises(FileNotFoundError):
        text.hf_download_model("org/model")
    snap = tmp_path / "hub" / "models--org--model" / "snapshots" / "abc"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text(json.dumps({
        "model_type": "llama", "vocab_size": 1000, "hidden_size": 64, "intermediate_size": 128,
        "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5,
        "rope_theta": 10000.0, "max_position_embeddings": 256}))
    d = text.hf_download_model("org/model")
    assert d == str(snap)
    cfg = text.HfTransformerConfig.from_file(os.path.join(d, "config.json"))
    assert cfg.model_type == "llama"
    lc = cfg.to_llama()
    assert lc.hidden_size == 64 and lc.num_key_value_heads == 2


# --------------------------------------------------------------------------- metrics / distributions
def test_ml_metrics():
    yt = torch.tensor([0, 1, 2, 2, 1, 0])
    yp = torch.tensor([0, 2, 2, 2, 1, 1])
    cm = ml.confusion_matrix(yt, yp)
    assert cm.tolist() == [[1, 1, 0], [0, 1, 1], [0, 0, 2]]
    assert ml.accuracy_score(yt, yp) == pytest.approx(4 / 6)
    p, r, f = ml.precision_recall_f1(yt, yp, "micro")
    assert p == pytest.approx(4 / 6) and r == pytest.approx(4 / 6) and f == pytest.approx(4 / 6)
    p, r, f = ml.precision_recall_f1(yt, yp, "macro")
    assert p == pytest.approx((1 + 0.5 + 2 / 3) / 3) and r == pytest.approx((0.5 + 0.5 + 1) / 3)
    a, b = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, 2.0, 5.0])
    assert ml.mean_squared_error(a, b) == pytest.approx(4 / 3)
    assert ml.mean_absolute_error(a, b) == pytest.approx(2 / 3)
    assert ml.r2_score(a, a) == pytest.approx(1.0)
    assert ml.roc_auc_score(torch.tensor([0, 0, 1, 1]), torch.tensor([0.1, 0.4, 0.35, 0.8])) == pytest.approx(0.75)
    assert ml.roc_auc_score(torch.tensor([0, 1]), torch.tensor([0.5, 0.5])) == pytest.approx(0.5)
    xtr, xte, ytr, yte = ml.train_test_split(torch.arange(20), torch.arange(20) * 2, test_size=0.25)
    assert len(xtr) == 15 and len(xte) == 5 and torch.equal(ytr, xtr * 2)
    assert sorted(torch.cat([xtr, xte]).tolist()) == list(range(20))


def test_distributions_reexport():
    from ferrotorch_b200 import distributions as D

    n = D.Normal(torch.zeros(3), torch.ones(3))
    assert D.kl_divergence(n, n).abs().max() == 0
    assert D.constraints.positive.check(torch.tensor(1.0))
    t = D.TransformedDistribution(n, [D.transforms.ExpTransform()])
    assert (t.sample() > 0).all()


def test_dist_checkpoint_uneven_reshard_and_reference_layout(tmp_path):
    """The reference's directory layout (rank_{r}.safetensors, num_ranks / tensor_specs) loads, and
    a world size that does not divide a dimension gives the first ranks one row more
    (ferrotorch-distributed/src/checkpoint.rs: compute_shard_sizes)."""
    assert dc.shard_sizes(8, 3) == [3, 3, 2] and dc.shard_sizes(2, 4) == [1, 1, 0, 0]
    full = _save(tmp_path / "ours", 2)
    got = [dc.load_distributed(str(tmp_path / "ours"), r, 3, uneven=True)[0]["w"] for r in range(3)]
    assert [g.shape[0] for g in got] == [3, 3, 2] and torch.equal(torch.cat(got), full["w"])
    # the reference's layout, written with uneven shards 5 + 3
    w = full["w"]
    ref = tmp_path / "ref"
    parts = [w[:5].contiguous(), w[5:].contiguous()]
    for r in range(2):
        dc.save_reference_distributed(str(ref), {"w": parts[r]}, {"w": 0}, {"w": [5, 3]}, r, 2)
    import json
    meta = json.loads((ref / "metadata.json").read_text())
    assert meta == {"num_ranks": 2, "tensor_specs": {"w": {"full_shape": [8, 6], "shard_dim": 0, "shard_sizes": [5, 3]}}}
    assert torch.equal(dc.load_distributed(str(ref), 1, 2)[0]["w"], parts[1])
    got = [dc.load_distributed(str(ref), r, 3)[0]["w"] for r in range(3)]
    assert torch.equal(torch.cat(got), w) and [g.shape[0] for g in got] == [3, 3, 2]
    (ref / "rank_1.safetensors").unlink()
    with pytest.raises(FileNotFoundError):
        dc.load_distributed(str(ref), 0, 4)
    with pytest.raises(ValueError):
        dc.load_distributed(str(ref), 4, 4)


def test_ml_bridge_covers_the_reference_surface():
    """Every public function of ferrotorch-ml (metrics.rs, datasets.rs, adapter.rs) exists here and
    a few agree with values worked out by hand."""
    names = """accuracy_score adjusted_mutual_info_score adjusted_rand_score array1_to_tensor array1_usize_to_tensor
    array2_to_tensor average_precision_score balanced_accuracy_score brier_score_loss calinski_harabasz_score
    cohen_kappa_score completeness_score confusion_matrix coverage_error d2_brier_score davies_bouldin_score dcg_score
    explained_variance_score f1_score fowlkes_mallows_score hamming_loss homogeneity_score
    label_ranking_average_precision_score label_ranking_loss load_breast_cancer load_iris load_wine log_loss make_blobs
    make_circles make_classification make_moons make_regression matthews_corrcoef max_error mean_absolute_error
    mean_absolute_percentage_error mean_squared_error median_absolute_error ndcg_score normalized_mutual_info_score
    precision_score r2_score recall_score roc_auc_score root_mean_squared_error silhouette_score tensor_to_array1
    tensor_to_array1_usize tensor_to_array2 top_k_accuracy_score v_measure_score zero_one_loss""".split()
    assert all(callable(getattr(ml, n)) for n in names)
    yt, yp = torch.tensor([0, 1, 2, 2, 1, 0]), torch.tensor([0, 2, 2, 2, 1, 1])
    assert ml.zero_one_loss(yt, yp) == pytest.approx(2 / 6) and ml.hamming_loss(yt, yp) == pytest.approx(2 / 6)
    assert ml.f1_score(yt, yp, average="macro") == pytest.approx(ml.precision_recall_f1(yt, yp)[2])
    assert ml.balanced_accuracy_score(yt, yp) == pytest.approx((0.5 + 0.5 + 1.0) / 3)
    a, b = torch.tensor([1.0, 2.0, 3.0]), torch.tensor([1.0, 2.0, 5.0])
    assert ml.max_error(a, b) == 2.0 and ml.root_mean_squared_error(a, b) == pytest.approx((4 / 3) ** 0.5)
    assert ml.median_absolute_error(a, b) == 0.0 and ml.mean_absolute_percentage_error(a, b) == pytest.approx(2 / 9)
    assert ml.adjusted_rand_score(yt, yt) == 1.0 and ml.v_measure_score(yt, yt) == pytest.approx(1.0)
    y, pr = torch.tensor([0, 1, 1, 0]), torch.tensor([0.1, 0.9, 0.8, 0.3])
    assert ml.brier_score_loss(y, pr) == pytest.approx(0.0375) and ml.d2_brier_score(y, pr) == pytest.approx(0.85)
    assert ml.average_precision_score(y, pr) == 1.0
    with pytest.raises(ValueError):
        ml.f1_score(torch.tensor([0.5, 1.0]), torch.tensor([0, 1]))          # labels must be integral
    with pytest.raises(ValueError):
        ml.tensor_to_array2(torch.zeros(3))
    x, t = ml.load_iris()
    assert x.shape == (150, 4) and t.unique().tolist() == [0.0, 1.0, 2.0] and ml.silhouette_score(x, t) > 0.4
    assert ml.load_wine()[0].shape == (178, 13) and ml.load_breast_cancer()[0].shape == (569, 30)
    X, Y = ml.make_moons(40, noise=0.1, seed=0)
    X2, _ = ml.make_moons(40, noise=0.1, seed=0)
    assert X.shape == (40, 2) and torch.equal(X, X2) and Y.unique().tolist() == [0.0, 1.0]
    assert ml.make_regression(20, 5, 3, seed=1)[0].shape == (20, 5) and ml.make_classification(30, 8, seed=1)[1].shape == (30,)
    assert ml.make_blobs(30, centers=4, seed=2)[1].unique().numel() == 4 and ml.make_circles(10, seed=0)[0].shape == (10, 2)


def test_lora_se_and_hooked_module():
    import ferrotorch_b200.nn as fnn

    torch.manual_seed(0)
    base = torch.nn.Linear(6, 4)
    lora = fnn.LoRALinear(base, rank=2, alpha=4.0)
    x = torch.randn(3, 6)
    assert torch.equal(lora(x), base(x))                               # B starts at zero
    assert not base.weight.requires_grad and lora.lora_a.shape == (2, 6) and lora.lora_b.shape == (4, 2)
    assert (lora.rank(), lora.alpha(), lora.base()) == (2, 4.0, base)
    with torch.no_grad():
        lora.lora_b.normal_()
    want = lora(x)
    assert torch.allclose(want, base(x) + 2.0 * x @ lora.lora_a.t() @ lora.lora_b.t(), atol=1e-6)
    want.sum().backward()
    assert lora.lora_a.grad is not None and base.weight.grad is None
    lora.merge()
    assert torch.allclose(lora.into_base()(x), want, atol=1e-5) and float(lora.lora_b.abs().sum()) == 0.0
    with pytest.raises(ValueError):
        fnn.LoRALinear(base, 0)
    se = fnn.SqueezeExcitation(8, 2)
    img = torch.randn(2, 8, 5, 5)
    gate = torch.sigmoid(se.fc2(torch.relu(se.fc1(img.mean((2, 3), keepdim=True)))))
    assert torch.allclose(se(img), img * gate, atol=1e-6) and sorted(se.state_dict()) == ["fc1.bias", "fc1.weight", "fc2.bias", "fc2.weight"]
    with pytest.raises(ValueError):
        fnn.SqueezeExcitation(0, 2)
    hm = fnn.HookedModule(torch.nn.Linear(3, 3))
    seen = []
    h1 = hm.register_forward_pre_hook(lambda i: i * 2)
    h2 = hm.register_forward_hook(lambda i, o: seen.append(o.shape))
    h3 = hm.register_backward_hook(lambda g: g * 0)
    inp = torch.ones(2, 3, requires_grad=True)
    out = hm(inp)
    assert torch.allclose(out, hm.inner()(torch.full((2, 3), 2.0))) and seen == [(2, 3)] and h1.id() != h2.id()
    out.sum().backward()
    assert float(inp.grad.abs().sum()) == 0.0                           # the backward hook replaced the gradient
    for h in (h1, h2, h3):
        h.remove()
    assert torch.allclose(hm(inp), hm.inner()(inp)) and len(seen) == 1
    assert fnn.PagedKVCache is not None and fnn.PagedAttentionManager is not None


@pytest.mark.parametrize("causal,nq,nk,block", [(False, 7, 13, 4), (True, 9, 9, 4), (True, 5, 11, 16), (False, 6, 6, 1)])
def test_tiled_attention_forward_and_backward(causal, nq, nk, block):
    import ferrotorch_b200.nn as fnn

    torch.manual_seed(0)
    q = torch.randn(2, nq, 8, dtype=torch.float64, requires_grad=True)
    k = torch.randn(2, nk, 8, dtype=torch.float64, requires_grad=True)
    v = torch.randn(2, nk, 5, dtype=torch.float64, requires_grad=True)
    want = fnn.standard_attention(q, k, v, causal)
    got = fnn.flash_attention(q, k, v, causal, block)
    assert torch.allclose(got, want, atol=1e-6)
    w = torch.randn_like(want)
    g1 = torch.autograd.grad((want * w).sum(), (q, k, v))
    g2 = torch.autograd.grad((got * w).sum(), (q, k, v))
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b, atol=1e-5), (a - b).abs().max()
    if not causal:
        sdpa = torch.nn.functional.scaled_dot_product_attention(q[:, None], k[:, None], v[:, None])[:, 0]
        assert torch.allclose(got, sdpa, atol=1e-6)
    for bad in ((q[0], k, v), (q, k[:, :, :4], v), (q, k, v[:, :3])):
        with pytest.raises(ValueError):
            fnn.flash_attention(*bad)
    with pytest.raises(ValueError):
        fnn.flash_attention(q, k, v, causal, 0)
    assert fnn.flex_attention is not None


def test_nn_reference_names_and_score_mods():
    import ferrotorch_b200.nn as fnn
    from ferrotorch_b200.core import flex_attention

    q, k, v = torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8), torch.randn(2, 2, 6, 8)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
    torch.testing.assert_close(flex_attention(q, k, v, fnn.causal_score_mod()), ref, rtol=1e-5, atol=1e-5)
    qi, ki = torch.arange(6).view(6, 1), torch.arange(6).view(1, 6)
    slopes = torch.tensor([0.5, 0.25])
    bias = slopes.view(1, 2, 1, 1) * (qi - ki).float()
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=bias)
    torch.testing.assert_close(flex_attention(q, k, v, fnn.alibi_score_mod(slopes)), ref, rtol=1e-5, atol=1e-5)
    table = torch.randn(7)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=table[(qi - ki).clamp(-3, 3) + 3])
    torch.testing.assert_close(flex_attention(q, k, v, fnn.relative_position_bias_score_mod(table, 3)), ref, rtol=1e-5, atol=1e-5)
    x = torch.randn(5, 16)
    heads = fnn.reshape_to_heads(x, 2, 5, 8)
    assert heads.shape == (2, 5, 8) and torch.equal(heads[1, 3], x[3, 8:]) and torch.equal(fnn.transpose_heads_to_2d(heads, 2, 5, 8), x)
    assert fnn.HardSwish is torch.nn.Hardswish and str(fnn.Reduction.Sum) == "sum" and fnn.FanMode.FanOut == "fan_out"
    assert torch.nn.functional.mse_loss(x, x + 1, reduction=fnn.Reduction.Sum).item() == pytest.approx(80.0)
    fnn.RotaryPositionEmbedding(8, 32, scaling=fnn.RoPEScaling.Yarn(4.0, 16))
    fnn.RotaryPositionEmbedding(8, 32, scaling=fnn.RoPEScaling.NtkAware(2.0))
    packed = fnn.pack_padded_sequence(fnn.pad_sequence([torch.ones(3, 2), torch.ones(2, 2)], batch_first=True), [3, 2], batch_first=True)
    assert isinstance(packed, fnn.PackedSequence) and fnn.max_pool2d(torch.randn(1, 1, 4, 4), 2).shape == (1, 1, 2, 2)
    qm = fnn.QatModel(torch.nn.Sequential(torch.nn.Linear(8, 4)), fnn.QatConfig(weight_bits=8))
    qm(torch.randn(2, 8))
    assert list(qm.convert().dequantized_state_dict()) == ["0.weight"]


def test_optim_configs_and_data_reference_names():
    import numpy as np

    import ferrotorch_b200.data as D
    import ferrotorch_b200.optim as O

    w = [torch.nn.Parameter(torch.randn(4, 4))]
    opt = O.AdamWConfig(lr=3e-4).build(w)
    assert isinstance(opt, O.AdamW) and opt.defaults["lr"] == 3e-4 and opt.defaults["weight_decay"] == 0.01
    assert O.AdamWConfig().betas == (0.9, 0.999) and O.AdamWConfig().eps == 1e-8
    sgd = O.SgdConfig()
    assert (sgd.momentum, sgd.dampening, sgd.weight_decay, sgd.nesterov, sgd.maximize) == (0, 0, 0, False, False)
    assert O.RmspropConfig().alpha == 0.99 and O.LbfgsConfig().history_size == 100 and O.Sgd is O.SGD
    assert O.LbfgsConfig(line_search_fn=O.LineSearchFn.StrongWolfe).build(w).defaults["line_search_fn"] == "strong_wolfe"
    for cfg in (O.AdamConfig, O.AdamaxConfig, O.NAdamConfig, O.RAdamConfig, O.AdagradConfig, O.AdadeltaConfig, O.AdafactorConfig,
                O.RpropConfig, O.AsgdConfig, O.MuonConfig, O.KfacConfig):
        o = cfg().build(w)
        w[0].grad = torch.randn(4, 4)
        o.step()
    gs = O.GradScalerConfig()
    assert (gs.init_scale, gs.growth_factor, gs.backoff_factor, gs.growth_interval, gs.enabled) == (65536.0, 2.0, 0.5, 2000, True)
    sch = O.OneCycleLR(opt, 0.1, total_steps=10, anneal_strategy=O.AnnealStrategy.Linear)
    assert isinstance(sch, O.LrScheduler) and O.SequentialLr is O.SequentialLR and O.CyclicMode.ExpRange == "exp_range"

    D.manual_seed(3)
    a = torch.rand(2)
    D.manual_seed(3)
    assert torch.equal(a, torch.rand(2))
    ds = D.MappedDataset(D.VecDataset([1, 2, 3, 4, 5]), lambda v: torch.tensor(float(v)) * 2)
    assert len(ds) == 5 and ds[4].item() == 10.0
    with pytest.raises(IndexError):
        D.VecDataset([1])[3]
    it = D.CollatedIter(D.BatchIter(ds, [0, 1, 2, 3, 4], 2))
    batches = list(D.PrefetchIter(it, 2))
    assert [b.tolist() for b in batches] == [[2.0, 4.0], [6.0, 8.0], [10.0]] and len(D.BatchIter(ds, range(5), 2, drop_last=True)) == 2

    def boom():
        yield 1
        raise RuntimeError("producer failed")

    with pytest.raises(RuntimeError, match="producer failed"):
        list(D.PrefetchIter(boom()))
    img = np.arange(2 * 3 * 3, dtype=np.uint8).reshape(2, 3, 3)          # H, W, C
    t = D.Compose([D.ToTensor(), D.Normalize([0.5, 0.5, 0.5], [0.5, 0.5, 0.5])])(img)
    assert t.shape == (3, 2, 3) and t[0, 0, 0].item() == pytest.approx(-1.0)
    g = torch.Generator().manual_seed(0)
    x = torch.arange(16.0).view(1, 4, 4)
    assert D.RandomCrop(2, generator=g)(x).shape == (1, 2, 2) and D.RandomCrop(4, padding=1, generator=g)(x).shape == (1, 4, 4)
    assert torch.equal(D.RandomHorizontalFlip(1.0)(x), x.flip(-1)) and torch.equal(D.RandomHorizontalFlip(0.0)(x), x)
    moved = D.ToDevice("cpu")({"a": [x, 3], "b": (x,)})
    assert moved["a"][1] == 3 and moved["b"][0] is x
    xs, ys = D.default_collate_pair([(torch.ones(2), 0), (torch.zeros(2), 1)])
    assert xs.shape == (2, 2) and ys.tolist() == [0, 1]
    assert list(D.WorkerInfo(1, 3).shard(10)) == [4, 5, 6] and D.WorkerInfo.current() is None and D.WorkerMode.CrossBatch
    assert len(list(D.MultiWorkerIter(ds, 2, 0))) == 3 and len(D.ConcatDataset([ds, ds])) == 10


def test_gpu_crate_names_without_a_gpu():
    from ferrotorch_b200 import cuda as C
    from ferrotorch_b200.utils import memory_guard as MG

    assert C.capture_status() is C.CaptureStatus.NotCapturing and str(C.CaptureMode.ThreadLocal) == "thread_local"
    assert C.GpuTensor is torch.Tensor and C.MemoryWatchdog is MG.MemoryWatchdog and C.MemoryStats is MG.MemoryStats
    alloc = C.CudaAllocator()
    assert alloc.allocated_bytes() == 0 and alloc.round_len(1000) == 1024 and alloc.round_len(3 << 20) == 4 << 20
    if not torch.cuda.is_available():
        with pytest.raises(C.GpuError):
            C.begin_capture()
        with pytest.raises(C.GpuError):
            C.init_cuda_backend()

    class FakeAlloc:
        used = 100

        def total_bytes(self):
            return 1000

        def used_bytes(self):
            return self.used

        def empty_cache(self):
            pass

    g = MG.MemoryGuard(FakeAlloc(), budget_bytes=1000)
    with MG.MemoryReservation(g, 400) as r:
        assert g.available() == 500 and r.nbytes == 400
        st = MG.MemoryStats.of(g)
        assert (st.used_bytes, st.reserved_bytes, st.available_bytes, st.budget_bytes) == (100, 400, 500, 1000)
    assert g.available() == 900
    with pytest.raises(ValueError):
        MG.MemoryReservation(g, 1000)


def test_bregman_kl_matches_closed_forms():
    import ferrotorch_b200.distributions as D

    pairs = [(D.Normal(torch.tensor([0.0, 1.0]), torch.tensor([1.0, 2.0])), D.Normal(torch.tensor([0.5, 0.0]), torch.tensor([1.5, 1.0]))),
             (D.Gamma(torch.tensor(2.0), torch.tensor(3.0)), D.Gamma(torch.tensor(1.5), torch.tensor(1.0))),
             (D.Bernoulli(torch.tensor([0.2, 0.7])), D.Bernoulli(torch.tensor([0.4, 0.6]))),
             (D.Poisson(torch.tensor(3.0)), D.Poisson(torch.tensor(5.0))),
             (D.Exponential(torch.tensor(2.0)), D.Exponential(torch.tensor(0.5)))]
    for p, q in pairs:
        torch.testing.assert_close(D.kl_expfamily_expfamily(p, q), D.kl_divergence(p, q), rtol=1e-5, atol=1e-6)
    with pytest.raises(NotImplementedError):
        D.kl_expfamily_expfamily(pairs[0][0], pairs[1][0])
    assert D.ExpRelaxedCategorical and D.DistConstraint is D.constraints.Constraint


def test_typed_launcher_names_resolve():
    from ferrotorch_b200 import cuda as C

    a, b = torch.randn(3, 4), torch.randn(3, 4)
    assert torch.equal(C.gpu_add(a, b), a + b) and torch.equal(C.gpu_relu_bf16(a.bfloat16()), a.bfloat16().relu())
    out = torch.empty(3, 4)
    assert C.gpu_mul_into(a, b, out) is out and torch.equal(out, a * b)
    with pytest.raises(C.GpuError):
        C.gpu_relu_bf16(a)                                       # the suffix names the dtype the call expects
    torch.testing.assert_close(C.gpu_matmul_f32_nt(a, b), a @ b.t())
    v, i = C.gpu_topk_f32(a, 2)
    assert torch.equal(v, a.topk(2).values)
    g = torch.arange(6.0)
    assert torch.equal(C.gpu_repeat_interleave_backward_f32(g, 2), torch.tensor([1.0, 5.0, 9.0]))
    x = torch.zeros(2, 3)
    idx = torch.tensor([[0, 1], [1, 2], [0, 1]])
    assert C.gpu_scatter_add_nd_f32(x, idx, torch.ones(3))[0, 1] == 2.0
    assert torch.equal(C.gpu_scatter_add_segments_f32(torch.ones(4, 2), torch.tensor([0, 0, 1, 0]), 2), torch.tensor([[3.0, 3.0], [1.0, 1.0]]))
    s = C.gpu_causal_mask_bf16(torch.zeros(3, 3, dtype=torch.bfloat16))
    assert s[0, 1] == float("-inf") and s[2, 0] == 0
    with pytest.raises(AttributeError):
        C.gpu_no_such_op


def test_launchers_added_for_graph_capture_and_normalisation_gradients():
    from ferrotorch_b200 import cuda as C

    torch.manual_seed(0)
    x = torch.randn(4, 6, 5, 5, dtype=torch.float64, requires_grad=True)
    w = torch.randn(6, dtype=torch.float64, requires_grad=True)
    b = torch.zeros(6, dtype=torch.float64, requires_grad=True)
    rm, rv = torch.randn(6, dtype=torch.float64), torch.rand(6, dtype=torch.float64) + 0.5
    for training in (True, False):
        y = torch.nn.functional.batch_norm(x, rm.clone(), rv.clone(), w, b, training, 0.1, 1e-5)
        g = torch.randn_like(y)
        want = torch.autograd.grad(y, (x, w, b), g)
        got = C.gpu_batch_norm_backward_f64(x.detach(), g, w.detach(), rm, rv, 1e-5, training)
        for a, e in zip(got, want):
            torch.testing.assert_close(a, e)
    for size in (3, 4, 5):
        y = torch.nn.functional.local_response_norm(x, size, 1e-2, 0.75, 2.0)
        g = torch.randn_like(y)
        den = C.gpu_local_response_norm_denominator(x.detach(), size, 1e-2, 0.75, 2.0)
        torch.testing.assert_close(x.detach() * den.pow(-0.75), y.detach())
        torch.testing.assert_close(C.gpu_local_response_norm_backward_f64(x.detach(), g, den, size, 1e-2, 0.75),
                                   torch.autograd.grad(y, x, g)[0])
    # positions and lengths that live in device memory (nothing is read back: usable under graph capture)
    dst, src = torch.zeros(2, 7, 3), torch.randn(2, 3)
    C.gpu_slice_write_indirect(src, dst, torch.tensor([4], dtype=torch.int32))
    assert torch.equal(dst[:, 4], src) and int((dst != 0).sum()) == 6
    m = C.gpu_causal_mask_indirect(torch.tensor([3]), 2, 5)
    assert m.shape == (2, 5) and m[1].tolist() == [0.0, 0.0, 0.0, -1e9, -1e9]
    inp, idx, s2 = torch.zeros(3, 4), torch.tensor([[0, 1, 0, 1], [2, 2, 2, 2]]), torch.arange(8.0).view(2, 4)
    assert torch.equal(C.gpu_scatter_reduce_nd_f32(inp, 0, idx, s2, 2, False), inp.scatter_reduce(0, idx, s2, "amax", include_self=False))
    be = C.CudaBackendImpl(0)
    assert torch.equal(be.relu_f32(torch.tensor([-1.0, 2.0])), torch.tensor([0.0, 2.0])) and "ordinal=0" in repr(be)
    with pytest.raises(AttributeError):
        be.no_such_kernel


def test_cache_and_rope_objects_answer_the_reference_method_names():
    from ferrotorch_b200 import nn as N

    r = N.RotaryPositionEmbedding.with_convention(16, 64, 10000.0, N.RoPEConvention.Interleaved)
    assert (r.dim, r.max_seq_len, r.base, r.convention, r.scaling) == (16, 64, 10000.0, "interleaved", None)
    x = torch.randn(2, 3, 5, 16)
    y = r.apply(x, 7)
    cos, sin = r._tables("cpu")
    c, s = cos[7:12], sin[7:12]
    xe, xo = x[..., 0::2], x[..., 1::2]
    torch.testing.assert_close(y, torch.stack([xe * c - xo * s, xe * s + xo * c], -1).flatten(-2))
    half = N.RotaryPositionEmbedding.with_scaling(16, 64, 10000.0, "half", N.RoPEScaling.Linear(2.0))
    assert half.convention == "half" and half.scaling == {"type": "linear", "factor": 2.0}
    h = half.apply(x, 0)
    ch, sh = half._tables("cpu")
    x1, x2 = x[..., :8], x[..., 8:]
    torch.testing.assert_close(h, torch.cat([x1 * ch[:5] - x2 * sh[:5], x2 * ch[:5] + x1 * sh[:5]], -1))
    for bad in (lambda: N.RotaryPositionEmbedding.with_convention(15, 64), lambda: r.apply(x, 60), lambda: r.apply(torch.randn(1, 2, 8)),
                lambda: N.RotaryPositionEmbedding.with_convention(16, 64, 1e4, "spiral")):
        with pytest.raises(ValueError):
            bad()
    kv = N.KVCache.with_dims(32, 1, 2, 16, dtype=torch.float32)
    assert kv.is_empty() and (kv.max_seq_len(), kv.batch_size(), kv.num_kv_heads(), kv.head_dim()) == (32, 1, 2, 16)
    k1, v1 = torch.randn(1, 2, 3, 16), torch.randn(1, 2, 3, 16)
    k, v = kv.update(k1, v1)
    k2, _ = kv.update(k1 * 2, v1)
    assert torch.equal(k, k1) and torch.equal(k2, torch.cat([k1, k1 * 2], 2)) and kv.seq_len() == 6 and not kv.is_empty()
    with pytest.raises(ValueError):
        kv.update(torch.randn(1, 3, 1, 16), torch.randn(1, 3, 1, 16))
    kv.reset()
    assert kv.is_empty()
    # paged cache: data in and out through the manager
    cache = N.PagedKVCache(2, 2, 8, num_blocks=16, max_seqs=4, max_seq_len=64, block_size=4, device="cpu", dtype=torch.float32)
    m = N.PagedAttentionManager(cache)
    a, b = m.add_sequence(), m.add_sequence()
    ka, va = torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    m.append_kv(a, ka[:5], va[:5])
    m.append_kv(b, torch.ones(3, 2, 8), torch.ones(3, 2, 8))
    m.append_kv(a, ka[5:].reshape(-1), va[5:].reshape(-1))            # flat, as the reference takes it
    m.append_kv(a, ka * 2, va * 2, layer=1)
    assert all(torch.equal(p, q) for p, q in zip(m.get_kv(a), (ka, va))) and torch.equal(m.get_kv(a, 1)[0], ka * 2)
    assert (cache.len(a), cache.len(), cache.num_pages(a), cache.num_pages()) == (6, 9, 2, 3) and cache.is_empty(3)
    assert torch.equal(cache.get_keys(a), ka) and torch.equal(cache.get_values(b), torch.ones(3, 2, 8))
    m.remove_sequence(a)
    assert cache.num_pages() == 1
    with pytest.raises(ValueError):
        m.get_kv(a)
    cache.free_all()
    assert cache.is_empty() and cache.num_pages() == 0
