"""Expectations taken from the reference's own unit tests (read as text) and restated here:
the same inputs must give the same answers in this framework."""
import math

import pytest
import torch

from ferrotorch_b200.ops import reference as R
from ferrotorch_b200.train import tensorboard as TB


def _inv_freq(dim, base, scaling=None):
    """Recover inv_freq from the tables: the angle at position 1 (all angles here are < pi)."""
    cos, sin = R.rope_tables(dim, 4, base, scaling)
    return torch.atan2(sin[1].double(), cos[1].double())


# ferrotorch-train/src/tensorboard.rs:568-593 (RFC 3720 vectors)
def test_crc32c_vectors():
    assert TB.crc32c(b"") == 0x00000000
    assert TB.crc32c(bytes(32)) == 0x8A9136AA
    assert TB.crc32c(bytes([0xFF] * 32)) == 0x62A8AB43
    assert TB.crc32c(bytes(range(32))) == 0x46DD794E
    assert TB.crc32c(b"abc") != TB.masked_crc(b"abc")


# ferrotorch-nn/src/transformer.rs:2165-2216
def test_rope_ntk_and_linear_inv_freq():
    dim, base, factor = 64, 10000.0, 4.0
    plain = _inv_freq(dim, base)
    ntk = _inv_freq(dim, base, {"type": "ntk", "factor": factor, "original_max": 2048})
    assert plain.numel() == 32 and abs(float(ntk[0] - plain[0])) < 1e-6      # highest frequency unchanged
    assert abs(float(ntk[31] / plain[31]) - 1.0 / factor) < 0.05            # lowest ~ linear interpolation
    cos, _ = R.rope_tables(8, 16, base, {"type": "linear", "factor": 2.0})
    cos_plain, _ = R.rope_tables(8, 16, base)
    assert torch.allclose(cos[2::2], cos_plain[1:8], atol=1e-6)              # position p/2


# ferrotorch-nn/src/transformer.rs:2219-2245 and the schedule at :357-392
def test_rope_yarn_inv_freq_piecewise_and_exact_schedule():
    dim, base, factor, orig = 64, 10000.0, 4.0, 2048
    plain = _inv_freq(dim, base)
    yarn = _inv_freq(dim, base, {"type": "yarn", "factor": factor, "original_max": orig})
    assert abs(float(yarn[0] - plain[0])) < 1e-6
    assert abs(float(yarn[31] / (plain[31] / factor)) - 1.0) < 0.1

    def corr(n_rot):
        return dim * math.log(orig / (n_rot * 2 * math.pi)) / (2 * math.log(base))

    low, high = max(math.floor(corr(32.0)), 0.0) / 2.0, min(math.ceil(corr(1.0)), dim - 1) / 2.0
    want = []
    for i in range(dim // 2):
        p = base ** (2.0 * i / dim)
        t = min(max((i - low) / (0.001 if high == low else high - low), 0.0), 1.0)
        want.append((1.0 / (factor * p)) * t + (1.0 / p) * (1.0 - t))
    assert torch.allclose(yarn, torch.tensor(want, dtype=torch.float64), rtol=2e-5, atol=1e-9)
    # no attention temperature in the reference's YaRN: cos(0) stays exactly 1
    cos, _ = R.rope_tables(dim, 4, base, {"type": "yarn", "factor": factor, "original_max": orig})
    assert float(cos[0].max()) == 1.0
    cos_hf, _ = R.rope_tables(dim, 4, base, {"type": "yarn", "factor": factor, "original_max": orig, "mscale": True})
    assert float(cos_hf[0, 0]) == pytest.approx(0.1 * math.log(factor) + 1.0)


# ferrotorch-nn/src/transformer.rs:2068-2080: position zero is the identity for both conventions
@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_position_zero_is_identity(interleaved):
    from ferrotorch_b200.ops import functional as F

    cos, sin = R.rope_tables(8, 16, 10000.0)
    x = torch.randn(1, 1, 2, 8)
    y = F.rope_(x.clone(), cos, sin, n_rot_heads=2, seq_len=1, interleaved=interleaved)
    assert torch.allclose(y, x, atol=1e-7)


# --------------------------------------------------------------------------- GGUF block decoders
# Vectors of ferrotorch-serialize/src/gguf.rs:1150-1250 (the decoder tests) and :1515-1630 (headers
# whose counts lie about the file's size must be rejected quickly, without a huge allocation).
def _f16_bytes(v):
    return list(torch.tensor([v], dtype=torch.float16).view(torch.uint8).tolist())


def _blocks(*rows):
    return torch.tensor([b for r in rows for b in r], dtype=torch.uint8)


def test_q4_0_known_values_both_orders():
    from ferrotorch_b200.serialize import gguf as G
    blk = _f16_bytes(1.0) + [0x88, 0x97, 0xA6] + [0x88] * 13
    raw = _blocks(blk)
    # the order the reference's decoder emits: byte j -> elements 2j, 2j + 1
    y = G.dequantize_blocks(raw, G.GGML_Q4_0, 32, nibble_order="interleaved")
    assert y[:6].tolist() == [0.0, 0.0, -1.0, 1.0, -2.0, 2.0] and y[6:].abs().max() == 0
    assert torch.equal(R.dequant_q4_0(raw.view(1, 18), "interleaved"), y)
    # the file format's order: byte j -> elements j, j + 16
    z = G.dequantize_blocks(raw, G.GGML_Q4_0, 32)
    assert z[:3].tolist() == [0.0, -1.0, -2.0] and z[16:19].tolist() == [0.0, 1.0, 2.0]
    assert torch.equal(R.dequant_q4_0(raw.view(1, 18)), z)
    # re-packing turns one convention's bytes into the other's
    rp = G.repack_nibbles(raw.clone(), G.GGML_Q4_0, to_interleaved=False)
    assert torch.equal(G.dequantize_blocks(rp, G.GGML_Q4_0, 32), y)
    assert torch.equal(G.repack_nibbles(rp.clone(), G.GGML_Q4_0, to_interleaved=True), raw)


def test_q4_0_scale_factor():
    from ferrotorch_b200.serialize import gguf as G
    raw = _blocks(_f16_bytes(0.5) + [0x97] + [0x88] * 15)
    y = G.dequantize_blocks(raw, G.GGML_Q4_0, 32, nibble_order="interleaved")
    assert y[:2].tolist() == [-0.5, 0.5]
    z = G.dequantize_blocks(raw, G.GGML_Q4_0, 32)
    assert z[0].item() == -0.5 and z[16].item() == 0.5


def test_q5_and_q4_1_orders_agree_up_to_permutation():
    from ferrotorch_b200.serialize import gguf as G
    g = torch.Generator().manual_seed(3)
    for t in (G.GGML_Q4_1, G.GGML_Q5_0, G.GGML_Q5_1):
        bb = G._BLOCK[t][1]
        raw = torch.randint(0, 256, (4, bb), generator=g, dtype=torch.uint8)
        raw[:, :2] = torch.tensor(_f16_bytes(0.25), dtype=torch.uint8)
        if t in (G.GGML_Q4_1, G.GGML_Q5_1):
            raw[:, 2:4] = torch.tensor(_f16_bytes(-1.5), dtype=torch.uint8)
        a = G.dequantize_blocks(raw.reshape(-1), t, 128).view(4, 32)
        b = G.dequantize_blocks(raw.reshape(-1), t, 128, nibble_order="interleaved").view(4, 32)
        if t == G.GGML_Q4_1:   # same nibbles, different positions
            assert torch.equal(b[:, 0::2], a[:, :16]) and torch.equal(b[:, 1::2], a[:, 16:])
        else:                  # the fifth bit comes from a different place too: check it by hand
            qh_off = 2 if t == G.GGML_Q5_0 else 4
            q_off = qh_off + 4
            qh = int.from_bytes(bytes(raw[0, qh_off:qh_off + 4].tolist()), "little")
            d, m = 0.25, (-1.5 if t == G.GGML_Q5_1 else 0.0)
            for j in range(16):
                byte = int(raw[0, q_off + j])
                lo = (byte & 15) | (((qh >> (2 * j)) & 1) << 4)
                hi = (byte >> 4) | (((qh >> (2 * j + 1)) & 1) << 4)
                off = 16 if t == G.GGML_Q5_0 else 0
                assert b[0, 2 * j].item() == (lo - off) * d + m and b[0, 2 * j + 1].item() == (hi - off) * d + m
                lo_g = (byte & 15) | (((qh >> j) & 1) << 4)
                hi_g = (byte >> 4) | (((qh >> (j + 16)) & 1) << 4)
                assert a[0, j].item() == (lo_g - off) * d + m and a[0, j + 16].item() == (hi_g - off) * d + m


def test_q8_0_identity_and_negative():
    from ferrotorch_b200.serialize import gguf as G
    raw = _blocks(_f16_bytes(1.0) + list(range(32)))
    assert G.dequantize_blocks(raw, G.GGML_Q8_0, 32).tolist() == [float(i) for i in range(32)]
    raw = _blocks(_f16_bytes(2.0) + [0xFF, 0xFE] + [0] * 30)
    assert G.dequantize_blocks(raw, G.GGML_Q8_0, 32)[:2].tolist() == [-2.0, -4.0]


def test_f16_values_and_specials():
    from ferrotorch_b200.serialize import gguf as G
    raw = _blocks(*[_f16_bytes(v) for v in (0.0, 1.0, -1.0, 0.5)])
    assert G.dequantize_blocks(raw, G.GGML_F16, 4).tolist() == [0.0, 1.0, -1.0, 0.5]
    raw = torch.tensor([0x00, 0x80, 0x00, 0x7C, 0x01, 0x7C, 0x01, 0x00], dtype=torch.uint8)
    y = G.dequantize_blocks(raw, G.GGML_F16, 4)
    assert y[0].item() == 0.0 and math.copysign(1.0, y[0].item()) == -1.0
    assert math.isinf(y[1].item()) and y[1].item() > 0 and math.isnan(y[2].item())
    assert y[3].item() == 2.0 ** -24    # smallest subnormal


def test_block_properties():
    from ferrotorch_b200.serialize import gguf as G
    assert G._BLOCK[G.GGML_F32] == (1, 4) and G._BLOCK[G.GGML_F16] == (1, 2)
    assert G._BLOCK[G.GGML_Q4_0] == (32, 18) and G._BLOCK[G.GGML_Q8_0] == (32, 34)


def _stub(tensor_count, kv_count, tail=b""):
    import struct
    return b"GGUF" + struct.pack("<IQQ", 3, tensor_count, kv_count) + tail


@pytest.mark.parametrize("payload", [
    b"GGUF",                                               # truncated after the magic
    _stub(0, 2 ** 64 - 1), _stub(2 ** 64 - 1, 0), _stub(2 ** 64 - 1, 2 ** 64 - 1),
    _stub(0, 100_000), _stub(100_000, 0),
    _stub(0, 1, (100).to_bytes(8, "little")),              # key length 100, no key bytes
    _stub(0, 1, (1).to_bytes(8, "little") + b"x" + (9).to_bytes(4, "little") + (4).to_bytes(4, "little")
          + (2 ** 64 - 1).to_bytes(8, "little")),          # array of 2^64 - 1 elements
    b"GGML" + bytes(20),                                   # wrong magic
])
def test_gguf_header_lies_are_rejected_fast(tmp_path, payload):
    import time
    from ferrotorch_b200.serialize import gguf as G
    p = tmp_path / "bad.gguf"
    p.write_bytes(payload)
    t0 = time.perf_counter()
    with pytest.raises(ValueError):
        G.GgufFile(str(p))
    assert time.perf_counter() - t0 < 1.0


def test_q4_0_planes_accept_both_orders():
    from ferrotorch_b200.ops import quant as Q
    raw = torch.randint(0, 256, (16, 18), dtype=torch.uint8, generator=torch.Generator().manual_seed(5))
    raw[:, :2] = torch.tensor(_f16_bytes(1.0), dtype=torch.uint8)
    for order in ("ggml", "interleaved"):
        nib, sc = Q.q4_0_planes(raw, 8, 64, order)
        assert torch.equal(Q.dequant_q4_0_planes(nib, sc).reshape(-1), R.dequant_q4_0(raw, order))


# --------------------------------------------------------------------------- native formats
# Layouts of ferrotorch-serialize/src/state_dict.rs:74-165 and checkpoint.rs:86-200: files the
# reference wrote must load here, and f32 files written here must be laid out the same way.
def _reference_state_dict_bytes():
    import struct
    head = ('{"name":"fc.bias","shape":[2],"dtype":"f32","byte_offset":0,"byte_length":8}\n'
            '{"name":"fc.weight","shape":[2,3],"dtype":"f32","byte_offset":8,"byte_length":24}\n')
    body = struct.pack("<2f", 0.5, -1.0) + struct.pack("<6f", *range(6))
    return head.encode() + b"\n---\n" + body


def test_native_state_dict_layout_matches_the_reference_writer():
    from ferrotorch_b200.serialize import state as S
    raw = _reference_state_dict_bytes()
    sd = S.loads_state_dict(raw)
    assert sd["fc.bias"].tolist() == [0.5, -1.0]
    assert sd["fc.weight"].tolist() == [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]
    # written in insertion order "weight, bias": the writer sorts, so the bytes come out identical
    again = S.dumps_state_dict({"fc.weight": sd["fc.weight"], "fc.bias": sd["fc.bias"]})
    assert again == raw
    assert S.dumps_state_dict({}) == b"\n---\n" and S.loads_state_dict(b"\n---\n") == {}
    f64 = S.loads_state_dict(b'{"name":"s","shape":[],"dtype":"f64","byte_offset":0,"byte_length":8}\n\n---\n'
                             + __import__("struct").pack("<d", 1.25))
    assert f64["s"].dtype == torch.float64 and f64["s"].item() == 1.25 and f64["s"].dim() == 0


@pytest.mark.parametrize("line,err", [
    ('{"name":"w","shape":[4],"dtype":"f32","byte_offset":0,"byte_length":16}', "needs bytes"),      # body too short
    ('{"name":"w","shape":[3],"dtype":"f32","byte_offset":0,"byte_length":8}', "does not match"),    # shape vs bytes
    ('{"name":"w","shape":[2],"dtype":"q7","byte_offset":0,"byte_length":8}', "unknown dtype"),
])
def test_native_state_dict_rejects_inconsistent_headers(line, err):
    from ferrotorch_b200.serialize import state as S
    with pytest.raises(ValueError, match=err):
        S.loads_state_dict(line.encode() + b"\n\n---\n" + bytes(8))
    with pytest.raises(ValueError, match="separator"):
        S.loads_state_dict(line.encode())


def test_reference_checkpoint_layout_round_trip(tmp_path):
    import struct
    from ferrotorch_b200.serialize import state as S
    sd = _reference_state_dict_bytes()
    meta = b'{"epoch":3,"step":1200}'
    opt = b'{"fc.weight":{"exp_avg":[0.1,0.2,0.3,0.4,0.5,0.6],"step":[1200]}}'
    blob = b"".join(struct.pack("<Q", len(x)) + x for x in (meta, opt, sd))
    p = tmp_path / "checkpoint_epoch_3.ftc"
    p.write_bytes(blob)
    ck = S.load_checkpoint(str(p))
    assert ck["epoch"] == 3 and ck["step"] == 1200
    assert ck["optimizer"]["fc.weight"]["step"] == [1200] and len(ck["optimizer"]["fc.weight"]["exp_avg"]) == 6
    assert ck["model"]["fc.weight"].shape == (2, 3)
    q = tmp_path / "back.ftc"
    S.save_reference_checkpoint(str(q), ck["model"], ck["optimizer"], epoch=3, step=1200)
    raw = q.read_bytes()
    assert raw[8:8 + len(meta)] == meta and raw.endswith(sd)
    again = S.load_checkpoint(str(q))
    assert again["optimizer"] == {"fc.weight": {"exp_avg": [0.1, 0.2, 0.3, 0.4, 0.5, 0.6], "step": [1200.0]}}
    # a section length that lies about the file's size is an error, not an allocation
    (tmp_path / "lie.ftc").write_bytes(struct.pack("<Q", 1 << 60) + b"{}")
    with pytest.raises(ValueError, match="claims"):
        S.load_checkpoint(str(tmp_path / "lie.ftc"))


# --------------------------------------------------------------------------- Llama configuration
# ferrotorch-llama/src/config.rs:50-215 (presets, from_hf, validate) and mlp.rs:57-72 (activations).
def test_llama_presets_and_from_hf_follow_the_reference():
    from ferrotorch_b200.models.llama import LlamaConfig
    c = LlamaConfig.llama3_8b()
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads,
            c.num_key_value_heads, c.rope_theta, c.max_position_embeddings, c.tie_word_embeddings) == \
        (128256, 4096, 14336, 32, 32, 8, 500000.0, 8192, False)
    c = LlamaConfig.llama3_3_70b_instruct()
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads,
            c.max_position_embeddings, c.head_dim, c.kv_group_size()) == (8192, 28672, 80, 64, 8, 131072, 128, 8)
    c = LlamaConfig.llama2_7b()
    assert (c.vocab_size, c.intermediate_size, c.num_key_value_heads, c.rope_theta, c.max_position_embeddings) == \
        (32000, 11008, 32, 10000.0, 4096)
    p = LlamaConfig.prosparse_7b()
    assert p.hidden_act == "fatrelu" and p.hidden_act_param == 0.01 and p.intermediate_size == 11008
    base = {"vocab_size": 100, "hidden_size": 64, "intermediate_size": 96, "num_hidden_layers": 2,
            "num_attention_heads": 4}
    assert LlamaConfig.from_hf(dict(base)).num_key_value_heads == 4          # absent -> multi-head
    assert LlamaConfig.from_hf(dict(base, hidden_act="swish")).hidden_act == "silu"
    assert LlamaConfig.from_hf(dict(base, hidden_act="fatrelu")).hidden_act_param == 0.01
    assert LlamaConfig.from_hf(dict(base, hidden_act="fatrelu", hidden_act_param=0.05)).hidden_act_param == 0.05
    for bad in (dict(base, hidden_act="tanh"), dict(base, num_key_value_heads=3), dict(base, vocab_size=0)):
        with pytest.raises(ValueError):
            LlamaConfig.from_hf(bad)


def test_fatrelu_gate_matches_its_definition_and_trains():
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.ops import functional as F
    gu = torch.tensor([[0.005, 0.01, -1.0, 2.0, 3.0, 3.0, 3.0, 3.0]])
    assert torch.allclose(F.swiglu(gu, "fatrelu", 0.01), torch.tensor([[0.0, 0.03, 0.0, 6.0]]), atol=1e-7)
    assert F.swiglu(gu, "fatrelu").tolist() == F.swiglu(gu, "fatrelu", 0.01).tolist()
    cfg = LlamaConfig.from_hf({"vocab_size": 64, "hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 1,
                               "num_attention_heads": 2, "hidden_act": "fatrelu"})
    m = LlamaForCausalLM(cfg)
    ids = torch.randint(0, 64, (2, 6))
    m(ids).float().logsumexp(-1).sum().backward()
    g = m.model.layers[0].mlp.gate_up_proj.weight.grad
    assert g is not None and torch.isfinite(g).all() and g.abs().sum() > 0


# ferrotorch-llama/src/generation.rs:20-228: config constructors, argument checks, stop rules
def test_generation_config_constructors_checks_and_stop_rules():
    from ferrotorch_b200.models.generation import GenerationConfig, generate
    from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    g = GenerationConfig.greedy(5)
    assert (g.max_new_tokens, g.temperature, g.top_k, g.top_p, g.repetition_penalty) == (5, 0.0, 0, 1.0, 1.0)
    n = GenerationConfig.nucleus(7, 0.9, 0.8)
    assert (n.top_p, n.temperature, n.do_sample) == (0.9, 0.8, True)
    assert GenerationConfig.sampling(3, 0.0).do_sample is False
    torch.manual_seed(0)
    m = LlamaForCausalLM(LlamaConfig(vocab_size=32, hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                                     num_attention_heads=2, num_key_value_heads=1)).eval()
    ids = torch.randint(0, 32, (2, 4))
    for bad in (GenerationConfig(temperature=-1.0), GenerationConfig(top_p=1.5), GenerationConfig(repetition_penalty=0.0)):
        with pytest.raises(ValueError):
            generate(m, ids, bad)
    with pytest.raises(ValueError):
        generate(m, ids[:, :0], g)
    full = generate(m, ids, GenerationConfig.greedy(6))
    assert full.shape == (2, 10)
    # any id of eos_token_ids ends a row; the run stops when every row has ended
    first = full[:, 4].tolist()
    out = generate(m, ids, GenerationConfig(max_new_tokens=6, temperature=0.0, eos_token_ids=tuple(set(first))))
    assert out.shape == (2, 5)
    # a streamer that returns False stops after that token
    seen = []
    out = generate(m, ids, GenerationConfig.greedy(6), streamer=lambda t: (seen.append(t.tolist()), len(seen) < 2)[1])
    assert out.shape == (2, 6) and len(seen) == 2 and torch.equal(out, full[:, :6])


# ferrotorch-hub/src/hf_config.rs: the Llama-3-8B config.json of its tests, defaults, validation
_LLAMA3_8B_JSON = """{
  "architectures": ["LlamaForCausalLM"], "attention_bias": false, "attention_dropout": 0.0,
  "bos_token_id": 128000, "eos_token_id": 128001, "hidden_act": "silu", "hidden_size": 4096,
  "initializer_range": 0.02, "intermediate_size": 14336, "max_position_embeddings": 8192,
  "model_type": "llama", "num_attention_heads": 32, "num_hidden_layers": 32, "num_key_value_heads": 8,
  "pretraining_tp": 1, "rms_norm_eps": 1e-05, "rope_scaling": null, "rope_theta": 500000.0,
  "tie_word_embeddings": false, "torch_dtype": "bfloat16", "transformers_version": "4.40.0.dev0",
  "use_cache": true, "vocab_size": 128256}"""


def test_hf_transformer_config_parses_and_validates():
    from ferrotorch_b200.models.llama import LlamaConfig
    from ferrotorch_b200.utils.text import HfTransformerConfig
    c = HfTransformerConfig.from_json_str(_LLAMA3_8B_JSON)
    assert (c.hidden_size, c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads(), c.intermediate_size,
            c.max_position_embeddings, c.vocab_size, c.tie_word_embeddings, c.hidden_act, c.torch_dtype,
            c.architectures, c.model_type) == (4096, 32, 32, 8, 14336, 8192, 128256, False, "silu", "bfloat16",
                                               ["LlamaForCausalLM"], "llama")
    assert abs(c.rms_norm_eps - 1e-5) < 1e-12 and c.rope_theta == 500000.0 and c.head_dim() == 128 and c.is_gqa()
    assert c.to_llama() == LlamaConfig.llama3_8b()
    small = {"hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4, "intermediate_size": 128,
             "max_position_embeddings": 256, "vocab_size": 100}
    d = HfTransformerConfig.from_dict(small)
    assert (d.rms_norm_eps, d.rope_theta, d.hidden_act, d.num_key_value_heads(), d.is_gqa()) == \
        (1e-6, 10000.0, "silu", 4, False)
    ll = d.to_llama()
    assert (ll.rms_norm_eps, ll.rope_theta) == (1e-6, 10000.0)
    with pytest.raises(ValueError, match="missing"):
        HfTransformerConfig.from_dict({k: v for k, v in small.items() if k != "vocab_size"})
    with pytest.raises(ValueError, match="parse"):
        HfTransformerConfig.from_json_str("{not json")
    for bad in (dict(small, hidden_size=66), dict(small, num_key_value_heads=3), dict(small, hidden_act="mish"),
                dict(small, vocab_size=0)):
        with pytest.raises(ValueError):
            HfTransformerConfig.from_dict(bad).validate()
