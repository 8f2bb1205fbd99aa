"""Checkpoint formats round-trip on CPU: SafeTensors (single, sharded, filtered), .pt, native
state dict, training checkpoint (sync + async), GGUF (all block types vs a NumPy restatement),
Llama HF key layout."""
import os
import struct

import numpy as np
import pytest
import torch

from ferrotorch_b200 import serialize as S
from ferrotorch_b200.models.llama import LlamaConfig, LlamaForCausalLM
from ferrotorch_b200.ops import reference as R


def _state():
    torch.manual_seed(0)
    return {"a.weight": torch.randn(5, 7), "b": torch.randn(3).to(torch.bfloat16), "c": torch.arange(6).view(2, 3),
            "empty": torch.zeros(0)}


def _same(x, y):
    assert x.keys() == y.keys()
    for k in x:
        assert x[k].dtype == y[k].dtype and x[k].shape == y[k].shape and torch.equal(x[k], y[k]), k


def test_safetensors_single_sharded_filtered(tmp_path):
    sd = _state()
    p = str(tmp_path / "m.safetensors")
    S.save_safetensors(sd, p)
    _same(S.load_safetensors(p), sd)
    assert set(S.load_safetensors(p, key_filter=lambda k: k.startswith("a"))) == {"a.weight"}
    assert S.load_safetensors(p, dtype=torch.bfloat16)["a.weight"].dtype == torch.bfloat16
    idx = S.save_safetensors_sharded(sd, str(tmp_path / "sh"), max_shard_bytes=64)
    seen = []
    _same(S.load_safetensors_sharded(idx, progress=lambda i, n: seen.append((i, n))), sd)
    assert seen and seen[-1][0] == seen[-1][1] > 1


def test_pt_and_native_state_dict(tmp_path):
    sd = _state()
    S.save_pytorch(sd, str(tmp_path / "m.pt"))
    _same(S.load_pytorch_state_dict(str(tmp_path / "m.pt")), sd)
    torch.save({"state_dict": sd, "epoch": 3}, str(tmp_path / "wrapped.pt"))
    _same(S.load_pytorch_state_dict(str(tmp_path / "wrapped.pt")), sd)
    _same(S.loads_state_dict(S.dumps_state_dict(sd)), sd)
    S.save_state_dict(sd, str(tmp_path / "m.ftsd"))
    _same(S.load_state_dict(str(tmp_path / "m.ftsd")), sd)


def test_training_checkpoint_sync_and_async(tmp_path):
    model = torch.nn.Linear(4, 3)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    model(torch.randn(2, 4)).sum().backward()
    opt.step()
    p = str(tmp_path / "ck.ftc")
    S.save_checkpoint(p, model.state_dict(), opt.state_dict(), epoch=2, step=17, extra={"scaler": {"scale": 65536.0}})
    ck = S.load_checkpoint(p)
    assert ck["epoch"] == 2 and ck["step"] == 17 and ck["extra"]["scaler"]["scale"] == 65536.0
    _same(ck["model"], dict(model.state_dict()))
    opt2 = torch.optim.AdamW(torch.nn.Linear(4, 3).parameters(), lr=1e-2)
    opt2.load_state_dict(ck["optimizer"])
    assert torch.equal(opt2.state_dict()["state"][0]["exp_avg"], opt.state_dict()["state"][0]["exp_avg"])
    fut = S.AsyncCheckpointer().save_async(str(tmp_path / "a.ftc"), model.state_dict(), opt.state_dict(), epoch=1)
    fut.wait()
    assert fut.is_done() and S.load_checkpoint(str(tmp_path / "a.ftc"))["epoch"] == 1
    with open(str(tmp_path / "bad"), "wb") as f:
        f.write(b"nope")
    with pytest.raises(ValueError):
        S.load_checkpoint(str(tmp_path / "bad"))


def _np_dequant(t, raw, n):
    b = np.frombuffer(raw, dtype=np.uint8)
    if t == S.gguf.GGML_F32:
        return b.view(np.float32).copy()
    if t == S.gguf.GGML_F16:
        return b.view(np.float16).astype(np.float32)
    be, bb = S.gguf._BLOCK[t]
    blk = b.reshape(-1, bb)
    d = blk[:, :2].copy().view(np.float16).astype(np.float32)
    out = np.zeros((blk.shape[0], 32), np.float32)
    if t in (S.gguf.GGML_Q4_0, S.gguf.GGML_Q4_1):
        o = 2 if t == S.gguf.GGML_Q4_0 else 4
        m = 0 if t == S.gguf.GGML_Q4_0 else blk[:, 2:4].copy().view(np.float16).astype(np.float32)
        lo, hi = (blk[:, o:o + 16] & 15).astype(np.float32), (blk[:, o:o + 16] >> 4).astype(np.float32)
        q = np.concatenate([lo, hi], 1)
        out = (q - 8) * d if t == S.gguf.GGML_Q4_0 else q * d + m
    elif t in (S.gguf.GGML_Q5_0, S.gguf.GGML_Q5_1):
        o = 2 if t == S.gguf.GGML_Q5_0 else 4
        m = 0 if t == S.gguf.GGML_Q5_0 else blk[:, 2:4].copy().view(np.float16).astype(np.float32)
        qh = blk[:, o:o + 4].copy().view(np.uint32)
        qs = blk[:, o + 4:o + 20]
        j = np.arange(16, dtype=np.uint32)
        h0 = (((qh >> j) << 4) & 0x10).astype(np.uint8)
        h1 = ((qh >> (j + 12)) & 0x10).astype(np.uint8)
        q = np.concatenate([(qs & 15) | h0, (qs >> 4) | h1], 1).astype(np.float32)
        out = (q - 16) * d if t == S.gguf.GGML_Q5_0 else q * d + m
    else:
        o = 2 if t == S.gguf.GGML_Q8_0 else 4
        out = blk[:, o:o + 32].copy().view(np.int8).astype(np.float32) * d
    return out.reshape(-1)[:n]


def test_gguf_reader_all_block_types(tmp_path):
    rng = np.random.default_rng(0)
    tensors, want = {}, {}
    for t, (be, bb) in S.gguf._BLOCK.items():
        if t == S.gguf.GGML_BF16:
            continue
        shape = (4, 64)
        n = 4 * 64
        raw = rng.integers(0, 256, n // be * bb, dtype=np.uint8)
        if be == 32:  # keep the fp16 scale fields finite
            blk = raw.reshape(-1, bb)
            blk[:, :2] = np.array([0.5], np.float16).view(np.uint8)
            if t in (S.gguf.GGML_Q4_1, S.gguf.GGML_Q5_1, S.gguf.GGML_Q8_1):
                blk[:, 2:4] = np.array([-1.25], np.float16).view(np.uint8)
        elif t == S.gguf.GGML_F16:
            raw = rng.standard_normal(n).astype(np.float16).view(np.uint8)
        else:
            raw = rng.standard_normal(n).astype(np.float32).view(np.uint8)
        tensors["t%d.weight" % t] = (t, shape, raw.tobytes())
        want["t%d.weight" % t] = _np_dequant(t, raw.tobytes(), n).reshape(shape)
    p = str(tmp_path / "x.gguf")
    S.write_gguf(p, tensors, {"general.architecture": "llama", "llama.block_count": 2, "x.f": 1.5, "x.b": True})
    with S.GgufFile(p) as f:
        assert f.version == 3 and f.metadata["general.architecture"] == "llama" and f.metadata["llama.block_count"] == 2
        for name, w in want.items():
            got = f.dequantize(name).numpy()
            assert got.shape == w.shape and np.array_equal(got, w), name
    with open(str(tmp_path / "bad.gguf"), "wb") as fh:
        fh.write(b"GGUF" + struct.pack("<I", 99) + b"\0" * 32)
    with pytest.raises(ValueError):
        S.GgufFile(str(tmp_path / "bad.gguf"))


def test_q4_0_quantise_roundtrip_and_key_map(tmp_path):
    torch.manual_seed(1)
    w = torch.randn(8, 128)
    blocks = S.quantize_q4_0(w)
    deq = R.dequant_q4_0(blocks).view(8, 128)
    assert (deq - w).abs().max() < w.abs().max() / 7
    p = str(tmp_path / "q.gguf")
    S.write_gguf(p, {"blk.0.attn_q.weight": (S.gguf.GGML_Q4_0, (8, 128), blocks.numpy().tobytes()),
                     "token_embd.weight": (S.gguf.GGML_F32, (4, 8), torch.ones(4, 8).numpy().tobytes())})
    sd = S.load_gguf_state_dict(p, dtype=torch.float32)
    assert set(sd) == {"model.layers.0.self_attn.q_proj.weight", "model.embed_tokens.weight"}
    assert torch.equal(sd["model.layers.0.self_attn.q_proj.weight"], deq)
    with S.GgufFile(p) as f:
        scales, nib = f.q4_0_planes("blk.0.attn_q.weight")
    assert scales.shape == (8, 4) and nib.shape == (8, 64)
    lo, hi = (nib.view(8, 4, 16) & 15).float() - 8, (nib.view(8, 4, 16) >> 4).float() - 8
    assert torch.equal((torch.cat([lo, hi], -1) * scales.float()[..., None]).view(8, 128), deq)
    assert S.gguf_key_to_hf("output.weight") == "lm_head.weight" and S.gguf_key_to_hf("rope_freqs.weight") is None


def test_llama_hf_state_dict_roundtrip_through_safetensors(tmp_path):
    cfg = LlamaConfig.tiny()
    cfg.num_hidden_layers = 1
    torch.manual_seed(2)
    m = LlamaForCausalLM(cfg)
    sd = m.hf_state_dict()
    assert "model.layers.0.self_attn.k_proj.weight" in sd and "model.layers.0.mlp.up_proj.weight" in sd
    S.save_safetensors(sd, str(tmp_path / "llama.safetensors"))
    m2 = LlamaForCausalLM(cfg)
    m2.load_hf_state_dict(S.load_safetensors(str(tmp_path / "llama.safetensors")))
    x = torch.randint(0, cfg.vocab_size, (1, 9))
    assert torch.equal(m(x), m2(x))
    bad = dict(sd)
    del bad["model.layers.0.self_attn.v_proj.weight"]
    with pytest.raises(KeyError):
        m2.load_hf_state_dict(bad)


def test_int4_checkpoint_layouts_round_trip():
    import torch

    from ferrotorch_b200.serialize import quant_loaders as Q

    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.1
    for pack, deq in ((Q.pack_gptq, Q.dequantize_gptq), (Q.pack_awq, Q.dequantize_awq)):
        qw, qz, sc = pack(w, 128)
        assert qw.dtype == torch.int32 and qz.dtype == torch.int32 and sc.dtype == torch.float16
        d = deq(qw, qz, sc, group_size=128)
        assert d.shape == w.shape and float((d - w).abs().max()) <= float(sc.float().max()) * 0.51 + 1e-3
    # GPTQ with an explicit (permuted) group index
    qw, qz, sc = Q.pack_gptq(w, 128)
    g_idx = torch.arange(256) // 128
    assert torch.equal(Q.dequantize_gptq(qw, qz, sc, g_idx), Q.dequantize_gptq(qw, qz, sc, group_size=128))
    wq, s, z = Q.pack_hqq(w, 64)
    assert wq.dtype == torch.uint8 and wq.numel() == w.numel() // 2
    d = Q.dequantize_hqq(wq, s, z, (64, 256), 64)
    assert float((d - w).abs().max()) <= float(s.max()) * 0.51
    # the AWQ interleave: nibble j of a word holds column [0, 2, 4, 6, 1, 3, 5, 7][j]
    word = int(Q._pack_int32(torch.arange(8, dtype=torch.int32).reshape(1, 8), 1, Q._AWQ_ORDER)[0, 0])
    assert [(word >> (4 * j)) & 0xF for j in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]
    # on to the fused dequant-GEMM's layout
    lin = Q.to_q4_linear(d)
    x = torch.randn(3, 256)
    ref = x @ d.t()
    assert float((lin(x) - ref).norm() / ref.norm()) < 0.15      # a second 4-bit rounding


def test_onnx_export_round_trip_without_an_onnx_package(tmp_path):
    """The hand-written protobuf encoder: export, parse back, evaluate with the reference
    evaluator, compare with the module."""
    import ferrotorch_b200.serialize as S
    from ferrotorch_b200.serialize import onnx as O
    from torch import nn

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.q, self.k, self.v, self.o = nn.Linear(8, 8), nn.Linear(8, 8, bias=False), nn.Linear(8, 8), nn.Linear(8, 4)

        def forward(self, x):
            a = torch.softmax(torch.matmul(self.q(x), self.k(x).transpose(-1, -2)) * 0.35, dim=-1)
            h = torch.matmul(a, self.v(x))
            h = torch.nn.functional.gelu(h) + torch.nn.functional.silu(x) - torch.tanh(x) / 2.0
            return self.o(h.reshape(2, 5, 8)).relu(), (1.0 - h).abs().sqrt()

    torch.manual_seed(0)
    m, x = Net().eval(), torch.randn(2, 5, 8)
    path = str(tmp_path / "m.onnx")
    cfg = S.OnnxExportConfig(input_names=["x"], output_names=["y", "z"], dynamic_axes={"x": {0: "batch"}})
    S.export_onnx(m, (x,), path, cfg)
    model = S.load_onnx(path)
    assert (model.ir_version, model.opset_version, model.producer_name) == (8, 17, "ferrotorch_b200")
    assert model.inputs == [("x", torch.float32, ["batch", 5, 8])]
    assert model.outputs == [("y", torch.float32, [2, 5, 4]), ("z", torch.float32, [2, 5, 8])]
    ops = {n.op_type for n in model.nodes}
    assert {"MatMul", "Softmax", "Transpose", "Erf", "Sigmoid", "Reshape", "Relu"} <= ops and "Gelu" not in ops   # opset 17
    assert sum(1 for t in model.initializers.values() if t.dim() == 2) == 4                                       # the four weights
    y, z = S.run_onnx(model, x)
    wy, wz = m(x)
    assert torch.allclose(y, wy, atol=1e-6) and torch.allclose(z, wz, atol=1e-6)
    with pytest.raises(O.OnnxExportError):
        S.run_onnx(model, x.double())
    with pytest.raises(O.OnnxExportError, match="no ONNX mapping"):
        S.export_onnx(lambda t: torch.cumsum(t, 0), (x,), str(tmp_path / "bad.onnx"))
    # wire format primitives
    w = O.ProtobufWriter().int(1, 300).int(2, -1).string(3, "ab").float(4, 1.5)
    assert w.finish()[:3] == bytes([0x08, 0xAC, 0x02])
    fields = O.read_message(w.finish())
    assert fields[0] == (1, 0, 300) and fields[1][2] == (1 << 64) - 1 and fields[2] == (3, 2, b"ab") and fields[3] == (4, 5, 1.5)
    for junk in (bytes([0x08]), bytes([0x0A, 0x05, 0x01]), bytes([0x0B])):
        with pytest.raises(O.OnnxExportError):
            O.read_message(junk)
    # an exported program carries its dynamic dimensions into the ONNX inputs
    from ferrotorch_b200 import jit as J
    lin = nn.Sequential(nn.Linear(4, 3), nn.Tanh()).eval()
    ep = J.export(lin, (torch.randn(3, 4),), [J.InputSpec([J.DimSpec.dynamic_range("n", 2, 16), J.DimSpec.static(4)])])
    S.export_from_program(ep, str(tmp_path / "p.onnx"))
    pm = S.load_onnx(str(tmp_path / "p.onnx"))
    assert pm.inputs[0][2] == ["n", 4]
    t = torch.randn(7, 4)
    assert torch.allclose(S.run_onnx(pm, t)[0], lin(t), atol=1e-6)
    with pytest.raises(O.OnnxExportError, match="no IR graph"):
        S.export_from_program(J.ExportedProgram.deserialize(ep.serialize()), str(tmp_path / "q.onnx"))


def test_pickle_inspection_and_mmap_load(tmp_path):
    import ferrotorch_b200.serialize as S

    sd = {"w": torch.arange(6.0).view(2, 3), "b": torch.ones(2, dtype=torch.bfloat16)}
    p = str(tmp_path / "m.pt")
    S.save_pytorch(sd, p)
    mm = S.load_pytorch_state_dict_mmap(p)
    assert torch.equal(mm["w"], sd["w"]) and mm["b"].dtype == torch.bfloat16
    imports = S.pickle_imports(p)
    assert "torch._utils._rebuild_tensor_v2" in imports and all(i.startswith(("torch.", "collections.")) for i in imports)
    import pickle
    ops = S.parse_pickle(pickle.dumps({"a": 1}, protocol=2))
    assert ops[0][0] == "PROTO" and ops[-1][0] == "STOP" and ("BININT1", 1) in ops
    with pytest.raises(ValueError):
        S.parse_pickle(b"\x80\x02}q\x00(X\x01")            # truncated stream
    evil = str(tmp_path / "evil.pt")
    torch.save({"x": os.path.join}, evil)                  # a function reference: visible before anything is loaded
    assert any("join" in i for i in S.pickle_imports(evil))


def test_gguf_and_checkpoint_reference_names(tmp_path):
    import ferrotorch_b200.serialize as S

    w = torch.randn(4, 64)
    blocks = S.quantize_q4_0(w)
    path = str(tmp_path / "m.gguf")
    S.write_gguf(path, {"blk.0.attn_q.weight": (int(S.GgmlType.Q4_0), (4, 64), bytes(blocks.reshape(-1).tolist())),
                        "output_norm.weight": (int(S.GgmlType.F32), (64,), torch.ones(64).numpy().tobytes())},
                 {"general.architecture": "llama"})
    f = S.load_gguf(path)
    infos = {i.name: i for i in S.tensor_infos(f)}
    q = infos["blk.0.attn_q.weight"]
    assert q.ggml_type is S.GgmlType.Q4_0 and q.shape == (4, 64) and q.numel() == 256 and q.nbytes == S.GgmlType.Q4_0.nbytes(256) == 144
    assert (S.GgmlType.Q4_0.block_size, S.GgmlType.Q4_0.type_size) == (32, 18) and f.metadata["general.architecture"] == "llama"
    deq = S.dequantize_gguf_tensor(f, "blk.0.attn_q.weight")
    assert deq.shape == (4, 64) and (deq - w).abs().max() < 0.5
    with open(path, "rb") as fh:
        g = S.parse_gguf_bytes(fh.read())
    torch.testing.assert_close(g.dequantize("blk.0.attn_q.weight"), deq)
    sd = S.load_gguf_state_dict_mmap(path, torch.float32)
    assert set(sd) == {"model.layers.0.self_attn.q_proj.weight", "model.norm.weight"}
    with pytest.raises(ValueError):
        S.GgmlType.Q4_0.nbytes(33)
    ck = S.TrainingCheckpoint({"w": w}, {"state": {}, "param_groups": [{"lr": 0.1, "params": [0]}]}, epoch=3, step=40, extra={"note": "x"})
    ck.save(str(tmp_path / "c.ftck"))
    back = S.TrainingCheckpoint.load(str(tmp_path / "c.ftck"))
    assert back.epoch == 3 and back.step == 40 and back.extra == {"note": "x"} and torch.equal(back.model_state["w"], w)
    assert back.optimizer_state["param_groups"][0]["lr"] == 0.1


def test_shared_block_decoder_equals_the_host_reader_for_every_quantised_type():
    """``gguf_blocks.h`` is what the device kernel compiles; run on the host it must reproduce the
    reader's dequantisation bit for bit (random bytes cover every nibble / high-bit / sign case)."""
    from ferrotorch_b200.serialize import gguf as G

    g = torch.Generator().manual_seed(0)
    for t in (G.GGML_Q4_0, G.GGML_Q4_1, G.GGML_Q5_0, G.GGML_Q5_1, G.GGML_Q8_0, G.GGML_Q8_1):
        be, bb = G._BLOCK[t]
        nblk = 64
        raw = torch.randint(0, 256, (nblk, bb), dtype=torch.uint8, generator=g)
        # finite fp16 scales / minima: rewrite the fp16 fields with values drawn from a normal range
        scale = (torch.rand(nblk, generator=g) * 0.1 + 1e-3).to(torch.float16).view(torch.uint8).view(nblk, 2)
        raw[:, 0:2] = scale
        if t in (G.GGML_Q4_1, G.GGML_Q5_1, G.GGML_Q8_1):
            raw[:, 2:4] = (torch.randn(nblk, generator=g) * 0.5).to(torch.float16).view(torch.uint8).view(nblk, 2)
        ref = G.dequantize_blocks(raw.reshape(-1), t, nblk * be)
        got = G.dequantize_pairwise_host(raw.reshape(-1), t, nblk * be)
        assert torch.equal(got, ref.reshape(-1)), "type %d" % t
    sub = torch.tensor([1, 0], dtype=torch.uint8)                     # fp16 subnormal 2^-24 as a scale
    blk = torch.cat([sub, torch.full((16,), 0x9F, dtype=torch.uint8)])
    v = G.dequantize_pairwise_host(blk, G.GGML_Q4_0, 32)
    assert v[0].item() == 7 * 2.0 ** -24 and v[16].item() == 1 * 2.0 ** -24
    with pytest.raises(ValueError):
        G.dequantize_pairwise_host(blk, G.GGML_F16, 32)
    with pytest.raises(ValueError):
        G.dequantize_on_device(blk, G.GGML_Q4_0, (32,))               # a host tensor is refused before any launch


def test_onnx_export_of_reductions_shape_ops_and_convolutional_layers(tmp_path):
    """The rest of the reference exporter's operator list (reductions, LogSoftmax, Squeeze /
    Unsqueeze, Concat, general Transpose, Gemm) and the layers of a small CNN (Conv, batch norm in
    eval mode, max / average / global pooling), checked with the reference evaluator."""
    import ferrotorch_b200.serialize as S
    from ferrotorch_b200.serialize import onnx as O
    from torch import nn

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.conv, self.bn = nn.Conv2d(3, 8, 3, 2, 1), nn.BatchNorm2d(8)
            self.dw = nn.Conv2d(8, 8, 3, padding=2, dilation=2, groups=8, bias=False)
            self.pool, self.avg, self.gap = nn.MaxPool2d(3, 2, 1), nn.AvgPool2d(2), nn.AdaptiveAvgPool2d(1)
            self.fc, self.ls = nn.Linear(8, 5), nn.LogSoftmax(dim=-1)

        def forward(self, x):
            h = self.dw(torch.relu(self.bn(self.conv(x))))
            h = self.gap(self.avg(self.pool(h))).flatten(1)
            z = self.fc(h)
            total, mean = z.sum(1, keepdim=True), z.mean(dim=-1)
            both = torch.cat([z, total], 1)
            moved = both.unsqueeze(0).permute(1, 0, 2).squeeze(1).transpose(0, 1)
            return self.ls(z), moved, mean, torch.prod(z, 1), z.sum()

    torch.manual_seed(0)
    net = Net().eval()
    with torch.no_grad():
        net.bn.running_mean.normal_()
        net.bn.running_var.uniform_(0.5, 1.5)
    x = torch.randn(2, 3, 20, 20)
    path = str(tmp_path / "cnn.onnx")
    S.export_onnx(net, (x,), path)
    model = S.load_onnx(path)
    ops = {n.op_type for n in model.nodes}
    assert {"Conv", "BatchNormalization", "MaxPool", "AveragePool", "GlobalAveragePool", "Gemm", "LogSoftmax", "ReduceSum", "ReduceMean",
            "ReduceProd", "Concat", "Unsqueeze", "Squeeze", "Transpose"} <= ops
    conv = [n for n in model.nodes if n.op_type == "Conv"]
    assert conv[0].attrs["strides"] == [2, 2] and conv[0].attrs["pads"] == [1, 1, 1, 1] and conv[1].attrs["group"] == 8 \
        and conv[1].attrs["dilations"] == [2, 2]
    with torch.no_grad():
        want = net(x)
    for got, w in zip(S.run_onnx(model, x), want):
        assert got.shape == w.shape and torch.allclose(got, w, atol=1e-5)
    # export_onnx switches a training-mode model to eval for the trace and back afterwards; a graph traced in
    # training mode by hand is refused (batch norm would use batch statistics)
    net.train()
    S.export_onnx(net, (x,), str(tmp_path / "train.onnx"))
    assert net.training
    for got, w in zip(S.run_onnx(S.load_onnx(str(tmp_path / "train.onnx")), x), want):
        assert torch.allclose(got, w, atol=1e-5)
    from ferrotorch_b200.jit.module import trace

    with pytest.raises(O.OnnxExportError, match="eval mode"):
        S.export_ir_graph_to_onnx(trace(net, (x,)), str(tmp_path / "bad.onnx"))


def test_state_dict_files_are_aligned_and_load_as_views(tmp_path):
    """Files written by ``save_state_dict`` start their tensor bytes on a 64-byte offset and place
    every tensor on a multiple of 8, so the parallel reader and the memory map both hand out views;
    the dense layout (``align=0``) stays byte-identical to ``dumps_state_dict``."""
    from ferrotorch_b200.serialize import state as S

    torch.manual_seed(0)
    sd = {"w": torch.randn(33, 7), "odd": torch.arange(5, dtype=torch.uint8), "h": torch.randn(3).bfloat16(), "i": torch.arange(7),
          "empty": torch.zeros(0), "b": torch.tensor([True, False, True])}
    path = str(tmp_path / "m.ftsd")
    S.save_state_dict(sd, path)
    raw = open(path, "rb").read()
    body = raw.find(b"\n---\n") + 5
    assert body % 64 == 0
    import json

    for line in raw[:body - 5].decode().splitlines():
        if line.strip():
            assert json.loads(line)["byte_offset"] % 8 == 0
    for kw in ({}, {"threads": 1}, {"mmap": True}):
        back = S.load_state_dict(path, **kw)
        assert set(back) == set(sd)
        for k, v in sd.items():
            assert back[k].dtype == v.dtype and back[k].shape == v.shape and torch.equal(back[k], v), (kw, k)
    eager = S.load_state_dict(path)
    assert eager["w"].untyped_storage().data_ptr() == eager["i"].untyped_storage().data_ptr(), "views of one buffer, not copies"
    S.save_state_dict(sd, path, align=0)
    assert open(path, "rb").read() == S.dumps_state_dict(sd)
    assert all(torch.equal(S.load_state_dict(path)[k], v) for k, v in sd.items())
    # the parallel reader: any region, and typed failures
    blob = bytes(range(256)) * 1000
    p2 = tmp_path / "blob.bin"
    p2.write_bytes(blob)
    for off, n in ((0, len(blob)), (3, 1000), (255999, 1), (100, 0)):
        assert bytes(S.read_file_parallel(str(p2), off, n, threads=3).numpy()) == blob[off:off + n]
    with pytest.raises(ValueError):
        S.read_file_parallel(str(p2), 10, len(blob))
    with pytest.raises(OSError):
        S.read_file_parallel(str(tmp_path / "missing.bin"))


def test_safetensors_parallel_loader_equals_the_library_loader(tmp_path):
    from ferrotorch_b200.serialize import state as S

    torch.manual_seed(1)
    sd = {"a.weight": torch.randn(17, 9), "a.bias": torch.randn(9).bfloat16(), "ids": torch.arange(11), "flag": torch.tensor([True, False]),
          "half": torch.randn(4, 4).half(), "empty": torch.zeros(0, 3), "bytes": torch.arange(7, dtype=torch.uint8)}
    path = str(tmp_path / "m.safetensors")
    S.save_safetensors(sd, path, metadata={"format": "pt"})
    lib = S.load_safetensors(path)
    for threads in (1, 4):
        got = S.load_safetensors_parallel(path, threads=threads)
        assert set(got) == set(sd)
        for k in sd:
            assert got[k].dtype == lib[k].dtype and got[k].shape == lib[k].shape and torch.equal(got[k], lib[k]), k
    only = S.load_safetensors_parallel(path, key_filter=lambda k: k.startswith("a."), dtype=torch.float16)
    assert set(only) == {"a.weight", "a.bias"} and only["a.weight"].dtype == torch.float16
    header, base = S.read_safetensors_header(path)
    assert header["__metadata__"] == {"format": "pt"} and header["ids"]["dtype"] == "I64" and base > 8
    # hostile headers: a length field larger than the file, offsets past the end, a shape that does not match its bytes
    raw = bytearray(open(path, "rb").read())
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((1 << 40).to_bytes(8, "little") + bytes(raw[8:]))
    with pytest.raises(ValueError):
        S.load_safetensors_parallel(str(bad))
    import json

    n = int.from_bytes(raw[:8], "little")
    hdr = json.loads(bytes(raw[8:8 + n]))
    for mutate in (lambda h: h["ids"].__setitem__("data_offsets", [0, 1 << 30]), lambda h: h["ids"].__setitem__("shape", [12])):
        h2 = json.loads(json.dumps(hdr))
        mutate(h2)
        blob = json.dumps(h2).encode()
        bad.write_bytes(len(blob).to_bytes(8, "little") + blob + bytes(raw[8 + n:]))
        with pytest.raises(ValueError):
            S.load_safetensors_parallel(str(bad))


# --------------------------------------------------------------------------- GGUF blocks as planes
@pytest.mark.parametrize("kind_name", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q8_1"])
def test_gguf_plane_split_and_expansion_equal_the_block_decoder(kind_name):
    """split on the host + torch expansion (the reference's split_q*_blocks / dequantize_q*_to_gpu
    pair) against the native decoder of raw blocks, bitwise, in both element orders."""
    import numpy as np

    import ferrotorch_b200 as ft
    from ferrotorch_b200.serialize import gguf as G
    from ferrotorch_b200.serialize import gguf_planes as P

    kind = P.GgufBlockKind[kind_name]
    assert kind.block_elements == 32 and kind.block_bytes == G._BLOCK[int(kind)][1]
    rng = np.random.default_rng(int(kind))
    nb = 41
    raw = rng.integers(0, 256, (nb, kind.block_bytes), dtype=np.uint8)
    raw[:, 0:2] = rng.standard_normal(nb).astype(np.float16).view(np.uint8).reshape(nb, 2)      # finite scales
    if kind.has_min or kind == P.GgufBlockKind.Q8_1:
        raw[:, 2:4] = rng.standard_normal(nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    t = torch.from_numpy(raw.reshape(-1).copy())
    split = getattr(ft.cubecl, "split_%s_blocks" % kind_name.lower())
    to_dev = getattr(ft.cubecl, "dequantize_%s_to_gpu" % kind_name.lower())
    planes = split(t, nb)
    assert len(planes) == 2 + int(kind.has_min) + int(kind.has_high_bits)
    assert planes[-1].shape == (nb, 8 if kind_name.startswith("Q8") else 4) and int(planes[-1].max()) < 2 ** 32
    for order in ("ggml", "interleaved"):
        want = G.dequantize_blocks(t, int(kind), nb * 32, order)
        assert torch.equal(to_dev(*planes, nb * 32, device="cpu", nibble_order=order), want)
    assert to_dev(*planes, nb * 32, device="cpu", dtype=torch.bfloat16).dtype == torch.bfloat16
    assert torch.equal(split(bytes(raw.reshape(-1)), nb)[0], planes[0])                        # bytes in, same planes
    with pytest.raises(ValueError):
        split(t[:-1], nb)
    with pytest.raises(ValueError):
        to_dev(*planes, nb * 32 - 32, device="cpu")
    with pytest.raises(TypeError):
        to_dev(planes[0], nb * 32, device="cpu")
