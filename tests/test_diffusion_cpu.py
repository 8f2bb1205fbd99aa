"""Latent-diffusion stack on tiny configs (CPU): shapes, checkpoint key names and parameter counts
of the SD-1.5 presets, scheduler algebra, guidance, determinism."""
import math

import pytest
import torch

from ferrotorch_b200.models import diffusion as D


def _tiny():
    torch.manual_seed(0)
    clip = D.ClipTextEncoder(D.ClipTextConfig(vocab_size=100, hidden_size=24, intermediate_size=48, num_hidden_layers=2,
                                              num_attention_heads=4, max_position_embeddings=16))
    unet = D.UNet2DConditionModel(D.UNet2DConditionConfig(
        block_out_channels=(16, 32), down_block_types=("CrossAttnDownBlock2D", "DownBlock2D"),
        up_block_types=("UpBlock2D", "CrossAttnUpBlock2D"), layers_per_block=1, cross_attention_dim=24,
        attention_head_dim=4, norm_num_groups=8))
    vae = D.AutoencoderKL(D.VaeConfig(block_out_channels=(8, 16, 16, 16), layers_per_block=1, norm_num_groups=4))
    return clip.eval(), unet.eval(), vae.eval()


def test_sd15_presets_have_the_published_sizes_and_key_names():
    with torch.device("meta"):
        unet, vae, clip = D.UNet2DConditionModel(), D.AutoencoderKL(), D.ClipTextEncoder()
    n = lambda m: sum(p.numel() for p in m.parameters())  # noqa: E731
    assert n(unet) == 859_520_964 and n(vae) == 83_653_863 and n(clip) == 123_060_480
    ks = set(unet.state_dict())
    for k in ["conv_in.weight", "time_embedding.linear_1.weight", "down_blocks.0.resnets.0.time_emb_proj.weight",
              "down_blocks.0.attentions.1.transformer_blocks.0.attn2.to_k.weight", "down_blocks.2.downsamplers.0.conv.bias",
              "down_blocks.1.attentions.0.transformer_blocks.0.ff.net.0.proj.weight", "mid_block.attentions.0.proj_in.weight",
              "up_blocks.0.upsamplers.0.conv.weight", "up_blocks.3.resnets.2.conv_shortcut.weight",
              "up_blocks.1.attentions.2.transformer_blocks.0.attn1.to_out.0.bias", "conv_norm_out.weight", "conv_out.bias"]:
        assert k in ks, k
    assert "down_blocks.3.attentions.0.norm.weight" not in ks and "down_blocks.3.downsamplers.0.conv.weight" not in ks
    sd = unet.state_dict()
    assert sd["up_blocks.1.resnets.0.conv1.weight"].shape == (1280, 2560, 3, 3)
    assert sd["up_blocks.3.resnets.2.conv1.weight"].shape == (320, 640, 3, 3)
    assert sd["down_blocks.0.attentions.0.transformer_blocks.0.attn2.to_k.weight"].shape == (320, 768)
    ks = set(vae.state_dict())
    for k in ["encoder.down_blocks.0.downsamplers.0.conv.weight", "decoder.up_blocks.1.resnets.2.conv1.weight",
              "decoder.mid_block.attentions.0.to_q.weight", "encoder.mid_block.attentions.0.group_norm.bias",
              "decoder.up_blocks.2.resnets.0.conv_shortcut.weight", "quant_conv.weight", "post_quant_conv.bias"]:
        assert k in ks, k
    ks = set(clip.state_dict())
    for k in ["text_model.embeddings.token_embedding.weight", "text_model.embeddings.position_embedding.weight",
              "text_model.encoder.layers.11.self_attn.out_proj.bias", "text_model.encoder.layers.0.mlp.fc1.weight",
              "text_model.final_layer_norm.weight"]:
        assert k in ks, k
    assert clip.state_dict()["text_model.embeddings.position_embedding.weight"].shape == (77, 768)


def test_clip_text_encoder_matches_transformers_and_is_causal():
    cfg = D.ClipTextConfig(vocab_size=100, hidden_size=24, intermediate_size=48, num_hidden_layers=2,
                           num_attention_heads=4, max_position_embeddings=16)
    torch.manual_seed(1)
    ours = D.ClipTextEncoder(cfg).eval()
    ids = torch.randint(0, 100, (2, 9))
    out = ours(ids)
    ids2 = ids.clone()
    ids2[:, 6:] = (ids2[:, 6:] + 1) % 100
    assert torch.allclose(ours(ids2)[:, :6], out[:, :6], atol=1e-6) and not torch.allclose(ours(ids2)[:, 6:], out[:, 6:])
    tr = pytest.importorskip("transformers")
    hf_cfg = tr.CLIPTextConfig(vocab_size=100, hidden_size=24, intermediate_size=48, num_hidden_layers=2,
                               num_attention_heads=4, max_position_embeddings=16, hidden_act="quick_gelu",
                               eos_token_id=99, bos_token_id=0, pad_token_id=1)
    hf = tr.CLIPTextModel(hf_cfg).eval()
    missing = ours.load_hf_state_dict(hf.state_dict())
    assert not missing.missing_keys and not missing.unexpected_keys
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state
        got = ours(ids)
    assert torch.allclose(got, want, atol=2e-5), (got - want).abs().max()
    with pytest.raises(ValueError):
        ours(torch.zeros(1, 17, dtype=torch.long))
    with pytest.raises(ValueError):
        ours(torch.full((1, 3), 100))
    with pytest.raises(ValueError):
        D.ClipTextConfig(hidden_size=10, num_attention_heads=4).validate()


def test_ddim_scheduler_algebra():
    s = D.DDIMScheduler(D.DDIMConfig.sd_v1_5())
    ts = s.set_timesteps(50)
    assert ts[:3] == [981, 961, 941] and ts[-1] == 1 and len(ts) == 50 and s.init_noise_sigma() == 1.0
    assert s.alphas_cumprod[0].item() == pytest.approx(1 - 0.00085) and s.alphas_cumprod[-1].item() == pytest.approx(0.0047, abs=2e-4)
    assert D.DDIMScheduler(D.DDIMConfig(timestep_spacing="trailing")).set_timesteps(4) == [999, 749, 499, 249]
    # a model that always predicts the true noise walks back to x0 (up to the last step's alpha_0)
    torch.manual_seed(0)
    x0, noise = torch.randn(2, 4, 8, 8), torch.randn(2, 4, 8, 8)
    x = s.add_noise(x0, noise, ts[0])
    for t in ts:
        x = s.step(noise, t, x)
    a0 = s.alphas_cumprod[0]
    assert torch.allclose(x, (a0.sqrt() * x0 + (1 - a0).sqrt() * noise).float(), atol=1e-5)
    one = D.DDIMScheduler(D.DDIMConfig(set_alpha_to_one=True))
    one.set_timesteps(10)
    x = one.add_noise(x0, noise, one.timesteps[0])
    for t in one.timesteps:
        x = one.step(noise, t, x)
    assert torch.allclose(x, x0, atol=1e-5)
    with pytest.raises(ValueError):
        s.set_timesteps(0)
    with pytest.raises(ValueError):
        D.DDIMScheduler(D.DDIMConfig(prediction_type="v_prediction"))
    with pytest.raises(RuntimeError):
        D.DDIMScheduler().step(noise, 5, x0)


def test_timestep_embedding_formula():
    e = D.timestep_embedding(torch.tensor([0, 7]), 8)
    assert torch.allclose(e[0], torch.tensor([1.0] * 4 + [0.0] * 4))
    f = [math.exp(-math.log(10000.0) * i / 4) for i in range(4)]
    assert torch.allclose(e[1], torch.tensor([math.cos(7 * x) for x in f] + [math.sin(7 * x) for x in f]), atol=1e-6)
    assert torch.allclose(D.timestep_embedding(torch.tensor([7]), 8, flip_sin_to_cos=False)[0, :4], e[1, 4:])


def test_unet_and_vae_shapes_and_checks():
    clip, unet, vae = _tiny()
    ctx = clip(torch.randint(0, 100, (2, 7)))
    x = torch.randn(2, 4, 8, 8)
    y = unet(x, 10, ctx)
    assert y.shape == x.shape and torch.isfinite(y).all()
    assert torch.allclose(unet(x, torch.tensor([10, 10]), ctx), y, atol=1e-6)
    assert not torch.allclose(unet(x, 500, ctx), y) and not torch.allclose(unet(x, 10, ctx * 0), y)
    with pytest.raises(ValueError):
        unet(torch.randn(2, 3, 8, 8), 1, ctx)
    with pytest.raises(ValueError):
        unet(torch.randn(2, 4, 7, 8), 1, ctx)
    with pytest.raises(ValueError):
        D.UNet2DConditionConfig(block_out_channels=(30, 64)).validate()
    img = torch.randn(2, 3, 32, 32)
    post = vae.encode(img)
    assert post.mean.shape == (2, 4, 4, 4) and post.mode() is post.mean and (post.kl() >= 0).all()
    z = vae.encode_with_scaling(img, seed=5)
    assert torch.equal(z, vae.encode_with_scaling(img, seed=5)) and not torch.equal(z, vae.encode_with_scaling(img, seed=6))
    assert vae.decode_with_scaling(z).shape == (2, 3, 32, 32)
    with pytest.raises(ValueError):
        vae.encode(torch.randn(1, 3, 30, 32))
    # attention weights of older VAE checkpoints (1x1 convolutions called query / key / value / proj_attn)
    sd = {}
    for k, v in vae.state_dict().items():
        p = k.split(".")
        if "attentions" in p and p[-2] in ("to_q", "to_k", "to_v"):
            k, v = ".".join(p[:-2] + [{"to_q": "query", "to_k": "key", "to_v": "value"}[p[-2]], p[-1]]), (v[:, :, None, None] if v.dim() == 2 else v)
        elif "attentions" in p and p[-3:-1] == ["to_out", "0"]:
            k, v = ".".join(p[:-3] + ["proj_attn", p[-1]]), (v[:, :, None, None] if v.dim() == 2 else v)
        sd[k] = v
    other = D.AutoencoderKL(vae.config)
    res = other.load_hf_state_dict(sd)
    assert not res.missing_keys and not res.unexpected_keys
    assert torch.allclose(other.eval().decode(z), vae.decode(z), atol=1e-6)


def test_pipeline_guidance_and_determinism():
    clip, unet, vae = _tiny()
    pipe = D.StableDiffusionPipeline(clip, unet, vae)
    ids = torch.randint(2, 100, (1, 6))
    a = pipe(ids, height=32, width=32, num_inference_steps=3, seed=4)
    b = pipe(ids, height=32, width=32, num_inference_steps=3, seed=4)
    c = pipe(ids, height=32, width=32, num_inference_steps=3, seed=5)
    assert a.shape == (1, 3, 32, 32) and torch.equal(a, b) and not torch.equal(a, c)
    assert D.to_uint8(a).shape == (1, 32, 32, 3) and D.to_uint8(a).dtype == torch.uint8
    cond, unc = pipe.encode_prompt(ids), pipe.encode_prompt(torch.full_like(ids, 1))
    lat = torch.randn(1, 4, 4, 4, generator=torch.Generator().manual_seed(0))
    img1, dumps = pipe.generate(cond, unc, lat, 2, guidance_scale=1.0, dump=True)
    assert len(dumps) == 2 and dumps[0].timestep == pipe.scheduler.timesteps[0]
    assert torch.allclose(dumps[0].guided_noise, dumps[0].noise_pred_cond, atol=1e-6)     # g = 1: the conditional branch alone
    img0, d0 = pipe.generate(cond, unc, lat, 2, guidance_scale=0.0, dump=True)
    assert torch.allclose(d0[0].guided_noise, d0[0].noise_pred_uncond, atol=1e-6) and not torch.allclose(img0, img1)
    with pytest.raises(ValueError):
        pipe.generate(cond, unc[:, :3], lat, 2)
    with pytest.raises(ValueError):
        pipe(ids, height=30, width=32)


def test_pipeline_directory_round_trip(tmp_path):
    clip, unet, vae = _tiny()
    pipe = D.StableDiffusionPipeline(clip, unet, vae, D.DDIMScheduler(D.DDIMConfig(set_alpha_to_one=True)))
    D.save_stable_diffusion(pipe, str(tmp_path / "sd"))
    for rel in ("text_encoder/model.safetensors", "unet/diffusion_pytorch_model.safetensors", "vae/config.json",
                "scheduler/scheduler_config.json"):
        assert (tmp_path / "sd" / rel).exists(), rel
    back = D.load_stable_diffusion(str(tmp_path / "sd"))
    assert back.scheduler.config.set_alpha_to_one and back.unet.config.block_out_channels == (16, 32)
    ids = torch.randint(2, 100, (1, 5))
    a = pipe(ids, height=32, width=32, num_inference_steps=2, seed=1)
    b = back(ids, height=32, width=32, num_inference_steps=2, seed=1)
    assert torch.allclose(a, b, atol=1e-6)
    (tmp_path / "sd" / "unet" / "diffusion_pytorch_model.safetensors").unlink()
    with pytest.raises(FileNotFoundError):
        D.load_stable_diffusion(str(tmp_path / "sd"))


def test_reference_block_names_and_part_loaders(tmp_path):
    import json
    import os

    from ferrotorch_b200.models import diffusion as D
    from ferrotorch_b200.serialize.state import save_safetensors

    assert D.CrossAttnDownBlock2D is D.DownBlock2D and D.VaeDecoder is D.Decoder and D.Attention is not None
    assert str(D.PredictionType.VPrediction) == "v_prediction" and D.TimestepSpacing.Leading == "leading"
    t = torch.tensor([0.0, 10.0])
    torch.testing.assert_close(D.Timesteps(16)(t), D.timestep_embedding(t, 16))
    cfg = D.VaeConfig(block_out_channels=(8, 16), layers_per_block=1, norm_num_groups=4, latent_channels=4)
    vae = D.AutoencoderKL(cfg)
    d = tmp_path / "vae"
    os.makedirs(d)
    with open(d / "config.json", "w") as f:
        json.dump({"block_out_channels": [8, 16], "layers_per_block": 1, "norm_num_groups": 4, "latent_channels": 4}, f)
    save_safetensors(vae.state_dict(), str(d / "diffusion_pytorch_model.safetensors"))
    dec, enc = D.load_vae_decoder(str(d)), D.load_vae_encoder(str(d))
    z = torch.randn(1, 4, 4, 4)
    torch.testing.assert_close(dec(z), vae.eval().decoder(z))
    assert isinstance(enc, D.VaeEncoder)
    with pytest.raises(FileNotFoundError):
        D.load_unet(str(tmp_path))


def test_device_fast_path_pieces_on_the_host():
    """The device twins are the plain modules plus an attention dispatcher and the Philox
    generator: on the host they must reproduce the plain pipeline, and the head-size padding the
    dispatcher does for the kernel must not change the result."""
    import copy

    from ferrotorch_b200.models import diffusion_gpu as G
    from ferrotorch_b200.utils.philox import PhiloxGenerator

    torch.manual_seed(11)
    assert [G.pad_head_dim(d) for d in (8, 40, 64, 80, 128, 160, 512)] == [64, 64, 64, 128, 128, None, None]
    for d, sq, sk, causal in ((40, 9, 9, False), (80, 7, 13, False), (64, 6, 6, True), (24, 5, 5, True)):
        q, k, v = torch.randn(2, 3, sq, d), torch.randn(2, 3, sk, d), torch.randn(2, 3, sk, d)
        want = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
        assert torch.allclose(G.attend(q, k, v, causal, force_padded=True), want, atol=1e-5), (d, causal)
    q = torch.randn(1, 1, 4, 160)
    before = G.stats["library"]
    G.attend(q, q, q, force_padded=True)                       # no kernel head size for 160: library call
    assert G.stats["library"] == before + 1

    clip, unet, vae = _tiny()
    plain = D.StableDiffusionPipeline(copy.deepcopy(clip), copy.deepcopy(unet), copy.deepcopy(vae))
    fast = G.GpuStableDiffusionPipeline(D.StableDiffusionPipeline(clip, unet, vae), device="cpu", dtype=torch.float32)
    ids = torch.randint(2, 100, (2, 6))
    lat = fast.initial_latents(2, 32, 32, seed=9)
    g = PhiloxGenerator(9)
    want = torch.from_numpy(g.generate_normal(lat.numel())).view_as(lat)
    assert torch.allclose(lat, want.to(lat.dtype)), "initial latents are the host generator's normal stream"
    assert torch.equal(lat, fast.initial_latents(2, 32, 32, seed=9)) and not torch.equal(lat, fast.initial_latents(2, 32, 32, seed=10))
    cond, unc = fast.text_encoder(ids), fast.text_encoder(torch.full_like(ids, 1))
    assert torch.allclose(cond, plain.encode_prompt(ids), atol=1e-5)
    got = fast.generate(cond, unc, lat, 3, guidance_scale=5.0)
    ref, _ = plain.generate(plain.encode_prompt(ids), plain.encode_prompt(torch.full_like(ids, 1)), lat, 3, guidance_scale=5.0)
    assert got.shape == (2, 3, 32, 32) and torch.allclose(got, ref, atol=1e-4)
    assert fast(ids, height=32, width=32, num_inference_steps=2, seed=3).shape == (2, 3, 32, 32)
    enc = G.GpuVaeEncoder(copy.deepcopy(vae.encoder), device="cpu", dtype=torch.float32)
    z1 = enc.sample(torch.randn(1, 3, 32, 32), R_gen(5))
    assert z1.shape[1] == vae.config.latent_channels and torch.isfinite(z1).all()
    assert D._attention_override is None, "the dispatcher is only installed while a twin runs"


def R_gen(seed):
    from ferrotorch_b200.ops.random import DevicePhilox

    return DevicePhilox(seed, "cpu")
