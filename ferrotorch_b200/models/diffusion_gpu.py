"""Device fast path of the latent-diffusion stack: the same sub-models as ``models/diffusion.py``
(same parameters, same checkpoints) with their hot operators on this framework's kernels.

The reference has a CUDA twin of every sub-model (``ferrotorch-diffusion/src/gpu/{clip,unet,vae,
vae_encoder,pipeline}.rs``: ``GpuClipTextEncoder``, ``GpuUNet2DConditional``, ``GpuVaeDecoder``,
``GpuVaeEncoder``, ``GpuStableDiffusionPipeline``) that re-implements each forward op for op on
its element kernels and draws noise with ``gpu_philox_normal``.  Here a twin is the *same module*
prepared for the device:

* parameters in bf16, feature maps channels-last;
* every dense ``nn.Conv2d`` re-classed to the tcgen05 GEMM convolution (``ops.conv``);
* attention through :func:`attend`: head sizes 64 and 128 run on the flash-attention kernel as
  they are, smaller ones (40 and 80 in a Stable-Diffusion-1.5 UNet) are zero-padded to the next
  supported size (zeros in q / k add nothing to the scores, zero columns of v give zero output
  columns that are cut off again; the softmax scale stays ``1 / sqrt(d)`` of the real size), larger
  ones (160; the VAE's single 512-wide head) stay on ``scaled_dot_product_attention``;
* initial latents and the VAE's posterior sample come from the device Philox generator
  (``ops.random.DevicePhilox``), so a (seed, offset) pair reproduces them on any device.

On a CPU every piece falls back to the plain module, which is what the tests compare against.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF
from torch import nn

from ..ops import random as R
from ..ops.conv import convert_convs
from . import diffusion as Dm

stats = {"flash": 0, "flash_padded": 0, "library": 0}


def _flash_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def pad_head_dim(d: int) -> int | None:
    """The kernel head size that serves a real head size ``d`` (``None``: no kernel for it)."""
    return 64 if d <= 64 else 128 if d <= 128 else None


def attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, force_padded: bool = False) -> torch.Tensor:
    """``q [B, H, Sq, D]``, ``k / v [B, H, Sk, D]`` -> ``[B, H, Sq, D]`` (the layout of
    ``scaled_dot_product_attention``).  ``force_padded`` runs the padding arithmetic through the
    reference attention on any device (what the CPU test checks)."""
    D = q.shape[-1]
    Dp = pad_head_dim(D)
    use_kernel = _flash_ok(q) and Dp is not None
    if not (use_kernel or force_padded) or Dp is None:
        stats["library"] += 1
        return tF.scaled_dot_product_attention(q, k, v, is_causal=causal)
    qt, kt, vt = (t.transpose(1, 2) for t in (q, k, v))                      # [B, S, H, D]
    if Dp != D:
        qt, kt, vt = (tF.pad(t, (0, Dp - D)) for t in (qt, kt, vt))
        stats["flash_padded"] += 1
    else:
        stats["flash"] += 1
    if use_kernel:
        from ..ops.attention import flash_attention

        o = flash_attention(qt.contiguous(), kt.contiguous(), vt.contiguous(), causal=causal, scale=D ** -0.5)
    else:
        from ..ops import reference as ref

        o = ref.attention(qt, kt, vt, causal=causal, scale=D ** -0.5)[0]
    return o[..., :D].transpose(1, 2)


class _Routed:
    """Context manager that sends the attention calls of ``models/diffusion.py`` through :func:`attend`."""

    def __enter__(self):
        Dm._attention_override = attend
        return self

    def __exit__(self, *exc):
        Dm._attention_override = None
        return False


def prepare(module: nn.Module, device="cuda", dtype=torch.bfloat16) -> nn.Module:
    """Move a sub-model to the device in its fast-path form (in place; returns it)."""
    module.to(device=device, dtype=dtype)
    if any(p.dim() == 4 for p in module.parameters()):
        module.to(memory_format=torch.channels_last)
    convert_convs(module)
    return module.eval()


class _Twin(nn.Module):
    def __init__(self, inner: nn.Module, device="cuda", dtype=torch.bfloat16):
        super().__init__()
        self.inner = prepare(inner, device, dtype)
        self.device_, self.dtype_ = torch.device(device), dtype

    @property
    def config(self):
        return self.inner.config

    def _in(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(self.device_)
        return x.to(self.dtype_) if x.is_floating_point() else x

    @torch.no_grad()
    def forward(self, *args, **kw):
        with _Routed():
            return self.inner(*[self._in(a) if torch.is_tensor(a) else a for a in args], **kw)


class GpuClipTextEncoder(_Twin):
    """``input_ids [B, 77]`` -> text states ``[B, 77, hidden]`` (causal self-attention, head size 64)."""


class GpuUNet2DConditional(_Twin):
    """``(latent, timestep, text states)`` -> predicted noise; convolutions on the GEMM kernels,
    self- and cross-attention through :func:`attend`."""


class GpuVaeDecoder(_Twin):
    """Latents -> image."""


class GpuVaeEncoder(_Twin):
    """Image -> posterior moments; :meth:`sample` draws from the posterior with the device generator."""

    def sample(self, image: torch.Tensor, generator: "R.DevicePhilox") -> torch.Tensor:
        moments = self.forward(image)
        mean, logvar = moments.float().chunk(2, dim=1)
        std = torch.exp(0.5 * logvar.clamp(-30.0, 20.0))
        eps = generator.normal(*mean.shape).to(mean.device)
        return (mean + std * eps).to(self.dtype_)


class GpuStableDiffusionPipeline:
    """Text-to-image on the device: the three twins above around the host-side DDIM scheduler
    (the scheduler works on a handful of scalars per step and stays on the host, as in the
    reference's ``GpuStableDiffusionPipeline``)."""

    def __init__(self, pipe: "Dm.StableDiffusionPipeline", device="cuda", dtype=torch.bfloat16):
        self.device, self.dtype = torch.device(device), dtype
        self.text_encoder = GpuClipTextEncoder(pipe.text_encoder, device, dtype)
        self.unet = GpuUNet2DConditional(pipe.unet, device, dtype)
        self.vae_decoder = GpuVaeDecoder(_DecodeWithScaling(pipe.vae), device, dtype)
        self.scheduler = pipe.scheduler

    def initial_latents(self, batch: int, height: int, width: int, seed: int = 0) -> torch.Tensor:
        """``[B, C, height / 8, width / 8]`` standard-normal latents from ``(seed, counter 0)`` of
        the Philox generator: the same values on the host and on any GPU."""
        c = self.unet.config.in_channels
        return R.DevicePhilox(seed, self.device).normal(batch, c, height // 8, width // 8).to(self.dtype)

    @torch.no_grad()
    def generate(self, cond: torch.Tensor, uncond: torch.Tensor, init_latent: torch.Tensor, num_inference_steps: int = 50,
                 guidance_scale: float = 7.5) -> torch.Tensor:
        sch = self.scheduler
        latent = (init_latent.to(self.device, torch.float32) * sch.init_noise_sigma())
        ctx = torch.cat([uncond, cond], 0)
        for t in sch.set_timesteps(num_inference_steps):
            inp = sch.scale_model_input(torch.cat([latent, latent], 0), t)
            eps_u, eps_c = self.unet(inp, t, ctx).float().chunk(2, 0)
            latent = sch.step(eps_u + guidance_scale * (eps_c - eps_u), t, latent)      # fp32 latents between steps
        return self.vae_decoder(latent).float()

    @torch.no_grad()
    def __call__(self, prompt_ids: torch.Tensor, negative_ids: torch.Tensor | None = None, height: int = 512, width: int = 512,
                 num_inference_steps: int = 50, guidance_scale: float = 7.5, seed: int = 0) -> torch.Tensor:
        if prompt_ids.dim() == 1:
            prompt_ids = prompt_ids[None]
        if height % 8 or width % 8:
            raise ValueError("height and width must be multiples of 8")
        if negative_ids is None:
            negative_ids = prompt_ids.clone()
            negative_ids[:, 1:] = prompt_ids[:, -1:]
        noise = self.initial_latents(prompt_ids.shape[0], height, width, seed)
        return self.generate(self.text_encoder(prompt_ids), self.text_encoder(negative_ids), noise, num_inference_steps,
                             guidance_scale)


class _DecodeWithScaling(nn.Module):
    def __init__(self, vae: "Dm.AutoencoderKL"):
        super().__init__()
        self.vae = vae

    def forward(self, latent):
        return self.vae.decode_with_scaling(latent)
