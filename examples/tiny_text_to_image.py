"""The latent-diffusion pipeline end to end on a miniature configuration: token ids -> CLIP text
states -> guided DDIM denoising in latent space -> VAE decoder -> PNG.  Random weights, so the image
is noise with structure; the point is the plumbing (swap the configs for ``sd_v1_5()`` presets and
load SafeTensors weights to get the real model)."""
import argparse
import os
import sys
import tempfile

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import vision  # noqa: E402
from ferrotorch_b200.models import diffusion as D  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--size", type=int, default=64)
    ap.add_argument("--out", default=os.path.join(tempfile.gettempdir(), "ferrotorch_b200_tiny.png"))
    args = ap.parse_args()
    torch.manual_seed(0)
    clip = D.ClipTextEncoder(D.ClipTextConfig(vocab_size=1000, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                              num_attention_heads=4, max_position_embeddings=16)).eval()
    unet = D.UNet2DConditionModel(D.UNet2DConditionConfig(
        block_out_channels=(32, 64), down_block_types=("CrossAttnDownBlock2D", "DownBlock2D"),
        up_block_types=("UpBlock2D", "CrossAttnUpBlock2D"), layers_per_block=1, cross_attention_dim=64,
        attention_head_dim=4, norm_num_groups=8)).eval()
    vae = D.AutoencoderKL(D.VaeConfig(block_out_channels=(16, 32, 32, 32), layers_per_block=1, norm_num_groups=8)).eval()
    pipe = D.StableDiffusionPipeline(clip, unet, vae, D.DDIMScheduler(D.DDIMConfig.sd_v1_5()))
    prompt = torch.tensor([[1, 17, 254, 3, 999, 2, 2, 2]])           # begin, four "words", end, padding
    image = pipe(prompt, height=args.size, width=args.size, num_inference_steps=args.steps, guidance_scale=7.5, seed=3)
    pixels = D.to_uint8(image)
    vision.write_tensor_as_image(args.out, (image[0] / 2 + 0.5).clamp(0, 1))
    back = vision.read_image(args.out)
    assert (back.width, back.height) == (args.size, args.size) and pixels.shape == (1, args.size, args.size, 3)
    print("timesteps", pipe.scheduler.timesteps, "-> wrote", args.out, "mean pixel", float(pixels.float().mean()))


if __name__ == "__main__":
    main()
