"""Image files <-> tensors, and the transforms of the reference that torchvision names differently
or does not have (ferrotorch-vision/src/io.rs; transforms/{noise,blur,normalize,to_tensor}.rs)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class RawImage:
    """Bytes in row-major HWC order, values 0..255; 3 (RGB) or 4 (RGBA) channels (io.rs:36-45)."""
    data: bytes
    width: int
    height: int
    channels: int

    def __post_init__(self):
        if self.channels not in (3, 4) or self.width <= 0 or self.height <= 0:
            raise ValueError("RawImage: need 3 or 4 channels and a positive size")
        if len(self.data) != self.width * self.height * self.channels:
            raise ValueError("RawImage: %d bytes for a %dx%dx%d image" % (len(self.data), self.height, self.width, self.channels))


def _read(path: str, mode: str) -> RawImage:
    from PIL import Image

    with Image.open(path) as im:
        im = im.convert(mode)
        return RawImage(im.tobytes(), im.width, im.height, len(mode))


def read_image(path: str) -> RawImage:
    """Any format Pillow decodes (PNG, JPEG, BMP, GIF ...) as RGB."""
    return _read(path, "RGB")


def read_image_rgba(path: str) -> RawImage:
    return _read(path, "RGBA")


def raw_image_to_tensor(raw: RawImage, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """HWC bytes -> ``[C, H, W]`` in [0, 1]."""
    t = torch.frombuffer(bytearray(raw.data), dtype=torch.uint8).view(raw.height, raw.width, raw.channels)
    return t.permute(2, 0, 1).to(dtype) / 255.0


def read_image_as_tensor(path: str, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    return raw_image_to_tensor(read_image(path), dtype)


def tensor_to_raw_image(tensor: torch.Tensor) -> RawImage:
    """``[C, H, W]`` (C = 3 or 4) in [0, 1] -> bytes; values are clamped, then rounded."""
    if tensor.dim() != 3 or tensor.shape[0] not in (3, 4):
        raise ValueError("tensor_to_raw_image: expected [3 or 4, H, W], got %s" % (tuple(tensor.shape),))
    b = (tensor.detach().float().cpu().clamp(0, 1) * 255.0).round().to(torch.uint8).permute(1, 2, 0).contiguous()
    return RawImage(b.numpy().tobytes(), tensor.shape[2], tensor.shape[1], tensor.shape[0])


def write_image(path: str, image: RawImage) -> None:
    """The file extension picks the format; JPEG has no alpha, so RGBA input loses it there."""
    from PIL import Image

    im = Image.frombytes("RGB" if image.channels == 3 else "RGBA", (image.width, image.height), bytes(image.data))
    if image.channels == 4 and str(path).lower().endswith((".jpg", ".jpeg")):
        im = im.convert("RGB")
    im.save(path)


def write_tensor_as_image(path: str, tensor: torch.Tensor) -> None:
    write_image(path, tensor_to_raw_image(tensor))


# --------------------------------------------------------------------------- transforms
_gen = torch.Generator()


def vision_manual_seed(seed: int) -> None:
    """Seed the generator the random transforms of this module draw from."""
    _gen.manual_seed(seed)


class VisionToTensor(nn.Module):
    """RawImage / PIL image / uint8 HWC array -> float ``[C, H, W]`` in [0, 1]."""

    def forward(self, x):
        if isinstance(x, RawImage):
            return raw_image_to_tensor(x)
        if isinstance(x, torch.Tensor):
            return (x.permute(2, 0, 1).float() / 255.0) if x.dtype == torch.uint8 else x
        import numpy as np

        a = np.asarray(x)
        if a.ndim == 2:
            a = a[:, :, None]
        return torch.from_numpy(a.copy()).permute(2, 0, 1).float() / 255.0


class VisionNormalize(nn.Module):
    """Per-channel ``(x - mean) / std`` on ``[C, H, W]`` or ``[B, C, H, W]``."""

    def __init__(self, mean, std):
        super().__init__()
        if len(mean) != len(std) or any(s == 0 for s in std):
            raise ValueError("VisionNormalize: mean and std need equal lengths and non-zero std")
        self.register_buffer("mean", torch.tensor(mean, dtype=torch.float32).view(-1, 1, 1))
        self.register_buffer("std", torch.tensor(std, dtype=torch.float32).view(-1, 1, 1))

    @classmethod
    def imagenet(cls) -> "VisionNormalize":
        """The ImageNet statistics every pretrained classifier of the zoo expects."""
        return cls((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))

    def forward(self, x):
        if x.shape[-3] != self.mean.shape[0]:
            raise ValueError("VisionNormalize: %d channels, %d means" % (x.shape[-3], self.mean.shape[0]))
        return (x - self.mean.to(x.dtype)) / self.std.to(x.dtype)


class GaussianNoise(nn.Module):
    """Adds N(mean, sigma^2) noise; ``clip`` keeps the result in [0, 1]."""

    def __init__(self, mean: float = 0.0, sigma: float = 0.1, clip: bool = True):
        super().__init__()
        if sigma < 0:
            raise ValueError("GaussianNoise: sigma must be >= 0")
        self.mean, self.sigma, self.clip = mean, sigma, clip

    def with_clip(self, clip: bool) -> "GaussianNoise":
        return GaussianNoise(self.mean, self.sigma, bool(clip))

    def forward(self, x):
        noise = torch.randn(x.shape, generator=_gen).to(x.device, x.dtype) * self.sigma + self.mean
        y = x + noise
        return y.clamp(0, 1) if self.clip else y


class RandomGaussianBlur(nn.Module):
    """With probability ``p`` blur with a Gaussian kernel whose sigma is drawn from ``sigma``."""

    def __init__(self, kernel_size: int = 3, sigma=(0.1, 2.0), p: float = 0.5):
        super().__init__()
        if kernel_size % 2 == 0 or kernel_size <= 0:
            raise ValueError("RandomGaussianBlur: kernel_size must be odd and positive")
        self.k, self.sigma, self.p = kernel_size, tuple(sigma), p

    def forward(self, x):
        if float(torch.rand((), generator=_gen)) >= self.p:
            return x
        s = self.sigma[0] + (self.sigma[1] - self.sigma[0]) * float(torch.rand((), generator=_gen))
        r = torch.arange(self.k, dtype=torch.float32) - self.k // 2
        k1 = torch.exp(-(r ** 2) / (2 * s * s))
        k1 = (k1 / k1.sum()).to(x.device, x.dtype)
        img = x if x.dim() == 4 else x[None]
        C, pad = img.shape[1], self.k // 2
        img = nn.functional.pad(img, (pad, pad, pad, pad), mode="reflect")
        img = nn.functional.conv2d(img, k1.view(1, 1, 1, -1).expand(C, 1, 1, -1), groups=C)
        img = nn.functional.conv2d(img, k1.view(1, 1, -1, 1).expand(C, 1, -1, 1), groups=C)
        return img if x.dim() == 4 else img[0]
