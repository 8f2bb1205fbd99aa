"""Image transforms on float tensors ``[C, H, W]`` / ``[B, C, H, W]``, written out.

The reference's list (ferrotorch-vision/src/transforms/: center_crop, random_crop,
random_horizontal_flip, random_vertical_flip, resize, random_resized_crop, random_rotation,
color_jitter, elastic_transform, trivial_augment_wide, compose, random_apply; noise, blur,
normalisation and to-tensor are in ``vision/io.py``).  Every random transform draws from the
module generator that ``vision_manual_seed`` seeds, so a seed reproduces a pipeline.  Geometry is
done with ``affine_grid`` / ``grid_sample`` / ``interpolate`` (bilinear, ``align_corners=False``),
the conventions of ``torchvision.transforms.functional`` on tensors, which the tests compare with.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tF
from torch import nn

from . import io as _io


def _rand() -> float:
    return float(torch.rand((), generator=_io._gen))


def _randint(lo: int, hi: int) -> int:
    """Uniform integer in ``[lo, hi]``."""
    return int(torch.randint(lo, hi + 1, (), generator=_io._gen))


def _uniform(lo: float, hi: float) -> float:
    return lo + (hi - lo) * _rand()


def _pair(v) -> tuple[int, int]:
    return (int(v), int(v)) if isinstance(v, (int, float)) else (int(v[0]), int(v[1]))


def _batched(x: torch.Tensor) -> tuple[torch.Tensor, bool]:
    return (x, False) if x.dim() == 4 else (x[None], True)


# --------------------------------------------------------------------------- deterministic pieces
def crop(x: torch.Tensor, top: int, left: int, height: int, width: int) -> torch.Tensor:
    """Window ``[top, top + height) x [left, left + width)``; parts outside the image are zeros."""
    H, W = x.shape[-2:]
    pt, pl = max(0, -top), max(0, -left)
    pb, pr = max(0, top + height - H), max(0, left + width - W)
    if pt or pl or pb or pr:
        x = tF.pad(x, (pl, pr, pt, pb))
        top, left = top + pt, left + pl
    return x[..., top:top + height, left:left + width]


def center_crop(x: torch.Tensor, size, fill: float = 0.0) -> torch.Tensor:
    """The central ``size`` window; an image smaller than the window is padded evenly with ``fill``
    first (the odd pixel goes to the right / bottom)."""
    h, w = _pair(size)
    H, W = x.shape[-2:]
    if h > H or w > W:
        pl, pt = (w - W) // 2 if w > W else 0, (h - H) // 2 if h > H else 0
        pr, pb = (w - W + 1) // 2 if w > W else 0, (h - H + 1) // 2 if h > H else 0
        x = tF.pad(x, (pl, pr, pt, pb), value=fill)
        H, W = x.shape[-2:]
    return crop(x, int(round((H - h) / 2.0)), int(round((W - w) / 2.0)), h, w)


INTERPOLATIONS = ("nearest", "bilinear", "bicubic")


def resize(x: torch.Tensor, size, antialias: bool = True, interpolation: str = "bilinear") -> torch.Tensor:
    """``size`` int: the smaller edge becomes ``size`` (aspect kept); pair: exact ``(h, w)``.
    ``interpolation``: nearest, bilinear or bicubic (anti-aliasing applies to the last two)."""
    interpolation = str(getattr(interpolation, "value", interpolation)).lower()
    if interpolation not in INTERPOLATIONS:
        raise ValueError("resize: interpolation must be one of %s, got %r" % (INTERPOLATIONS, interpolation))
    H, W = x.shape[-2:]
    if isinstance(size, int):
        short, long = (W, H) if W <= H else (H, W)
        new_short, new_long = size, int(size * long / short)
        h, w = (new_long, new_short) if W <= H else (new_short, new_long)
    else:
        h, w = _pair(size)
    if (h, w) == (H, W):
        return x
    xb, squeeze = _batched(x)
    if interpolation == "nearest":
        y = tF.interpolate(xb, size=(h, w), mode="nearest")
    else:
        y = tF.interpolate(xb, size=(h, w), mode=interpolation, align_corners=False, antialias=antialias)
    return y[0] if squeeze else y


def hflip(x: torch.Tensor) -> torch.Tensor:
    return x.flip(-1)


def vflip(x: torch.Tensor) -> torch.Tensor:
    return x.flip(-2)


def _affine_sample(x: torch.Tensor, theta: torch.Tensor, fill: float = 0.0, mode: str = "bilinear", out_size=None) -> torch.Tensor:
    """``theta [2, 3]`` maps output pixel offsets from the centre to input pixel offsets from the centre.
    ``out_size (h, w)``: a canvas of another size around the same centre."""
    xb, squeeze = _batched(x)
    B, C, H, W = xb.shape
    oh, ow = out_size if out_size is not None else (H, W)
    xs = torch.linspace(-ow * 0.5 + 0.5, ow * 0.5 - 0.5, steps=ow, device=x.device)
    ys = torch.linspace(-oh * 0.5 + 0.5, oh * 0.5 - 0.5, steps=oh, device=x.device)
    yy, xx = torch.meshgrid(ys, xs, indexing="ij")
    base = torch.stack([xx, yy, torch.ones_like(xx)], -1)                         # [oh, ow, 3]
    H_in, W_in, H, W = H, W, oh, ow
    # normalise the matrix first, then apply it: the order matters for which side of a pixel edge
    # a nearest-neighbour sample falls on
    scaled = theta.to(torch.float32).t().to(x.device) / torch.tensor([0.5 * W_in, 0.5 * H_in], device=x.device)
    grid = (base.view(1, H * W, 3) @ scaled[None]).view(1, H, W, 2).expand(B, -1, -1, -1)
    ones = torch.ones((B, 1, H_in, W_in), dtype=xb.dtype, device=x.device)
    out = tF.grid_sample(torch.cat([xb, ones], 1), grid.to(xb.dtype), mode=mode, padding_mode="zeros", align_corners=False)
    img, mask = out[:, :C], out[:, C:]
    if mode == "nearest":
        img = torch.where(mask < 0.5, torch.full_like(img, fill), img)
    else:
        img = img * mask + (1 - mask) * fill                                      # blend the fill in at the border
    return img[0] if squeeze else img


def _inverse_affine(angle: float, translate, scale: float, shear, center=(0.0, 0.0)) -> list:
    """Output -> input matrix ``[a, b, tx, c, d, ty]`` of rotation / shear / scale about ``center`` (an
    offset from the image centre) followed by a translation."""
    rot, sx, sy = math.radians(angle), math.radians(shear[0]), math.radians(shear[1])
    a = math.cos(rot - sy) / math.cos(sy)
    b = -math.cos(rot - sy) * math.tan(sx) / math.cos(sy) - math.sin(rot)
    c = math.sin(rot - sy) / math.cos(sy)
    d = -math.sin(rot - sy) * math.tan(sx) / math.cos(sy) + math.cos(rot)
    (tx, ty), (cx, cy) = translate, center
    inv = [d / scale, -b / scale, 0.0, -c / scale, a / scale, 0.0]
    inv[2] = inv[0] * (-cx - tx) + inv[1] * (-cy - ty) + cx
    inv[5] = inv[3] * (-cx - tx) + inv[4] * (-cy - ty) + cy
    return inv


def affine(x: torch.Tensor, angle: float = 0.0, translate=(0.0, 0.0), scale: float = 1.0, shear=(0.0, 0.0), fill: float = 0.0,
           mode: str = "nearest") -> torch.Tensor:
    """Rotation (degrees, clockwise as the image is displayed), translation (pixels), isotropic
    scale and shear (degrees along x and y) about the centre: the output -> input matrix is the
    inverse of ``T(translate) * R(angle) * Shear * S(scale)``."""
    rot, sx, sy = math.radians(angle), math.radians(shear[0]), math.radians(shear[1])
    a = math.cos(rot - sy) / math.cos(sy)
    b = -math.cos(rot - sy) * math.tan(sx) / math.cos(sy) - math.sin(rot)
    c = math.sin(rot - sy) / math.cos(sy)
    d = -math.sin(rot - sy) * math.tan(sx) / math.cos(sy) + math.cos(rot)
    tx, ty = translate
    inv = [d / scale, -b / scale, 0.0, -c / scale, a / scale, 0.0]
    inv[2] = inv[0] * (-tx) + inv[1] * (-ty)
    inv[5] = inv[3] * (-tx) + inv[4] * (-ty)
    return _affine_sample(x, torch.tensor([inv[:3], inv[3:]]), fill, mode)


def rotate(x: torch.Tensor, angle: float, fill: float = 0.0, mode: str = "nearest", expand: bool = False, center=None) -> torch.Tensor:
    """Counter-clockwise rotation by ``angle`` degrees.  ``center``: the pivot ``(x, y)`` in pixels from
    the top-left corner (default: the image centre).  ``expand``: grow the canvas so that the whole
    rotated image fits (meant for rotations about the centre) instead of keeping the input's size."""
    if not expand and center is None:
        return affine(x, angle=-angle, fill=fill, mode=mode)
    H, W = x.shape[-2:]
    cf = (0.0, 0.0) if center is None else (float(center[0]) - W * 0.5, float(center[1]) - H * 0.5)
    inv = _inverse_affine(-angle, (0.0, 0.0), 1.0, (0.0, 0.0), cf)
    out_size = None
    if expand:
        theta = torch.tensor([inv[:3], inv[3:]], dtype=torch.float32)
        corners = torch.tensor([[-0.5 * W, -0.5 * H, 1.0], [-0.5 * W, 0.5 * H, 1.0], [0.5 * W, 0.5 * H, 1.0], [0.5 * W, -0.5 * H, 1.0]])
        pts = corners @ theta.t()
        lo, hi = pts.min(0).values + torch.tensor([W * 0.5, H * 0.5]), pts.max(0).values + torch.tensor([W * 0.5, H * 0.5])
        tol = 1e-4                                   # cut float noise before rounding outwards
        size = torch.ceil((hi / tol).trunc() * tol) - torch.floor((lo / tol).trunc() * tol)
        out_size = (int(size[1]), int(size[0]))
    return _affine_sample(x, torch.tensor([inv[:3], inv[3:]]), fill, mode, out_size)


def _gray(x: torch.Tensor) -> torch.Tensor:
    r, g, b = x.unbind(-3)
    return (0.2989 * r + 0.587 * g + 0.114 * b).unsqueeze(-3)     # the weights torchvision uses (ITU-R 601-2 rounded)


def _blend(a: torch.Tensor, b: torch.Tensor, ratio: float) -> torch.Tensor:
    return (ratio * a + (1.0 - ratio) * b).clamp(0, 1)


def adjust_brightness(x, f: float):
    return _blend(x, torch.zeros_like(x), f)


def adjust_contrast(x, f: float):
    mean = (_gray(x) if x.shape[-3] == 3 else x).mean((-3, -2, -1), keepdim=True)
    return _blend(x, mean, f)


def adjust_saturation(x, f: float):
    return _blend(x, _gray(x), f) if x.shape[-3] == 3 else x


def adjust_hue(x, f: float):
    """Shift the hue by ``f`` turns (``-0.5 .. 0.5``) through HSV."""
    if x.shape[-3] != 3 or f == 0:
        return x
    r, g, b = x.unbind(-3)
    mx, mn = x.max(-3).values, x.min(-3).values
    eq = mx == mn
    cr = mx - mn
    ones = torch.ones_like(mx)
    s = cr / torch.where(eq, ones, mx)
    crd = torch.where(eq, ones, cr)
    rc, gc, bc = (mx - r) / crd, (mx - g) / crd, (mx - b) / crd
    hr = (mx == r) * (bc - gc)
    hg = ((mx == g) & (mx != r)) * (2.0 + rc - bc)
    hb = ((mx != g) & (mx != r)) * (4.0 + gc - rc)
    h = ((hr + hg + hb) / 6.0 + 1.0) % 1.0
    h = (h + f) % 1.0
    i = torch.floor(h * 6.0)
    fr = h * 6.0 - i
    i = i.to(torch.int32) % 6
    p, q, t = (mx * (1.0 - s)).clamp(0, 1), (mx * (1.0 - s * fr)).clamp(0, 1), (mx * (1.0 - s * (1.0 - fr))).clamp(0, 1)
    sel = i.unsqueeze(-3) == torch.arange(6, device=x.device).view(-1, 1, 1)
    a1, a2, a3 = torch.stack((mx, q, p, p, t, mx), -3), torch.stack((t, mx, mx, q, p, p), -3), torch.stack((p, p, t, mx, mx, q), -3)
    return torch.stack([(a1 * sel).sum(-3), (a2 * sel).sum(-3), (a3 * sel).sum(-3)], -3)


def posterize(x, bits: int):
    q = (x * 255).to(torch.uint8) & (0xFF << (8 - bits) & 0xFF)
    return q.float() / 255


def solarize(x, threshold: float):
    return torch.where(x >= threshold, 1.0 - x, x)


def autocontrast(x):
    lo, hi = x.amin((-2, -1), keepdim=True), x.amax((-2, -1), keepdim=True)
    scale = torch.where(hi > lo, 1.0 / (hi - lo).clamp(min=1e-12), torch.ones_like(hi))
    lo = torch.where(hi > lo, lo, torch.zeros_like(lo))
    return ((x - lo) * scale).clamp(0, 1)


def adjust_sharpness(x, f: float):
    xb, squeeze = _batched(x)
    C = xb.shape[1]
    k = torch.tensor([[1.0, 1.0, 1.0], [1.0, 5.0, 1.0], [1.0, 1.0, 1.0]], device=x.device, dtype=x.dtype) / 13.0
    blurred = xb.clone()
    if min(xb.shape[-2:]) > 2:
        blurred[..., 1:-1, 1:-1] = tF.conv2d(xb, k.view(1, 1, 3, 3).expand(C, 1, 3, 3), groups=C)
    y = _blend(xb, blurred, f)
    return y[0] if squeeze else y


# --------------------------------------------------------------------------- transform objects
def _changed(obj, **attrs):
    """A shallow copy of a transform with some attributes replaced (the ``with_*`` builders return these)."""
    import copy

    out = copy.copy(obj)
    for k, v in attrs.items():
        setattr(out, k, v)
    return out


class Compose(nn.Module):
    def __init__(self, transforms):
        super().__init__()
        self.transforms = list(transforms)

    def __len__(self) -> int:
        return len(self.transforms)

    def len(self) -> int:
        return len(self.transforms)

    def is_empty(self) -> bool:
        return not self.transforms

    def forward(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class RandomApply(nn.Module):
    """Apply the whole list with probability ``p``."""

    def __init__(self, transforms, p: float = 0.5):
        super().__init__()
        self.transforms, self.p = list(transforms), p

    def forward(self, x):
        if _rand() >= self.p:
            return x
        for t in self.transforms:
            x = t(x)
        return x


class RandomChoice(nn.Module):
    """One of the transforms per call: uniformly, or with the probabilities given to :meth:`with_p`."""

    def __init__(self, transforms, p=None):
        super().__init__()
        self.transforms, self.p = list(transforms), None
        if p is not None:
            self.p = self._checked(p)

    def _checked(self, p):
        p = [float(v) for v in p]
        if len(p) != len(self.transforms) or any(v < 0 for v in p) or sum(p) <= 0:
            raise ValueError("RandomChoice: need one non-negative weight per transform, not all zero")
        return [v / sum(p) for v in p]

    def with_p(self, p) -> "RandomChoice":
        return _changed(self, p=self._checked(p))

    def forward(self, x):
        if self.p is None:
            return self.transforms[_randint(0, len(self.transforms) - 1)](x)
        u, acc = _rand(), 0.0
        for t, w in zip(self.transforms, self.p):
            acc += w
            if u < acc:
                return t(x)
        return self.transforms[-1](x)


class CenterCrop(nn.Module):
    def __init__(self, size, fill: float = 0.0):
        super().__init__()
        self.size, self.fill = _pair(size), fill

    def with_fill(self, fill: float) -> "CenterCrop":
        return _changed(self, fill=float(fill))

    def forward(self, x):
        return center_crop(x, self.size, self.fill)


class Resize(nn.Module):
    def __init__(self, size, antialias: bool = True, interpolation: str = "bilinear"):
        super().__init__()
        self.size, self.antialias, self.interpolation = size, antialias, interpolation

    def with_interpolation(self, interpolation: str) -> "Resize":
        return _changed(self, interpolation=interpolation)

    def with_antialias(self, antialias: bool) -> "Resize":
        return _changed(self, antialias=bool(antialias))

    def forward(self, x):
        return resize(x, self.size, self.antialias, self.interpolation)


class RandomCrop(nn.Module):
    """``padding``: pixels added on every side before cropping, one number or ``(vertical, horizontal)``;
    ``fill``: their value; ``pad_if_needed``: also pad an image that is still smaller than the crop."""

    def __init__(self, size, padding=0, pad_if_needed: bool = False, fill: float = 0.0):
        super().__init__()
        self.size, self.padding, self.pad_if_needed, self.fill = _pair(size), padding, pad_if_needed, fill

    @classmethod
    def square(cls, size: int) -> "RandomCrop":
        return cls((size, size))

    def with_padding(self, padding: int) -> "RandomCrop":
        return _changed(self, padding=int(padding))

    def with_padding_hw(self, pad_h: int, pad_w: int) -> "RandomCrop":
        return _changed(self, padding=(int(pad_h), int(pad_w)))

    def with_pad_if_needed(self, flag: bool = True) -> "RandomCrop":
        return _changed(self, pad_if_needed=bool(flag))

    def with_fill(self, fill: float) -> "RandomCrop":
        return _changed(self, fill=float(fill))

    def forward(self, x):
        ph, pw = (self.padding, self.padding) if isinstance(self.padding, int) else self.padding
        if ph or pw:
            x = tF.pad(x, (pw, pw, ph, ph), value=self.fill)
        h, w = self.size
        H, W = x.shape[-2:]
        if self.pad_if_needed and (H < h or W < w):
            x = tF.pad(x, (max(0, w - W), max(0, w - W), max(0, h - H), max(0, h - H)), value=self.fill)
            H, W = x.shape[-2:]
        if H < h or W < w:
            raise ValueError("RandomCrop: crop %s larger than image %s" % ((h, w), (H, W)))
        return crop(x, _randint(0, H - h), _randint(0, W - w), h, w)


class RandomHorizontalFlip(nn.Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return hflip(x) if _rand() < self.p else x


class RandomVerticalFlip(nn.Module):
    def __init__(self, p: float = 0.5):
        super().__init__()
        self.p = p

    def forward(self, x):
        return vflip(x) if _rand() < self.p else x


class RandomResizedCrop(nn.Module):
    """A window of ``scale`` x the image area and an aspect ratio drawn log-uniformly from
    ``ratio`` (ten attempts, then the central crop at the nearest allowed ratio), resized to ``size``."""

    def __init__(self, size, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0), antialias: bool = True, interpolation: str = "bilinear"):
        super().__init__()
        self.size, self.scale, self.ratio, self.antialias = _pair(size), tuple(scale), tuple(ratio), antialias
        self.interpolation = interpolation

    def with_antialias(self, antialias: bool) -> "RandomResizedCrop":
        return _changed(self, antialias=bool(antialias))

    def with_interpolation(self, interpolation: str) -> "RandomResizedCrop":
        return _changed(self, interpolation=interpolation)

    def get_params(self, H: int, W: int):
        area = H * W
        for _ in range(10):
            target = area * _uniform(*self.scale)
            ar = math.exp(_uniform(math.log(self.ratio[0]), math.log(self.ratio[1])))
            w, h = int(round(math.sqrt(target * ar))), int(round(math.sqrt(target / ar)))
            if 0 < w <= W and 0 < h <= H:
                return _randint(0, H - h), _randint(0, W - w), h, w
        in_ratio = W / H
        if in_ratio < self.ratio[0]:
            w, h = W, int(round(W / self.ratio[0]))
        elif in_ratio > self.ratio[1]:
            h, w = H, int(round(H * self.ratio[1]))
        else:
            w, h = W, H
        return (H - h) // 2, (W - w) // 2, h, w

    def forward(self, x):
        t, l, h, w = self.get_params(*x.shape[-2:])
        return resize(crop(x, t, l, h, w), self.size, self.antialias, self.interpolation)


class RandomRotation(nn.Module):
    def __init__(self, degrees, fill: float = 0.0, mode: str = "nearest", expand: bool = False, center=None):
        super().__init__()
        self.degrees = (-float(degrees), float(degrees)) if isinstance(degrees, (int, float)) else tuple(degrees)
        self.fill, self.mode, self.expand, self.center = fill, mode, expand, center

    def with_fill(self, fill: float) -> "RandomRotation":
        return _changed(self, fill=float(fill))

    def with_interpolation(self, mode: str) -> "RandomRotation":
        mode = str(getattr(mode, "value", mode)).lower()
        if mode not in ("nearest", "bilinear"):
            raise ValueError("RandomRotation: interpolation must be nearest or bilinear, got %r" % mode)
        return _changed(self, mode=mode)

    def with_expand(self, expand: bool = True) -> "RandomRotation":
        return _changed(self, expand=bool(expand))

    def with_center(self, center) -> "RandomRotation":
        return _changed(self, center=(float(center[0]), float(center[1])))

    def forward(self, x):
        return rotate(x, _uniform(*self.degrees), self.fill, self.mode, self.expand, self.center)


class ColorJitter(nn.Module):
    """Brightness, contrast, saturation factors from ``[max(0, 1 - v), 1 + v]``, hue shift from
    ``[-v, v]``, applied in a random order."""

    def __init__(self, brightness: float = 0.0, contrast: float = 0.0, saturation: float = 0.0, hue: float = 0.0):
        super().__init__()
        if not 0 <= hue <= 0.5:
            raise ValueError("ColorJitter: hue must be in [0, 0.5]")
        self.b, self.c, self.s, self.h = brightness, contrast, saturation, hue
        self.ranges = None

    @classmethod
    def from_ranges(cls, brightness=None, contrast=None, saturation=None, hue=None) -> "ColorJitter":
        """Explicit ``(low, high)`` factor ranges (``None`` = leave that property alone); hue within ``[-0.5, 0.5]``."""
        out = cls()
        rs = {"b": brightness, "c": contrast, "s": saturation, "h": hue}
        for k, r in rs.items():
            if r is None:
                continue
            lo, hi = float(r[0]), float(r[1])
            if lo > hi or (k == "h" and not -0.5 <= lo <= hi <= 0.5) or (k != "h" and lo < 0):
                raise ValueError("ColorJitter.from_ranges: bad range %r for %s" % (r, k))
            rs[k] = (lo, hi)
        out.ranges = rs
        return out

    def _range(self, k: str):
        if self.ranges is not None:
            return self.ranges[k]
        v = getattr(self, k)
        if not v:
            return None
        return (-v, v) if k == "h" else (max(0.0, 1 - v), 1 + v)

    def forward(self, x):
        ops = []
        for k, fn in (("b", adjust_brightness), ("c", adjust_contrast), ("s", adjust_saturation), ("h", adjust_hue)):
            r = self._range(k)
            if r is not None:
                ops.append(lambda t, f=_uniform(*r), fn=fn: fn(t, f))
        for i in torch.randperm(len(ops), generator=_io._gen).tolist():
            x = ops[i](x)
        return x


class ElasticTransform(nn.Module):
    """Displace every pixel by a smooth random field: uniform noise in ``[-1, 1]`` blurred with a
    Gaussian of ``sigma`` pixels and scaled by ``alpha`` pixels."""

    def __init__(self, alpha: float = 50.0, sigma: float = 5.0, fill: float = 0.0, interpolation: str = "bilinear"):
        super().__init__()
        self.alpha, self.sigma, self.fill, self.interpolation = alpha, sigma, fill, interpolation

    @classmethod
    def new_range(cls, alpha_range, sigma_range) -> "ElasticTransform":
        """``alpha`` and ``sigma`` drawn uniformly from the given ``(low, high)`` ranges at every call."""
        (a0, a1), (s0, s1) = alpha_range, sigma_range
        if a0 > a1 or s0 > s1 or s0 <= 0:
            raise ValueError("ElasticTransform.new_range: need low <= high and a positive sigma")
        return cls((float(a0), float(a1)), (float(s0), float(s1)))

    def with_fill(self, fill: float) -> "ElasticTransform":
        return _changed(self, fill=float(fill))

    def with_interpolation(self, interpolation: str) -> "ElasticTransform":
        interpolation = str(getattr(interpolation, "value", interpolation)).lower()
        if interpolation not in ("nearest", "bilinear"):
            raise ValueError("ElasticTransform: interpolation must be nearest or bilinear, got %r" % interpolation)
        return _changed(self, interpolation=interpolation)

    def forward(self, x):
        xb, squeeze = _batched(x)
        B, C, H, W = xb.shape
        alpha = _uniform(*self.alpha) if isinstance(self.alpha, tuple) else float(self.alpha)
        sigma = _uniform(*self.sigma) if isinstance(self.sigma, tuple) else float(self.sigma)
        k = int(8 * sigma + 1) | 1
        r = torch.arange(k, dtype=torch.float32) - k // 2
        g = torch.exp(-(r ** 2) / (2 * sigma ** 2))
        g = g / g.sum()
        field = torch.rand((2, 1, H, W), generator=_io._gen) * 2 - 1
        pad = k // 2
        if pad:
            field = tF.pad(field, (pad, pad, pad, pad), mode="reflect" if pad < min(H, W) else "replicate")
            field = tF.conv2d(tF.conv2d(field, g.view(1, 1, 1, -1)), g.view(1, 1, -1, 1))
        dx, dy = field[0, 0] * alpha / (W / 2), field[1, 0] * alpha / (H / 2)
        ys = (torch.arange(H, dtype=torch.float32) + 0.5) / (H / 2) - 1
        xs = (torch.arange(W, dtype=torch.float32) + 0.5) / (W / 2) - 1
        yy, xx = torch.meshgrid(ys, xs, indexing="ij")
        grid = torch.stack([xx + dx, yy + dy], -1)[None].expand(B, -1, -1, -1).to(xb.device, xb.dtype)
        ones = torch.ones((B, 1, H, W), dtype=xb.dtype, device=xb.device)
        out = tF.grid_sample(torch.cat([xb, ones], 1), grid, mode=self.interpolation, padding_mode="zeros", align_corners=False)
        y = out[:, :C] * out[:, C:] + (1 - out[:, C:]) * self.fill
        return y[0] if squeeze else y


class TrivialAugmentWide(nn.Module):
    """One operation per image, chosen uniformly, with a magnitude chosen uniformly from
    ``num_magnitude_bins`` levels of the operation's range (Mueller & Hutter 2021, "wide" ranges)."""

    def __init__(self, num_magnitude_bins: int = 31, fill: float = 0.0):
        super().__init__()
        self.bins, self.fill = num_magnitude_bins, fill

    def _space(self):
        n = self.bins
        lin = lambda hi: torch.linspace(0.0, hi, n)  # noqa: E731
        return {"Identity": (None, False), "ShearX": (lin(0.99), True), "ShearY": (lin(0.99), True), "TranslateX": (lin(32.0), True),
                "TranslateY": (lin(32.0), True), "Rotate": (lin(135.0), True), "Brightness": (lin(0.99), True), "Color": (lin(0.99), True),
                "Contrast": (lin(0.99), True), "Sharpness": (lin(0.99), True),
                "Posterize": (8 - (torch.arange(n) / ((n - 1) / 6)).round().int(), False), "Solarize": (torch.linspace(1.0, 0.0, n), False),
                "AutoContrast": (None, False), "Equalize": (None, False)}

    def apply_op(self, x, name: str, mag: float):
        if name == "ShearX":
            return affine(x, shear=(math.degrees(math.atan(mag)), 0.0), fill=self.fill)
        if name == "ShearY":
            return affine(x, shear=(0.0, math.degrees(math.atan(mag))), fill=self.fill)
        if name == "TranslateX":
            return affine(x, translate=(int(mag), 0), fill=self.fill)
        if name == "TranslateY":
            return affine(x, translate=(0, int(mag)), fill=self.fill)
        if name == "Rotate":
            return rotate(x, mag, self.fill)
        if name == "Brightness":
            return adjust_brightness(x, 1.0 + mag)
        if name == "Color":
            return adjust_saturation(x, 1.0 + mag)
        if name == "Contrast":
            return adjust_contrast(x, 1.0 + mag)
        if name == "Sharpness":
            return adjust_sharpness(x, 1.0 + mag)
        if name == "Posterize":
            return posterize(x, int(mag))
        if name == "Solarize":
            return solarize(x, mag)
        if name == "AutoContrast":
            return autocontrast(x)
        if name == "Equalize":
            return equalize(x)
        return x

    def forward(self, x):
        space = self._space()
        name = list(space)[_randint(0, len(space) - 1)]
        mags, signed = space[name]
        mag = float(mags[_randint(0, self.bins - 1)]) if mags is not None else 0.0
        if signed and _rand() < 0.5:
            mag = -mag
        return self.apply_op(x, name, mag)


def equalize(x: torch.Tensor) -> torch.Tensor:
    """Histogram equalisation per channel on the 8-bit levels of the image."""
    xb, squeeze = _batched(x)
    q = (xb * 255).round().clamp(0, 255).to(torch.int64)
    out = torch.empty_like(xb)
    for b in range(q.shape[0]):
        for c in range(q.shape[1]):
            ch = q[b, c]
            hist = torch.bincount(ch.flatten(), minlength=256)
            nz = hist[hist != 0]
            step = torch.div(nz[:-1].sum(), 255, rounding_mode="floor") if len(nz) else torch.tensor(0)
            if int(step) == 0:
                out[b, c] = xb[b, c]
                continue
            lut = torch.div(torch.cumsum(hist, 0) + torch.div(step, 2, rounding_mode="floor"), step, rounding_mode="floor")
            lut = tF.pad(lut, (1, 0))[:-1].clamp(0, 255)
            out[b, c] = lut[ch].to(xb.dtype) / 255
    return out[0] if squeeze else out
