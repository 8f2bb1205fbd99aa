"""EfficientNet-B0, MobileNetV3, Inception v3, Swin-T and the LRASPP segmentation head as this
package's own modules.

The reference implements them in ``ferrotorch-vision/src/models/`` (``efficientnet.rs``,
``mobilenet.rs``, ``inception.rs``, ``swin.rs``, ``segmentation/lraspp.rs``) with torchvision's
parameter names so that torchvision checkpoints load; the modules here keep those names (the
tests load a torchvision state dict with ``strict=True`` and compare outputs).  Dense
convolutions are re-classed to :class:`ops.conv.IgemmConv2d` (tcgen05 GEMM convolutions on a
GPU with bf16 activations; depthwise ones stay on the library path), and window attention runs on
``scaled_dot_product_attention`` with the relative-position bias as its additive mask.
"""
from __future__ import annotations

import math
from functools import partial

import torch
import torch.nn.functional as tF
from torch import nn

from ..ops.conv import convert_convs


def _make_divisible(v: float, divisor: int = 8) -> int:
    new = max(divisor, int(v + divisor / 2) // divisor * divisor)
    return new + divisor if new < 0.9 * v else new


def _cna(cin, cout, k=3, stride=1, groups=1, act=nn.ReLU, norm=nn.BatchNorm2d, dilation=1):
    """``Sequential(conv, norm, act)``: the layout and key names of torchvision's ``Conv2dNormActivation``."""
    layers = [nn.Conv2d(cin, cout, k, stride, (k - 1) // 2 * dilation, dilation=dilation, groups=groups, bias=False),
              norm(cout)]
    if act is not None:
        layers.append(act(inplace=True) if act is not nn.GELU else act())
    return nn.Sequential(*layers)


class SqueezeExcitation(nn.Module):
    """Channel gate: global mean -> fc1 -> act -> fc2 -> gate (1 x 1 convolutions ``fc1`` / ``fc2``)."""

    def __init__(self, channels: int, squeeze: int, act=nn.ReLU, gate=nn.Sigmoid):
        super().__init__()
        self.fc1, self.fc2 = nn.Conv2d(channels, squeeze, 1), nn.Conv2d(squeeze, channels, 1)
        self.act, self.gate = act(), gate()

    def forward(self, x):
        s = self.gate(self.fc2(self.act(self.fc1(x.mean((2, 3), keepdim=True)))))
        return x * s


def _drop_path(x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    """Stochastic depth, one draw per sample."""
    if not training or p == 0.0:
        return x
    keep = torch.empty((x.shape[0],) + (1,) * (x.dim() - 1), device=x.device, dtype=x.dtype).bernoulli_(1 - p)
    return x * keep / (1 - p)


# --------------------------------------------------------------------------- EfficientNet
class MBConv(nn.Module):
    def __init__(self, cin, cout, k, stride, expand, sd_prob):
        super().__init__()
        self.use_res, self.sd_prob = stride == 1 and cin == cout, sd_prob
        hidden = _make_divisible(cin * expand)
        act = nn.SiLU
        layers = []
        if hidden != cin:
            layers.append(_cna(cin, hidden, 1, act=act))
        layers += [_cna(hidden, hidden, k, stride, groups=hidden, act=act),
                   SqueezeExcitation(hidden, max(1, cin // 4), act=partial(nn.SiLU, inplace=True)),
                   _cna(hidden, cout, 1, act=None)]
        self.block = nn.Sequential(*layers)

    def forward(self, x):
        y = self.block(x)
        return x + _drop_path(y, self.sd_prob, self.training) if self.use_res else y


class EfficientNet(nn.Module):
    # expand, kernel, stride, in, out, layers  (B0; width / depth multipliers scale the last three)
    B0 = [(1, 3, 1, 32, 16, 1), (6, 3, 2, 16, 24, 2), (6, 5, 2, 24, 40, 2), (6, 3, 2, 40, 80, 3), (6, 5, 1, 80, 112, 3),
          (6, 5, 2, 112, 192, 4), (6, 3, 1, 192, 320, 1)]

    def __init__(self, width: float = 1.0, depth: float = 1.0, dropout: float = 0.2, num_classes: int = 1000,
                 stochastic_depth_prob: float = 0.2):
        super().__init__()
        ch = lambda c: _make_divisible(c * width)  # noqa: E731
        cfg = [(e, k, s, ch(i), ch(o), int(math.ceil(n * depth))) for e, k, s, i, o, n in self.B0]
        total, done = sum(c[-1] for c in cfg), 0
        feats = [_cna(3, cfg[0][3], 3, 2, act=nn.SiLU)]
        for e, k, s, cin, cout, n in cfg:
            stage = []
            for j in range(n):
                stage.append(MBConv(cin if j == 0 else cout, cout, k, s if j == 0 else 1, e,
                                    stochastic_depth_prob * done / total))
                done += 1
            feats.append(nn.Sequential(*stage))
        last = cfg[-1][4]
        feats.append(_cna(last, 4 * last, 1, act=nn.SiLU))
        self.features = nn.Sequential(*feats)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Sequential(nn.Dropout(dropout, inplace=True), nn.Linear(4 * last, num_classes))
        convert_convs(self)

    def forward(self, x):
        return self.classifier(torch.flatten(self.avgpool(self.features(x)), 1))


def efficientnet_b0(**kw):
    return EfficientNet(1.0, 1.0, 0.2, **kw)


# --------------------------------------------------------------------------- MobileNetV3
class InvertedResidualV3(nn.Module):
    def __init__(self, cin, k, hidden, cout, use_se, act, stride, dilation, norm):
        super().__init__()
        self.use_res = stride == 1 and cin == cout
        self.out_channels, self._is_cn = cout, stride > 1
        a = nn.Hardswish if act == "HS" else nn.ReLU
        layers = []
        if hidden != cin:
            layers.append(_cna(cin, hidden, 1, act=a, norm=norm))
        layers.append(_cna(hidden, hidden, k, 1 if dilation > 1 else stride, groups=hidden, act=a, norm=norm, dilation=dilation))
        if use_se:
            layers.append(SqueezeExcitation(hidden, _make_divisible(hidden // 4), gate=nn.Hardsigmoid))
        layers.append(_cna(hidden, cout, 1, act=None, norm=norm))
        self.block = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.block(x) if self.use_res else self.block(x)


def _v3_settings(arch: str, dilated: bool = False, reduced_tail: bool = False):
    r, d = (2 if reduced_tail else 1), (2 if dilated else 1)
    if arch == "large":
        rows = [(16, 3, 16, 16, False, "RE", 1, 1), (16, 3, 64, 24, False, "RE", 2, 1), (24, 3, 72, 24, False, "RE", 1, 1),
                (24, 5, 72, 40, True, "RE", 2, 1), (40, 5, 120, 40, True, "RE", 1, 1), (40, 5, 120, 40, True, "RE", 1, 1),
                (40, 3, 240, 80, False, "HS", 2, 1), (80, 3, 200, 80, False, "HS", 1, 1), (80, 3, 184, 80, False, "HS", 1, 1),
                (80, 3, 184, 80, False, "HS", 1, 1), (80, 3, 480, 112, True, "HS", 1, 1), (112, 3, 672, 112, True, "HS", 1, 1),
                (112, 5, 672, 160 // r, True, "HS", 2, d), (160 // r, 5, 960 // r, 160 // r, True, "HS", 1, d),
                (160 // r, 5, 960 // r, 160 // r, True, "HS", 1, d)]
        return rows, 1280 // r
    rows = [(16, 3, 16, 16, True, "RE", 2, 1), (16, 3, 72, 24, False, "RE", 2, 1), (24, 3, 88, 24, False, "RE", 1, 1),
            (24, 5, 96, 40, True, "HS", 2, 1), (40, 5, 240, 40, True, "HS", 1, 1), (40, 5, 240, 40, True, "HS", 1, 1),
            (40, 5, 120, 48, True, "HS", 1, 1), (48, 5, 144, 48, True, "HS", 1, 1), (48, 5, 288, 96 // r, True, "HS", 2, d),
            (96 // r, 5, 576 // r, 96 // r, True, "HS", 1, d), (96 // r, 5, 576 // r, 96 // r, True, "HS", 1, d)]
    return rows, 1024 // r


class MobileNetV3(nn.Module):
    def __init__(self, arch: str = "large", num_classes: int = 1000, dropout: float = 0.2, dilated: bool = False,
                 reduced_tail: bool = False):
        super().__init__()
        rows, last_channel = _v3_settings(arch, dilated, reduced_tail)
        norm = partial(nn.BatchNorm2d, eps=0.001, momentum=0.01)
        feats = [_cna(3, rows[0][0], 3, 2, act=nn.Hardswish, norm=norm)]
        feats += [InvertedResidualV3(*row, norm=norm) for row in rows]
        cin = rows[-1][3]
        feats.append(_cna(cin, 6 * cin, 1, act=nn.Hardswish, norm=norm))
        self.features = nn.Sequential(*feats)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Sequential(nn.Linear(6 * cin, last_channel), nn.Hardswish(inplace=True),
                                        nn.Dropout(dropout, inplace=True), nn.Linear(last_channel, num_classes))
        convert_convs(self)

    def forward(self, x):
        return self.classifier(torch.flatten(self.avgpool(self.features(x)), 1))


def mobilenet_v3_large(**kw):
    return MobileNetV3("large", **kw)


def mobilenet_v3_small(**kw):
    return MobileNetV3("small", **kw)


# --------------------------------------------------------------------------- LRASPP
class LRASPPHead(nn.Module):
    def __init__(self, low_channels, high_channels, num_classes, inter_channels=128):
        super().__init__()
        self.cbr = nn.Sequential(nn.Conv2d(high_channels, inter_channels, 1, bias=False), nn.BatchNorm2d(inter_channels),
                                 nn.ReLU(inplace=True))
        self.scale = nn.Sequential(nn.AdaptiveAvgPool2d(1), nn.Conv2d(high_channels, inter_channels, 1, bias=False),
                                   nn.Sigmoid())
        self.low_classifier = nn.Conv2d(low_channels, num_classes, 1)
        self.high_classifier = nn.Conv2d(inter_channels, num_classes, 1)

    def forward(self, low, high):
        x = self.cbr(high) * self.scale(high)
        x = tF.interpolate(x, size=low.shape[-2:], mode="bilinear", align_corners=False)
        return self.low_classifier(low) + self.high_classifier(x)


class LRASPP(nn.Module):
    """Lite R-ASPP on a dilated MobileNetV3-Large: the 1/8-resolution features (40 channels) and the
    last features (960 channels) feed the head; the result is resized to the input."""

    def __init__(self, num_classes: int = 21, inter_channels: int = 128):
        super().__init__()
        feats = MobileNetV3("large", dilated=True).features
        stages = [0] + [i for i, b in enumerate(feats) if getattr(b, "_is_cn", False)] + [len(feats) - 1]
        self.low_pos, self.high_pos = stages[-4], stages[-1]
        self.backbone = nn.Sequential(*list(feats.children())[: self.high_pos + 1])
        self.classifier = LRASPPHead(feats[self.low_pos].out_channels, feats[self.high_pos][0].out_channels, num_classes,
                                     inter_channels)
        convert_convs(self)

    def forward(self, x):
        size, low = x.shape[-2:], None
        for i, layer in enumerate(self.backbone):
            x = layer(x)
            if i == self.low_pos:
                low = x
        out = self.classifier(low, x)
        return {"out": tF.interpolate(out, size=size, mode="bilinear", align_corners=False)}


def lraspp_mobilenet_v3_large(num_classes: int = 21, **kw):
    return LRASPP(num_classes, **kw)


# --------------------------------------------------------------------------- Inception v3
class BasicConv2d(nn.Module):
    def __init__(self, cin, cout, **kw):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, bias=False, **kw)
        self.bn = nn.BatchNorm2d(cout, eps=0.001)

    def forward(self, x):
        return tF.relu(self.bn(self.conv(x)), inplace=True)


class InceptionA(nn.Module):
    def __init__(self, cin, pool_features):
        super().__init__()
        self.branch1x1 = BasicConv2d(cin, 64, kernel_size=1)
        self.branch5x5_1 = BasicConv2d(cin, 48, kernel_size=1)
        self.branch5x5_2 = BasicConv2d(48, 64, kernel_size=5, padding=2)
        self.branch3x3dbl_1 = BasicConv2d(cin, 64, kernel_size=1)
        self.branch3x3dbl_2 = BasicConv2d(64, 96, kernel_size=3, padding=1)
        self.branch3x3dbl_3 = BasicConv2d(96, 96, kernel_size=3, padding=1)
        self.branch_pool = BasicConv2d(cin, pool_features, kernel_size=1)

    def forward(self, x):
        return torch.cat([self.branch1x1(x), self.branch5x5_2(self.branch5x5_1(x)),
                          self.branch3x3dbl_3(self.branch3x3dbl_2(self.branch3x3dbl_1(x))),
                          self.branch_pool(tF.avg_pool2d(x, 3, 1, 1))], 1)


class InceptionB(nn.Module):
    def __init__(self, cin):
        super().__init__()
        self.branch3x3 = BasicConv2d(cin, 384, kernel_size=3, stride=2)
        self.branch3x3dbl_1 = BasicConv2d(cin, 64, kernel_size=1)
        self.branch3x3dbl_2 = BasicConv2d(64, 96, kernel_size=3, padding=1)
        self.branch3x3dbl_3 = BasicConv2d(96, 96, kernel_size=3, stride=2)

    def forward(self, x):
        return torch.cat([self.branch3x3(x), self.branch3x3dbl_3(self.branch3x3dbl_2(self.branch3x3dbl_1(x))),
                          tF.max_pool2d(x, 3, 2)], 1)


class InceptionC(nn.Module):
    def __init__(self, cin, c7):
        super().__init__()
        self.branch1x1 = BasicConv2d(cin, 192, kernel_size=1)
        self.branch7x7_1 = BasicConv2d(cin, c7, kernel_size=1)
        self.branch7x7_2 = BasicConv2d(c7, c7, kernel_size=(1, 7), padding=(0, 3))
        self.branch7x7_3 = BasicConv2d(c7, 192, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_1 = BasicConv2d(cin, c7, kernel_size=1)
        self.branch7x7dbl_2 = BasicConv2d(c7, c7, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_3 = BasicConv2d(c7, c7, kernel_size=(1, 7), padding=(0, 3))
        self.branch7x7dbl_4 = BasicConv2d(c7, c7, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7dbl_5 = BasicConv2d(c7, 192, kernel_size=(1, 7), padding=(0, 3))
        self.branch_pool = BasicConv2d(cin, 192, kernel_size=1)

    def forward(self, x):
        b7 = self.branch7x7_3(self.branch7x7_2(self.branch7x7_1(x)))
        d = self.branch7x7dbl_5(self.branch7x7dbl_4(self.branch7x7dbl_3(self.branch7x7dbl_2(self.branch7x7dbl_1(x)))))
        return torch.cat([self.branch1x1(x), b7, d, self.branch_pool(tF.avg_pool2d(x, 3, 1, 1))], 1)


class InceptionD(nn.Module):
    def __init__(self, cin):
        super().__init__()
        self.branch3x3_1 = BasicConv2d(cin, 192, kernel_size=1)
        self.branch3x3_2 = BasicConv2d(192, 320, kernel_size=3, stride=2)
        self.branch7x7x3_1 = BasicConv2d(cin, 192, kernel_size=1)
        self.branch7x7x3_2 = BasicConv2d(192, 192, kernel_size=(1, 7), padding=(0, 3))
        self.branch7x7x3_3 = BasicConv2d(192, 192, kernel_size=(7, 1), padding=(3, 0))
        self.branch7x7x3_4 = BasicConv2d(192, 192, kernel_size=3, stride=2)

    def forward(self, x):
        b7 = self.branch7x7x3_4(self.branch7x7x3_3(self.branch7x7x3_2(self.branch7x7x3_1(x))))
        return torch.cat([self.branch3x3_2(self.branch3x3_1(x)), b7, tF.max_pool2d(x, 3, 2)], 1)


class InceptionE(nn.Module):
    def __init__(self, cin):
        super().__init__()
        self.branch1x1 = BasicConv2d(cin, 320, kernel_size=1)
        self.branch3x3_1 = BasicConv2d(cin, 384, kernel_size=1)
        self.branch3x3_2a = BasicConv2d(384, 384, kernel_size=(1, 3), padding=(0, 1))
        self.branch3x3_2b = BasicConv2d(384, 384, kernel_size=(3, 1), padding=(1, 0))
        self.branch3x3dbl_1 = BasicConv2d(cin, 448, kernel_size=1)
        self.branch3x3dbl_2 = BasicConv2d(448, 384, kernel_size=3, padding=1)
        self.branch3x3dbl_3a = BasicConv2d(384, 384, kernel_size=(1, 3), padding=(0, 1))
        self.branch3x3dbl_3b = BasicConv2d(384, 384, kernel_size=(3, 1), padding=(1, 0))
        self.branch_pool = BasicConv2d(cin, 192, kernel_size=1)

    def forward(self, x):
        b3 = self.branch3x3_1(x)
        b3 = torch.cat([self.branch3x3_2a(b3), self.branch3x3_2b(b3)], 1)
        d = self.branch3x3dbl_2(self.branch3x3dbl_1(x))
        d = torch.cat([self.branch3x3dbl_3a(d), self.branch3x3dbl_3b(d)], 1)
        return torch.cat([self.branch1x1(x), b3, d, self.branch_pool(tF.avg_pool2d(x, 3, 1, 1))], 1)


class InceptionAux(nn.Module):
    def __init__(self, cin, num_classes):
        super().__init__()
        self.conv0 = BasicConv2d(cin, 128, kernel_size=1)
        self.conv1 = BasicConv2d(128, 768, kernel_size=5)
        self.fc = nn.Linear(768, num_classes)

    def forward(self, x):
        x = self.conv1(self.conv0(tF.avg_pool2d(x, 5, 3)))
        return self.fc(torch.flatten(tF.adaptive_avg_pool2d(x, 1), 1))


class Inception3(nn.Module):
    """Inception v3 (299 x 299 inputs).  In training mode with ``aux_logits`` the forward returns
    ``(logits, aux_logits)``; in eval mode the logits."""

    def __init__(self, num_classes: int = 1000, aux_logits: bool = True, transform_input: bool = False, dropout: float = 0.5):
        super().__init__()
        self.aux_logits, self.transform_input = aux_logits, transform_input
        self.Conv2d_1a_3x3 = BasicConv2d(3, 32, kernel_size=3, stride=2)
        self.Conv2d_2a_3x3 = BasicConv2d(32, 32, kernel_size=3)
        self.Conv2d_2b_3x3 = BasicConv2d(32, 64, kernel_size=3, padding=1)
        self.maxpool1 = nn.MaxPool2d(3, 2)
        self.Conv2d_3b_1x1 = BasicConv2d(64, 80, kernel_size=1)
        self.Conv2d_4a_3x3 = BasicConv2d(80, 192, kernel_size=3)
        self.maxpool2 = nn.MaxPool2d(3, 2)
        self.Mixed_5b, self.Mixed_5c, self.Mixed_5d = InceptionA(192, 32), InceptionA(256, 64), InceptionA(288, 64)
        self.Mixed_6a = InceptionB(288)
        self.Mixed_6b, self.Mixed_6c = InceptionC(768, 128), InceptionC(768, 160)
        self.Mixed_6d, self.Mixed_6e = InceptionC(768, 160), InceptionC(768, 192)
        self.AuxLogits = InceptionAux(768, num_classes) if aux_logits else None
        self.Mixed_7a, self.Mixed_7b, self.Mixed_7c = InceptionD(768), InceptionE(1280), InceptionE(2048)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.dropout = nn.Dropout(dropout)
        self.fc = nn.Linear(2048, num_classes)
        convert_convs(self)

    def forward(self, x):
        if self.transform_input:   # ImageNet-normalised input -> the (x - 0.5) / 0.5 scaling of the original weights
            scale = x.new_tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1) / 0.5
            shift = (x.new_tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1) - 0.5) / 0.5
            x = x * scale + shift
        x = self.maxpool1(self.Conv2d_2b_3x3(self.Conv2d_2a_3x3(self.Conv2d_1a_3x3(x))))
        x = self.maxpool2(self.Conv2d_4a_3x3(self.Conv2d_3b_1x1(x)))
        x = self.Mixed_6a(self.Mixed_5d(self.Mixed_5c(self.Mixed_5b(x))))
        x = self.Mixed_6e(self.Mixed_6d(self.Mixed_6c(self.Mixed_6b(x))))
        aux = self.AuxLogits(x) if self.AuxLogits is not None and self.training else None
        x = self.Mixed_7c(self.Mixed_7b(self.Mixed_7a(x)))
        x = self.fc(self.dropout(torch.flatten(self.avgpool(x), 1)))
        return (x, aux) if aux is not None else x


def inception_v3(**kw):
    return Inception3(**kw)


# --------------------------------------------------------------------------- Swin transformer
def _relative_position_index(ws: int) -> torch.Tensor:
    coords = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)   # [2, ws*ws]
    rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0) + (ws - 1)
    return (rel[..., 0] * (2 * ws - 1) + rel[..., 1]).flatten()


class ShiftedWindowAttention(nn.Module):
    """Multi-head attention inside ``ws x ws`` windows of a ``[B, H, W, C]`` map, optionally after
    a cyclic shift by ``shift`` (then tokens that were not neighbours before the shift are masked
    from each other); a learned bias per relative position is added to the scores."""

    def __init__(self, dim: int, window: int, shift: int, heads: int):
        super().__init__()
        self.dim, self.ws, self.shift, self.heads = dim, window, shift, heads
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.relative_position_bias_table = nn.Parameter(torch.zeros((2 * window - 1) ** 2, heads))
        nn.init.trunc_normal_(self.relative_position_bias_table, std=0.02)
        self.register_buffer("relative_position_index", _relative_position_index(window))

    def _bias(self) -> torch.Tensor:
        n = self.ws * self.ws
        return self.relative_position_bias_table[self.relative_position_index].view(n, n, -1).permute(2, 0, 1)   # [heads, n, n]

    def forward(self, x):
        B, H, W, C = x.shape
        ws = self.ws
        pad_b, pad_r = (ws - H % ws) % ws, (ws - W % ws) % ws
        x = tF.pad(x, (0, 0, 0, pad_r, 0, pad_b))
        Hp, Wp = H + pad_b, W + pad_r
        sh = [0 if ws >= Hp else self.shift, 0 if ws >= Wp else self.shift]     # a window that covers the map needs no shift
        if sum(sh) > 0:
            x = torch.roll(x, shifts=(-sh[0], -sh[1]), dims=(1, 2))
        nH, nW = Hp // ws, Wp // ws
        win = x.view(B, nH, ws, nW, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(B * nH * nW, ws * ws, C)
        qkv = self.qkv(win).reshape(win.shape[0], ws * ws, 3, self.heads, C // self.heads).permute(2, 0, 3, 1, 4)
        mask = self._bias().unsqueeze(0)                                          # [1, heads, n, n]
        if sum(sh) > 0:
            region = x.new_zeros((Hp, Wp))
            cnt = 0
            for hs in ((0, -ws), (-ws, -sh[0]), (-sh[0], None)) if sh[0] else ((0, None),):
                for wsl in ((0, -ws), (-ws, -sh[1]), (-sh[1], None)) if sh[1] else ((0, None),):
                    region[hs[0]:hs[1], wsl[0]:wsl[1]] = cnt
                    cnt += 1
            region = region.view(nH, ws, nW, ws).permute(0, 2, 1, 3).reshape(nH * nW, ws * ws)
            diff = region.unsqueeze(1) - region.unsqueeze(2)
            amask = torch.zeros_like(diff).masked_fill(diff != 0, -100.0)        # [windows, n, n]
            mask = (mask.unsqueeze(1) + amask.view(1, nH * nW, 1, ws * ws, ws * ws)).expand(B, -1, -1, -1, -1)
            mask = mask.reshape(B * nH * nW, self.heads, ws * ws, ws * ws)
        o = tF.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], attn_mask=mask.to(qkv.dtype))
        o = self.proj(o.transpose(1, 2).reshape(win.shape[0], ws * ws, C))
        x = o.view(B, nH, nW, ws, ws, C).permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, C)
        if sum(sh) > 0:
            x = torch.roll(x, shifts=(sh[0], sh[1]), dims=(1, 2))
        return x[:, :H, :W, :].contiguous()


class SwinBlock(nn.Module):
    def __init__(self, dim, heads, window, shift, mlp_ratio=4.0, sd_prob=0.0):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-5)
        self.attn = ShiftedWindowAttention(dim, window, shift, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-5)
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), nn.GELU(), nn.Dropout(0.0),
                                 nn.Linear(int(dim * mlp_ratio), dim), nn.Dropout(0.0))
        self.sd_prob = sd_prob

    def forward(self, x):
        x = x + _drop_path(self.attn(self.norm1(x)), self.sd_prob, self.training)
        return x + _drop_path(self.mlp(self.norm2(x)), self.sd_prob, self.training)


class PatchMerging(nn.Module):
    """2 x 2 neighbouring tokens -> one token of twice the width."""

    def __init__(self, dim):
        super().__init__()
        self.reduction = nn.Linear(4 * dim, 2 * dim, bias=False)
        self.norm = nn.LayerNorm(4 * dim, eps=1e-5)

    def forward(self, x):
        H, W = x.shape[1:3]
        x = tF.pad(x, (0, 0, 0, W % 2, 0, H % 2))
        x = torch.cat([x[:, 0::2, 0::2], x[:, 1::2, 0::2], x[:, 0::2, 1::2], x[:, 1::2, 1::2]], -1)
        return self.reduction(self.norm(x))


class _ToChannelsLast(nn.Module):
    def forward(self, x):
        return x.permute(0, 2, 3, 1)


class SwinTransformer(nn.Module):
    def __init__(self, patch: int = 4, embed_dim: int = 96, depths=(2, 2, 6, 2), heads=(3, 6, 12, 24), window: int = 7,
                 mlp_ratio: float = 4.0, stochastic_depth_prob: float = 0.2, num_classes: int = 1000):
        super().__init__()
        feats = [nn.Sequential(nn.Conv2d(3, embed_dim, patch, patch), _ToChannelsLast(), nn.LayerNorm(embed_dim, eps=1e-5))]
        total, done = sum(depths), 0
        for i, (d, h) in enumerate(zip(depths, heads)):
            dim = embed_dim * 2 ** i
            blocks = []
            for j in range(d):
                blocks.append(SwinBlock(dim, h, window, 0 if j % 2 == 0 else window // 2, mlp_ratio,
                                        stochastic_depth_prob * done / (total - 1)))
                done += 1
            feats.append(nn.Sequential(*blocks))
            if i < len(depths) - 1:
                feats.append(PatchMerging(dim))
        self.features = nn.Sequential(*feats)
        width = embed_dim * 2 ** (len(depths) - 1)
        self.norm = nn.LayerNorm(width, eps=1e-5)
        self.head = nn.Linear(width, num_classes)

    def forward(self, x):
        x = self.norm(self.features(x))                 # [B, H, W, C]
        return self.head(x.mean((1, 2)))


def swin_t(**kw):
    return SwinTransformer(4, 96, (2, 2, 6, 2), (3, 6, 12, 24), 7, stochastic_depth_prob=0.2, **kw)


OWN_MODELS = {"efficientnet_b0": efficientnet_b0, "mobilenet_v3_large": mobilenet_v3_large,
              "mobilenet_v3_small": mobilenet_v3_small, "inception_v3": inception_v3, "swin_t": swin_t, "swin_tiny": swin_t,
              "lraspp": lraspp_mobilenet_v3_large, "lraspp_mobilenet_v3_large": lraspp_mobilenet_v3_large}
