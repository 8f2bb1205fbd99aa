"""Image classifiers and segmentation heads beyond ResNet, as this package's own modules.

The reference implements these families in ``ferrotorch-vision/src/models/`` (``vgg.rs``,
``mobilenet.rs``, ``vit.rs``, ``convnext.rs``, ``densenet.rs``, ``segmentation/fcn.rs``,
``segmentation/deeplabv3.rs``, ``segmentation/aspp.rs``) with torchvision's parameter names, so
that torchvision checkpoints load.  The modules here keep those names too (the tests load a
torchvision state dict with ``strict=True`` and compare outputs), are built from ``torch.nn``
layers, and route their hot operators to this framework's kernels on a GPU with bf16
activations: every ``nn.Conv2d`` is re-classed to :class:`ops.conv.IgemmConv2d` (tcgen05 GEMM
convolutions), the vision transformer's attention runs on the flash-attention kernel, the
segmentation models sit on this package's own :class:`models.resnet.ResNet`.
"""
from __future__ import annotations

import torch
import torch.nn.functional as tF
from torch import nn

from ..ops.conv import convert_convs
from .resnet import ResNet, resnet50


def _conv_bn_act(cin, cout, k=3, stride=1, groups=1, act=nn.ReLU6, dilation=1):
    """``Sequential(conv, bn, act)`` with the layout (and key names ``0`` / ``1``) of torchvision's
    ``Conv2dNormActivation``."""
    pad = (k - 1) // 2 * dilation
    layers = [nn.Conv2d(cin, cout, k, stride, pad, dilation=dilation, groups=groups, bias=False), nn.BatchNorm2d(cout)]
    if act is not None:
        layers.append(act(inplace=True))
    return nn.Sequential(*layers)


# --------------------------------------------------------------------------- VGG
_VGG_CFG = {"A": [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
            "D": [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"]}


class VGG(nn.Module):
    def __init__(self, cfg: str = "D", batch_norm: bool = False, num_classes: int = 1000, dropout: float = 0.5):
        super().__init__()
        layers, cin = [], 3
        for v in _VGG_CFG[cfg]:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                layers.append(nn.Conv2d(cin, v, 3, padding=1))
                if batch_norm:
                    layers.append(nn.BatchNorm2d(v))
                layers.append(nn.ReLU(inplace=True))
                cin = v
        self.features = nn.Sequential(*layers)
        self.avgpool = nn.AdaptiveAvgPool2d(7)
        self.classifier = nn.Sequential(nn.Linear(512 * 49, 4096), nn.ReLU(True), nn.Dropout(dropout),
                                        nn.Linear(4096, 4096), nn.ReLU(True), nn.Dropout(dropout),
                                        nn.Linear(4096, num_classes))
        convert_convs(self)

    def forward(self, x):
        return self.classifier(torch.flatten(self.avgpool(self.features(x)), 1))


def vgg11(**kw):
    return VGG("A", **kw)


def vgg16(**kw):
    return VGG("D", **kw)


# --------------------------------------------------------------------------- MobileNetV2
class InvertedResidual(nn.Module):
    def __init__(self, cin, cout, stride, expand):
        super().__init__()
        hidden = int(round(cin * expand))
        self.use_res = stride == 1 and cin == cout
        layers = []
        if expand != 1:
            layers.append(_conv_bn_act(cin, hidden, 1))
        layers += [_conv_bn_act(hidden, hidden, 3, stride, groups=hidden), nn.Conv2d(hidden, cout, 1, bias=False),
                   nn.BatchNorm2d(cout)]
        self.conv = nn.Sequential(*layers)

    def forward(self, x):
        return x + self.conv(x) if self.use_res else self.conv(x)


class MobileNetV2(nn.Module):
    SETTINGS = [[1, 16, 1, 1], [6, 24, 2, 2], [6, 32, 3, 2], [6, 64, 4, 2], [6, 96, 3, 1], [6, 160, 3, 2], [6, 320, 1, 1]]

    def __init__(self, num_classes: int = 1000, dropout: float = 0.2):
        super().__init__()
        feats, cin = [_conv_bn_act(3, 32, 3, 2)], 32
        for t, c, n, s in self.SETTINGS:
            for i in range(n):
                feats.append(InvertedResidual(cin, c, s if i == 0 else 1, t))
                cin = c
        feats.append(_conv_bn_act(cin, 1280, 1))
        self.features = nn.Sequential(*feats)
        self.classifier = nn.Sequential(nn.Dropout(dropout), nn.Linear(1280, num_classes))
        convert_convs(self)

    def forward(self, x):
        x = self.features(x)
        return self.classifier(torch.flatten(tF.adaptive_avg_pool2d(x, 1), 1))


def mobilenet_v2(**kw):
    return MobileNetV2(**kw)


# --------------------------------------------------------------------------- Vision transformer
class SelfAttention(nn.Module):
    """Multi-head self-attention with ``nn.MultiheadAttention``'s parameter names
    (``in_proj_weight``, ``in_proj_bias``, ``out_proj``).  CUDA bf16 inputs with a head size of 64 or
    128 run on the flash-attention kernel; everything else on ``scaled_dot_product_attention``."""

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.in_proj_weight = nn.Parameter(torch.empty(3 * dim, dim))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * dim))
        self.out_proj = nn.Linear(dim, dim)
        nn.init.xavier_uniform_(self.in_proj_weight)

    def forward(self, x):
        B, S, E = x.shape
        hd = E // self.heads
        qkv = tF.linear(x, self.in_proj_weight, self.in_proj_bias).view(B, S, 3, self.heads, hd)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]              # [B, S, H, hd]
        if x.is_cuda and x.dtype == torch.bfloat16 and hd in (64, 128):
            from ..ops.attention import flash_attention

            o = flash_attention(q.contiguous(), k.contiguous(), v.contiguous(), causal=False)
        else:
            o = tF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        return self.out_proj(o.reshape(B, S, E))


class EncoderBlock(nn.Module):
    def __init__(self, dim, heads, mlp_dim, dropout=0.0):
        super().__init__()
        self.ln_1 = nn.LayerNorm(dim, eps=1e-6)
        self.self_attention = SelfAttention(dim, heads)
        self.dropout = nn.Dropout(dropout)
        self.ln_2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = nn.Sequential(nn.Linear(dim, mlp_dim), nn.GELU(), nn.Dropout(dropout), nn.Linear(mlp_dim, dim),
                                 nn.Dropout(dropout))

    def forward(self, x):
        x = x + self.dropout(self.self_attention(self.ln_1(x)))
        return x + self.mlp(self.ln_2(x))


class _Encoder(nn.Module):
    def __init__(self, seq_len, layers, heads, dim, mlp_dim, dropout):
        super().__init__()
        self.pos_embedding = nn.Parameter(torch.empty(1, seq_len, dim).normal_(std=0.02))
        self.dropout = nn.Dropout(dropout)
        self.layers = nn.Sequential()
        for i in range(layers):
            self.layers.add_module("encoder_layer_%d" % i, EncoderBlock(dim, heads, mlp_dim, dropout))
        self.ln = nn.LayerNorm(dim, eps=1e-6)

    def forward(self, x):
        return self.ln(self.layers(self.dropout(x + self.pos_embedding)))


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch_size=16, num_layers=12, num_heads=12, hidden_dim=768, mlp_dim=3072,
                 num_classes=1000, dropout=0.0):
        super().__init__()
        assert image_size % patch_size == 0
        self.image_size, self.patch_size, self.hidden_dim = image_size, patch_size, hidden_dim
        self.conv_proj = nn.Conv2d(3, hidden_dim, patch_size, patch_size)
        self.class_token = nn.Parameter(torch.zeros(1, 1, hidden_dim))
        self.encoder = _Encoder((image_size // patch_size) ** 2 + 1, num_layers, num_heads, hidden_dim, mlp_dim, dropout)
        self.heads = nn.Sequential()
        self.heads.add_module("head", nn.Linear(hidden_dim, num_classes))

    def forward(self, x):
        B = x.shape[0]
        x = self.conv_proj(x).flatten(2).transpose(1, 2)                 # [B, patches, dim]
        x = torch.cat([self.class_token.expand(B, -1, -1).to(x.dtype), x], dim=1)
        return self.heads(self.encoder(x)[:, 0])


def vit_b_16(**kw):
    return VisionTransformer(**kw)


# --------------------------------------------------------------------------- ConvNeXt
class LayerNorm2d(nn.LayerNorm):
    """LayerNorm over the channel dimension of an NCHW tensor."""

    def forward(self, x):
        return tF.layer_norm(x.permute(0, 2, 3, 1), self.normalized_shape, self.weight, self.bias, self.eps).permute(0, 3, 1, 2)


class _Permute(nn.Module):
    def __init__(self, dims):
        super().__init__()
        self.dims = dims

    def forward(self, x):
        return x.permute(*self.dims)


class CNBlock(nn.Module):
    def __init__(self, dim, layer_scale=1e-6):
        super().__init__()
        self.block = nn.Sequential(nn.Conv2d(dim, dim, 7, padding=3, groups=dim), _Permute([0, 2, 3, 1]),
                                   nn.LayerNorm(dim, eps=1e-6), nn.Linear(dim, 4 * dim), nn.GELU(),
                                   nn.Linear(4 * dim, dim), _Permute([0, 3, 1, 2]))
        self.layer_scale = nn.Parameter(torch.ones(dim, 1, 1) * layer_scale)

    def forward(self, x):
        return x + self.layer_scale * self.block(x)


class ConvNeXt(nn.Module):
    def __init__(self, depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), num_classes=1000):
        super().__init__()
        feats = [nn.Sequential(nn.Conv2d(3, dims[0], 4, 4), LayerNorm2d(dims[0], eps=1e-6))]
        for i, (d, c) in enumerate(zip(depths, dims)):
            feats.append(nn.Sequential(*[CNBlock(c) for _ in range(d)]))
            if i + 1 < len(dims):
                feats.append(nn.Sequential(LayerNorm2d(c, eps=1e-6), nn.Conv2d(c, dims[i + 1], 2, 2)))
        self.features = nn.Sequential(*feats)
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.classifier = nn.Sequential(LayerNorm2d(dims[-1], eps=1e-6), nn.Flatten(1), nn.Linear(dims[-1], num_classes))
        convert_convs(self)

    def forward(self, x):
        return self.classifier(self.avgpool(self.features(x)))


def convnext_tiny(**kw):
    return ConvNeXt(**kw)


# --------------------------------------------------------------------------- DenseNet
class _DenseLayer(nn.Module):
    def __init__(self, cin, growth, bn_size):
        super().__init__()
        self.norm1, self.relu1 = nn.BatchNorm2d(cin), nn.ReLU(inplace=True)
        self.conv1 = nn.Conv2d(cin, bn_size * growth, 1, bias=False)
        self.norm2, self.relu2 = nn.BatchNorm2d(bn_size * growth), nn.ReLU(inplace=True)
        self.conv2 = nn.Conv2d(bn_size * growth, growth, 3, padding=1, bias=False)

    def forward(self, feats: list):
        x = self.conv1(self.relu1(self.norm1(torch.cat(feats, 1))))
        return self.conv2(self.relu2(self.norm2(x)))


class _DenseBlock(nn.ModuleDict):
    def __init__(self, n, cin, growth, bn_size):
        super().__init__()
        for i in range(n):
            self["denselayer%d" % (i + 1)] = _DenseLayer(cin + i * growth, growth, bn_size)

    def forward(self, x):
        feats = [x]
        for layer in self.values():
            feats.append(layer(feats))
        return torch.cat(feats, 1)


class DenseNet(nn.Module):
    def __init__(self, growth=32, blocks=(6, 12, 24, 16), init_features=64, bn_size=4, num_classes=1000):
        super().__init__()
        f = nn.Sequential()
        f.add_module("conv0", nn.Conv2d(3, init_features, 7, 2, 3, bias=False))
        f.add_module("norm0", nn.BatchNorm2d(init_features))
        f.add_module("relu0", nn.ReLU(inplace=True))
        f.add_module("pool0", nn.MaxPool2d(3, 2, 1))
        c = init_features
        for i, n in enumerate(blocks):
            f.add_module("denseblock%d" % (i + 1), _DenseBlock(n, c, growth, bn_size))
            c += n * growth
            if i + 1 < len(blocks):
                t = nn.Sequential()
                t.add_module("norm", nn.BatchNorm2d(c))
                t.add_module("relu", nn.ReLU(inplace=True))
                t.add_module("conv", nn.Conv2d(c, c // 2, 1, bias=False))
                t.add_module("pool", nn.AvgPool2d(2, 2))
                f.add_module("transition%d" % (i + 1), t)
                c //= 2
        f.add_module("norm5", nn.BatchNorm2d(c))
        self.features = f
        self.classifier = nn.Linear(c, num_classes)
        convert_convs(self)

    def forward(self, x):
        x = tF.relu(self.features(x), inplace=True)
        return self.classifier(torch.flatten(tF.adaptive_avg_pool2d(x, 1), 1))


def densenet121(**kw):
    return DenseNet(**kw)


# --------------------------------------------------------------------------- segmentation on the own ResNet
class _Backbone(nn.Module):
    """The ResNet trunk up to ``layer4`` (its children keep their names, so checkpoint keys are
    ``backbone.conv1.weight``, ``backbone.layer1.0...`` as with torchvision's ``IntermediateLayerGetter``)."""

    def __init__(self, net: ResNet):
        super().__init__()
        for name in ("conv1", "bn1", "relu", "maxpool", "layer1", "layer2", "layer3", "layer4"):
            setattr(self, name, getattr(net, name))

    def forward(self, x):
        from ..ops.batchnorm import batch_norm_act

        x = self.maxpool(batch_norm_act(self.conv1(x), self.bn1))
        return self.layer4(self.layer3(self.layer2(self.layer1(x))))


class FCNHead(nn.Sequential):
    def __init__(self, cin, classes):
        super().__init__(nn.Conv2d(cin, cin // 4, 3, padding=1, bias=False), nn.BatchNorm2d(cin // 4), nn.ReLU(),
                         nn.Dropout(0.1), nn.Conv2d(cin // 4, classes, 1))


class _ASPPPooling(nn.Sequential):
    def __init__(self, cin, cout):
        super().__init__(nn.AdaptiveAvgPool2d(1), nn.Conv2d(cin, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU())

    def forward(self, x):
        size = x.shape[-2:]
        for m in self:
            x = m(x)
        return tF.interpolate(x, size=size, mode="bilinear", align_corners=False)


class ASPP(nn.Module):
    def __init__(self, cin, rates=(12, 24, 36), cout=256):
        super().__init__()
        mods = [nn.Sequential(nn.Conv2d(cin, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU())]
        for r in rates:
            mods.append(nn.Sequential(nn.Conv2d(cin, cout, 3, padding=r, dilation=r, bias=False), nn.BatchNorm2d(cout), nn.ReLU()))
        mods.append(_ASPPPooling(cin, cout))
        self.convs = nn.ModuleList(mods)
        self.project = nn.Sequential(nn.Conv2d(len(mods) * cout, cout, 1, bias=False), nn.BatchNorm2d(cout), nn.ReLU(),
                                     nn.Dropout(0.5))

    def forward(self, x):
        return self.project(torch.cat([m(x) for m in self.convs], 1))


class DeepLabHead(nn.Sequential):
    def __init__(self, cin, classes, rates=(12, 24, 36)):
        super().__init__(ASPP(cin, rates), nn.Conv2d(256, 256, 3, padding=1, bias=False), nn.BatchNorm2d(256), nn.ReLU(),
                         nn.Conv2d(256, classes, 1))


class SegmentationModel(nn.Module):
    """Backbone (own ResNet-50 with dilated ``layer3`` / ``layer4``, output stride 8) + head,
    logits resized to the input; returns ``{"out": logits}`` like torchvision's models."""

    def __init__(self, head: nn.Module, backbone: ResNet | None = None):
        super().__init__()
        net = backbone or resnet50(replace_stride_with_dilation=(False, True, True))
        self.backbone = _Backbone(net)
        self.classifier = head
        convert_convs(self)

    def forward(self, x):
        size = x.shape[-2:]
        y = self.classifier(self.backbone(x))
        return {"out": tF.interpolate(y, size=size, mode="bilinear", align_corners=False)}

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    def with_atrous_rates(self, rates) -> "SegmentationModel":
        """A DeepLabV3 model with another set of dilation rates in its pyramid head (freshly initialised head,
        same backbone object): ``(6, 12, 18)`` for output stride 16, ``(12, 24, 36)`` for 8."""
        if not isinstance(self.classifier, DeepLabHead):
            raise TypeError("with_atrous_rates: this model's head is a %s, not a DeepLabV3 head" % type(self.classifier).__name__)
        classes = self.classifier[-1].out_channels
        out = SegmentationModel.__new__(SegmentationModel)
        nn.Module.__init__(out)
        out.backbone, out.classifier = self.backbone, DeepLabHead(2048, classes, tuple(rates))
        convert_convs(out.classifier)
        return out


def fcn_resnet50(num_classes: int = 21, **kw):
    return SegmentationModel(FCNHead(2048, num_classes), **kw)


def deeplabv3_resnet50(num_classes: int = 21, **kw):
    return SegmentationModel(DeepLabHead(2048, num_classes), **kw)


OWN_MODELS = {"vgg11": vgg11, "vgg16": vgg16, "mobilenet_v2": mobilenet_v2, "vit_b_16": vit_b_16,
              "convnext_tiny": convnext_tiny, "densenet121": densenet121, "fcn": fcn_resnet50, "fcn_resnet50": fcn_resnet50,
              "deeplabv3": deeplabv3_resnet50, "deeplabv3_resnet50": deeplabv3_resnet50}
