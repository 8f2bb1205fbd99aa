"""ResNet-18 / 34 / 50 (ferrotorch-vision/src/models/resnet.rs:325 ``Bottleneck``, :565 ``ResNet``,
:1071 ``resnet50``) and a small model registry (models/registry.rs).

Convolutions are ``nn.Conv2d`` modules re-classed to :class:`ops.conv.IgemmConv2d`: on a GPU with
bf16 activations their forward and all three gradients run on this library's tcgen05 GEMM kernels
(1 x 1 as plain GEMMs, k x k in the shifted-row form, the 3-channel stem through an im2col
matrix; ``ops/conv.py``), the max pool on the NHWC kernel of ``ops/pool.py``; every batch norm
runs fused with the ReLU and the residual add that follow it (``ops/batchnorm.py``: two reads and one write of the activation
in the forward, no stored ReLU mask); the data-parallel gradient exchange and the SGD update run
through the fused ``ft_ddp_reduce_update`` kernel when trained with ``FlatTrainer`` + ``FusedDDP``.  State-dict
keys match torchvision's (``conv1.weight``, ``layer1.0.conv1.weight``, ``fc.weight`` ...).
"""
from __future__ import annotations

import torch
from torch import nn

from ..ops.batchnorm import batch_norm_act as _bn
from ..ops.conv import convert_convs as _convert_convs
from ..ops.pool import MaxPool2d as _MaxPool2d


def _downsample(seq: nn.Sequential, x: torch.Tensor) -> torch.Tensor:
    """The projection shortcut ``Sequential(conv, bn)`` with the fused batch norm (no ReLU)."""
    if len(seq) == 2 and isinstance(seq[1], nn.BatchNorm2d):
        return _bn(seq[0](x), seq[1], relu=False)
    return seq(x)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, inplanes, planes, stride=1, downsample=None, dilation=1):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 3, stride, dilation, dilation=dilation, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.relu = nn.ReLU(inplace=True)
        self.conv2 = nn.Conv2d(planes, planes, 3, 1, dilation, dilation=dilation, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else _downsample(self.downsample, x)
        out = _bn(self.conv1(x), self.bn1)
        return _bn(self.conv2(out), self.bn2, residual=idt)


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, dilation=1):
        super().__init__()
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride, dilation, dilation=dilation, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv3 = nn.Conv2d(planes, planes * 4, 1, bias=False)
        self.bn3 = nn.BatchNorm2d(planes * 4)
        self.relu = nn.ReLU(inplace=True)
        self.downsample = downsample

    def forward(self, x):
        idt = x if self.downsample is None else _downsample(self.downsample, x)
        out = _bn(self.conv1(x), self.bn1)
        out = _bn(self.conv2(out), self.bn2)
        return _bn(self.conv3(out), self.bn3, residual=idt)


class ResNet(nn.Module):
    def __init__(self, block, layers, num_classes: int = 1000, replace_stride_with_dilation=(False, False, False),
                 zero_init_residual: bool = False):
        super().__init__()
        self.inplanes, self.dilation = 64, 1
        self.conv1 = nn.Conv2d(3, 64, 7, 2, 3, bias=False)
        self.bn1 = nn.BatchNorm2d(64)
        self.relu = nn.ReLU(inplace=True)
        self.maxpool = _MaxPool2d(3, 2, 1)
        self.layer1 = self._make_layer(block, 64, layers[0])
        self.layer2 = self._make_layer(block, 128, layers[1], 2, replace_stride_with_dilation[0])
        self.layer3 = self._make_layer(block, 256, layers[2], 2, replace_stride_with_dilation[1])
        self.layer4 = self._make_layer(block, 512, layers[3], 2, replace_stride_with_dilation[2])
        self.avgpool = nn.AdaptiveAvgPool2d(1)
        self.fc = nn.Linear(512 * block.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.ones_(m.weight)
                nn.init.zeros_(m.bias)
        if zero_init_residual:
            for m in self.modules():
                if isinstance(m, Bottleneck):
                    nn.init.zeros_(m.bn3.weight)
                elif isinstance(m, BasicBlock):
                    nn.init.zeros_(m.bn2.weight)
        _convert_convs(self)     # same parameters and state-dict keys; forward through ops.conv.conv2d

    def _make_layer(self, block, planes, blocks, stride=1, dilate=False):
        prev_dilation = self.dilation
        if dilate:
            self.dilation *= stride
            stride = 1
        down = None
        if stride != 1 or self.inplanes != planes * block.expansion:
            down = nn.Sequential(nn.Conv2d(self.inplanes, planes * block.expansion, 1, stride, bias=False),
                                 nn.BatchNorm2d(planes * block.expansion))
        layers = [block(self.inplanes, planes, stride, down, prev_dilation)]
        self.inplanes = planes * block.expansion
        layers += [block(self.inplanes, planes, dilation=self.dilation) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        x = self.maxpool(_bn(self.conv1(x), self.bn1))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


def resnet18(**kw):
    return ResNet(BasicBlock, [2, 2, 2, 2], **kw)


def resnet34(**kw):
    return ResNet(BasicBlock, [3, 4, 6, 3], **kw)


def resnet50(**kw):
    return ResNet(Bottleneck, [3, 4, 6, 3], **kw)


_REGISTRY = {"resnet18": resnet18, "resnet34": resnet34, "resnet50": resnet50}


def register_model(name: str, ctor) -> None:
    _REGISTRY[name] = ctor


def list_models() -> list[str]:
    return sorted(_REGISTRY)


def create_model(name: str, **kw) -> nn.Module:
    """Registry lookup for the ResNet family and anything added with :func:`register_model`
    (``vision.build`` serves the other families of ferrotorch-vision/src/models from this package's
    own modules and only then falls back to this function); a name unknown here is finally tried
    as a torchvision constructor name."""
    if name in _REGISTRY:
        return _REGISTRY[name](**kw)
    try:
        import torchvision.models as tvm

        return tvm.get_model(name, weights=None, **kw)
    except Exception as e:  # noqa: BLE001
        raise KeyError("unknown model %r (registered: %s)" % (name, list_models())) from e


# --------------------------------------------------------------------------- inference: batch norm folded into the convolutions
def fold_conv_bn(conv: nn.Conv2d, bn: nn.BatchNorm2d):
    """``(weight, bias)`` of the convolution that computes ``bn(conv(x))`` with the norm's running
    statistics: ``w' = w * g / sqrt(var + eps)`` per output channel, ``b' = beta + (b - mean) * g / sqrt(var + eps)``."""
    scale = (bn.weight if bn.weight is not None else torch.ones_like(bn.running_var)).float() / torch.sqrt(bn.running_var.float() + bn.eps)
    w = conv.weight.float() * scale.view(-1, 1, 1, 1)
    b0 = conv.bias.float() if conv.bias is not None else torch.zeros_like(bn.running_mean).float()
    b = (bn.bias.float() if bn.bias is not None else 0.0) + (b0 - bn.running_mean.float()) * scale
    return w.to(conv.weight.dtype), b.to(conv.weight.dtype)


class _FoldedConv(nn.Module):
    """A convolution with its batch norm folded in; ``forward(x, residual, relu)`` is one call of
    ``ops.conv.conv2d`` (the implicit-GEMM kernel with bias / residual / ReLU in its epilogue when
    that kernel is switched on and takes the shape; ``torch.nn.functional.conv2d`` otherwise)."""

    def __init__(self, conv: nn.Conv2d, bn: nn.BatchNorm2d):
        super().__init__()
        w, b = fold_conv_bn(conv, bn)
        self.weight = nn.Parameter(w.contiguous(memory_format=torch.channels_last), requires_grad=False)
        self.bias = nn.Parameter(b, requires_grad=False)
        self.stride, self.padding, self.dilation, self.groups = conv.stride, conv.padding, conv.dilation, conv.groups

    def forward(self, x, residual=None, relu: bool = False):
        from ..ops.conv import conv2d

        return conv2d(x, self.weight, self.bias, self.stride, self.padding, self.dilation, self.groups, residual, relu)


class _FusedBlock(nn.Module):
    def __init__(self, block):
        super().__init__()
        names = ("conv1", "conv2", "conv3") if isinstance(block, Bottleneck) else ("conv1", "conv2")
        self.convs = nn.ModuleList(_FoldedConv(getattr(block, n), getattr(block, n.replace("conv", "bn"))) for n in names)
        d = block.downsample
        self.down = _FoldedConv(d[0], d[1]) if d is not None else None

    def forward(self, x):
        idt = x if self.down is None else self.down(x)
        out = x
        for c in self.convs[:-1]:
            out = c(out, relu=True)
        return self.convs[-1](out, residual=idt, relu=True)


class FusedInferenceResNet(nn.Module):
    """A trained :class:`ResNet` rewritten for inference: every batch norm is folded into the
    convolution in front of it, so a block is two or three convolution calls whose epilogues add
    the bias, the shortcut and apply the ReLU -- no separate normalisation, add or activation pass
    over the activations.  Weights are copies: the source model is left as it was."""

    def __init__(self, model: ResNet):
        super().__init__()
        if model.training:
            raise ValueError("FusedInferenceResNet: call model.eval() first (folding uses the running statistics)")
        self.stem = _FoldedConv(model.conv1, model.bn1)
        from ..ops.pool import MaxPool2d

        mp = model.maxpool
        self.maxpool = MaxPool2d(mp.kernel_size, mp.stride, mp.padding)     # the NHWC kernel when switched on, torch otherwise
        self.avgpool, self.fc = model.avgpool, model.fc
        self.blocks = nn.Sequential(*[_FusedBlock(b) for layer in (model.layer1, model.layer2, model.layer3, model.layer4)
                                      for b in layer])

    @torch.no_grad()
    def forward(self, x):
        x = self.blocks(self.maxpool(self.stem(x, relu=True)))
        return self.fc(torch.flatten(self.avgpool(x), 1))


def fuse_for_inference(model: ResNet) -> FusedInferenceResNet:
    return FusedInferenceResNet(model)
