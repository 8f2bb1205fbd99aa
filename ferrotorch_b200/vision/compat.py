"""The reference's ``ferrotorch-vision`` names (ferrotorch-vision/src/lib.rs re-exports: datasets,
transforms, detection / segmentation building blocks, the model registry, feature extraction).
Every name points at this package's own code: models, heads, anchors and the feature extractor
(``models/detection.py``, ``models/vision_zoo.py``, ``ops/det_ops.py``), the dataset readers
(``vision/datasets.py``) and the tensor transforms (``vision/own_transforms.py``, ``vision/io.py``)."""
from __future__ import annotations

import enum
from typing import Callable, Dict

import torch
from torch import nn

from .datasets import Cifar10, Cifar100, DatasetFormatError, ImageFolder, Mnist  # noqa: F401
from .own_transforms import (CenterCrop, ColorJitter, Compose, ElasticTransform, RandomApply, RandomChoice, RandomCrop,  # noqa: F401
                             RandomHorizontalFlip, RandomResizedCrop, RandomRotation, RandomVerticalFlip, Resize,
                             TrivialAugmentWide)

from ..models import detection as _det
from ..models import vision_zoo as _zoo
from ..models.detection import (FeaturePyramidNetwork, MaskRCNNHeads as MaskHead, MaskRCNNPredictor as MaskPredictor,  # noqa: F401
                                RegionProposalNetwork as Rpn, RPNHead as RpnHead, TwoMLPHead as TwoMlpHead)
from ..models.vision_zoo import ASPP as Aspp, DeepLabHead as DeepLabV3Head, FCNHead as FcnHead  # noqa: F401
from ..ops.det_ops import AnchorGenerator  # noqa: F401

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)
FPN_OUT_CHANNELS = 256
SSD_FM_SIZES = (38, 19, 10, 5, 3, 1)
SSD_ANCHORS_PER_SCALE = (4, 6, 6, 6, 4, 4)
SSD_TOTAL_ANCHORS = sum(f * f * a for f, a in zip(SSD_FM_SIZES, SSD_ANCHORS_PER_SCALE))     # 8732


Ssd300 = _det.SSD300
FasterRcnn, MaskRcnn = _det.FasterRCNN, _det.MaskRCNN
DeepLabV3 = Fcn = _zoo.SegmentationModel
Detections = Dict[str, torch.Tensor]          # {"boxes", "labels", "scores"}: what the detectors return per image
MaskDetections = Dict[str, torch.Tensor]      # ... plus "masks"
SsdDetections = Dict[str, torch.Tensor]
MnistSample = CifarSample = tuple             # (image, label)
ModelConstructor = Callable[..., nn.Module]


class Split(enum.Enum):
    Train = "train"
    Test = "test"

    @property
    def train(self) -> bool:
        return self is Split.Train


class RpnConfig:
    """Settings of the region-proposal network (ferrotorch-vision/src/models/detection/rpn.rs
    ``RpnConfig::default_eval``: 1000 proposals before and after NMS, NMS at 0.7, no score
    threshold, boxes below 1e-3 pixels dropped)."""

    def __init__(self, pre_nms_top_n=1000, post_nms_top_n=1000, nms_thresh=0.7, score_thresh=0.0, min_size=1e-3):
        self.__dict__.update({k: v for k, v in locals().items() if k != "self"})

    @classmethod
    def default_eval(cls) -> "RpnConfig":
        return cls()

    def build(self, anchor_generator, head) -> "Rpn":
        c = self.__dict__
        return Rpn(head.cls_logits.in_channels, anchor_generator, c["pre_nms_top_n"], c["post_nms_top_n"], c["nms_thresh"],
                   c["score_thresh"], c["min_size"], head=head)


fasterrcnn_resnet50_fpn = _det.fasterrcnn_resnet50_fpn
maskrcnn_resnet50_fpn = _det.maskrcnn_resnet50_fpn
ssd300_vgg16 = _det.ssd300_vgg16
deeplabv3_resnet50 = _zoo.deeplabv3_resnet50
fcn_resnet50 = _zoo.fcn_resnet50


def ResNet50Dilated(num_classes: int = 1000, **kw) -> nn.Module:
    """ResNet-50 with strides of the last two stages replaced by dilation (output stride 8),
    the segmentation backbone."""
    from ..models.resnet import resnet50

    return resnet50(num_classes=num_classes, replace_stride_with_dilation=(False, True, True), **kw)


class ModelRegistry:
    """Name -> constructor over every model this package can build."""

    def __init__(self):
        self._extra: dict = {}

    def register(self, name: str, ctor: ModelConstructor) -> None:
        if name in self.names():
            raise ValueError("model %r is already registered" % name)
        self._extra[name] = ctor

    def names(self) -> list:
        from . import available

        return sorted(set(available()) | set(self._extra))

    def contains(self, name: str) -> bool:
        return name in self.names()

    def get(self, name: str, **kw) -> nn.Module:
        from . import build

        if name in self._extra:
            return self._extra[name](**kw)
        return build(name, **kw)

    # the reference's method names (ferrotorch-vision/src/models/registry.rs)
    register_model = register
    get_model = get

    def list_models(self) -> list:
        return self.names()


_registry = ModelRegistry()


def get_model(name: str, **kw) -> nn.Module:
    return _registry.get(name, **kw)


class FeatureExtractor(nn.Module):
    """Intermediate activations by sub-module name: ``{output name: tensor}``
    (ferrotorch-vision/src/models/feature_extractor.rs).  ``return_nodes`` maps dotted sub-module
    names (``"layer2"``, ``"features.3"``) to output names, or lists the names to keep as they
    are; the outputs are collected by forward hooks during one ordinary forward pass."""

    def __init__(self, model: nn.Module, return_nodes):
        super().__init__()
        self.body = model
        self.nodes = dict(return_nodes) if isinstance(return_nodes, dict) else {n: n for n in return_nodes}
        for n in self.nodes:
            model.get_submodule(n)                      # raises on an unknown name

    def forward(self, x: torch.Tensor) -> dict:
        got, handles = {}, []
        for node, name in self.nodes.items():
            handles.append(self.body.get_submodule(node).register_forward_hook(
                lambda _m, _i, out, name=name: got.__setitem__(name, out)))
        try:
            self.body(x)
        finally:
            for h in handles:
                h.remove()
        return {name: got[name] for name in self.nodes.values()}


def create_feature_extractor(model: nn.Module, return_nodes) -> FeatureExtractor:
    return FeatureExtractor(model, return_nodes)

__all__ = [_n for _n, _o in list(globals().items())
           if not _n.startswith("_") and type(_o).__name__ != "module" and _n not in ("annotations", "Callable", "Dict", "Any", "Hashable")]
