"""The reference's ``ferrotorch-vision`` names over torchvision (ferrotorch-vision/src/lib.rs
re-exports: datasets, transforms, detection / segmentation building blocks, the model registry,
feature extraction).  Nothing here computes: each name points at the torchvision object that
provides the behaviour, or wraps this package's registry."""
from __future__ import annotations

import enum
from typing import Callable, Dict

import torch
from torch import nn

import torchvision
from torchvision import transforms as T
from torchvision.datasets import CIFAR10 as Cifar10, CIFAR100 as Cifar100, MNIST as Mnist  # noqa: F401
from torchvision.models import detection as _det, segmentation as _seg
from torchvision.models.detection.anchor_utils import AnchorGenerator  # noqa: F401
from torchvision.models.detection.faster_rcnn import TwoMLPHead as TwoMlpHead  # noqa: F401
from torchvision.models.detection.mask_rcnn import MaskRCNNHeads as MaskHead, MaskRCNNPredictor as MaskPredictor  # noqa: F401
from torchvision.models.detection.rpn import RegionProposalNetwork as Rpn, RPNHead as RpnHead  # noqa: F401
from torchvision.models.feature_extraction import create_feature_extractor as _tv_extractor
from torchvision.models.segmentation.deeplabv3 import ASPP as Aspp, DeepLabHead as DeepLabV3Head  # noqa: F401
from torchvision.models.segmentation.fcn import FCNHead as FcnHead  # noqa: F401
from torchvision.ops import FeaturePyramidNetwork  # noqa: F401

IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)
FPN_OUT_CHANNELS = 256
SSD_FM_SIZES = (38, 19, 10, 5, 3, 1)
SSD_ANCHORS_PER_SCALE = (4, 6, 6, 6, 4, 4)
SSD_TOTAL_ANCHORS = sum(f * f * a for f, a in zip(SSD_FM_SIZES, SSD_ANCHORS_PER_SCALE))     # 8732

CenterCrop, ColorJitter, RandomApply, RandomChoice = T.CenterCrop, T.ColorJitter, T.RandomApply, T.RandomChoice
RandomResizedCrop, RandomRotation, RandomVerticalFlip, Resize = T.RandomResizedCrop, T.RandomRotation, T.RandomVerticalFlip, T.Resize

from torchvision.models.detection.ssd import SSD as Ssd300  # noqa: E402

FasterRcnn, MaskRcnn = _det.FasterRCNN, _det.MaskRCNN
DeepLabV3, Fcn = _seg.DeepLabV3, _seg.FCN
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
    """Keyword arguments of the region-proposal network with torchvision's Faster R-CNN defaults."""

    def __init__(self, pre_nms_top_n_train=2000, pre_nms_top_n_test=1000, post_nms_top_n_train=2000,
                 post_nms_top_n_test=1000, nms_thresh=0.7, fg_iou_thresh=0.7, bg_iou_thresh=0.3,
                 batch_size_per_image=256, positive_fraction=0.5, score_thresh=0.0):
        self.__dict__.update({k: v for k, v in locals().items() if k != "self"})

    def build(self, anchor_generator, head) -> "Rpn":
        c = self.__dict__
        return Rpn(anchor_generator, head, c["fg_iou_thresh"], c["bg_iou_thresh"], c["batch_size_per_image"],
                   c["positive_fraction"], {"training": c["pre_nms_top_n_train"], "testing": c["pre_nms_top_n_test"]},
                   {"training": c["post_nms_top_n_train"], "testing": c["post_nms_top_n_test"]}, c["nms_thresh"], c["score_thresh"])


def _no_weights(ctor):
    def make(num_classes: int | None = None, **kw):
        kw.setdefault("weights", None)
        kw.setdefault("weights_backbone", None)
        if num_classes is not None:
            kw["num_classes"] = num_classes
        return ctor(**kw)
    make.__name__ = ctor.__name__
    make.__doc__ = "``torchvision``'s %s with random weights unless ``weights=`` is given." % ctor.__name__
    return make


fasterrcnn_resnet50_fpn = _no_weights(_det.fasterrcnn_resnet50_fpn)
maskrcnn_resnet50_fpn = _no_weights(_det.maskrcnn_resnet50_fpn)
ssd300_vgg16 = _no_weights(_det.ssd300_vgg16)
deeplabv3_resnet50 = _no_weights(_seg.deeplabv3_resnet50)
fcn_resnet50 = _no_weights(_seg.fcn_resnet50)


def ResNet50Dilated(num_classes: int = 1000, **kw) -> nn.Module:
    """ResNet-50 with strides of the last two stages replaced by dilation (output stride 8),
    the segmentation backbone."""
    return torchvision.models.resnet50(weights=None, num_classes=num_classes, replace_stride_with_dilation=[False, True, True], **kw)


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


_registry = ModelRegistry()


def get_model(name: str, **kw) -> nn.Module:
    return _registry.get(name, **kw)


class FeatureExtractor(nn.Module):
    """Intermediate activations by node name: ``{output name: tensor}``."""

    def __init__(self, model: nn.Module, return_nodes):
        super().__init__()
        self.body = _tv_extractor(model, return_nodes)

    def forward(self, x: torch.Tensor) -> dict:
        return self.body(x)


def create_feature_extractor(model: nn.Module, return_nodes) -> FeatureExtractor:
    return FeatureExtractor(model, return_nodes)

__all__ = [_n for _n, _o in list(globals().items())
           if not _n.startswith("_") and type(_o).__name__ != "module" and _n not in ("annotations", "Callable", "Dict", "Any", "Hashable")]
