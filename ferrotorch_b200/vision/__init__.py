"""Vision: models, transforms, datasets and detection ops.

The reference's ``ferrotorch-vision`` has ten classifier families, seven detectors, four
segmenters, a model registry, MNIST / CIFAR / ImageFolder readers, 17 transforms, image IO and
NMS / RoIAlign (ferrotorch-vision/src/models/*, datasets/*, transforms/*, ops/*).  Here the ResNet
family (``models/resnet.py``: channels-last bf16, convolutions on the tcgen05 GEMM, fused batch-norm
kernels) and VGG-11/16, MobileNetV2, ViT-B/16, ConvNeXt-Tiny, DenseNet-121, FCN and DeepLabV3
(``models/vision_zoo.py``) and EfficientNet-B0, MobileNetV3, Inception v3, Swin-T and LRASPP
(``models/vision_families.py``) are this package's own, with torchvision's parameter names and
their dense convolutions and attention on this framework's kernels; Faster / Mask / Keypoint
R-CNN, RetinaNet, FCOS, SSD300 and the reference's small YOLO (``models/detection.py``) with their
NMS / RoI-align / anchor operators (``ops/det_ops.py``) are own code as well, and so are the
MNIST / CIFAR / image-folder readers (``vision/datasets.py``) and the tensor transforms
(``vision/own_transforms.py``, ``vision/io.py``).  Only ``ssdlite`` (not in the reference's
registry) still comes from ``torchvision``.  One registry serves all of them under the
reference's names.
"""
from __future__ import annotations

import torch
from torch import nn

from ..models.resnet import create_model, list_models, register_model, resnet18, resnet34, resnet50  # noqa: F401

from ..ops.det_ops import (batched_nms, box_area, box_convert, box_iou, clip_boxes_to_image, complete_box_iou,  # noqa: F401,E402
                           decode_boxes, distance_box_iou, focal_loss, generalized_box_iou, nms, remove_small_boxes, roi_align,
                           roi_align_with_aligned, roi_pool, sigmoid_focal_loss)

try:
    import torchvision
    from torchvision import transforms  # noqa: F401  (torchvision's PIL / tensor transforms, as a convenience)
    from torchvision.datasets import CIFAR10, CIFAR100, MNIST  # noqa: F401  (its downloading dataset classes)

    HAVE_TORCHVISION = True
except Exception:  # noqa: BLE001
    torchvision = None
    HAVE_TORCHVISION = False

# reference name -> torchvision constructor name
CLASSIFIERS = {"vgg11": "vgg11", "vgg16": "vgg16", "vit_b_16": "vit_b_16", "efficientnet_b0": "efficientnet_b0",
               "convnext_tiny": "convnext_tiny", "swin_t": "swin_t", "mobilenet_v2": "mobilenet_v2",
               "mobilenet_v3_small": "mobilenet_v3_small", "mobilenet_v3_large": "mobilenet_v3_large",
               "densenet121": "densenet121", "inception_v3": "inception_v3"}
DETECTORS = {"faster_rcnn": "fasterrcnn_resnet50_fpn", "mask_rcnn": "maskrcnn_resnet50_fpn",
             "keypoint_rcnn": "keypointrcnn_resnet50_fpn", "retinanet": "retinanet_resnet50_fpn",
             "fcos": "fcos_resnet50_fpn", "ssd300": "ssd300_vgg16", "ssdlite": "ssdlite320_mobilenet_v3_large"}
SEGMENTERS = {"deeplabv3": "deeplabv3_resnet50", "fcn": "fcn_resnet50", "lraspp": "lraspp_mobilenet_v3_large"}


def _tv(name: str, **kw) -> nn.Module:
    if not HAVE_TORCHVISION:
        raise ImportError("torchvision is needed for %r" % name)
    kw.setdefault("weights", None)
    if name in DETECTORS.values() or name in SEGMENTERS.values():
        kw.setdefault("weights_backbone", None)
    return torchvision.models.get_model(name, **kw)


def build(name: str, **kw) -> nn.Module:
    """One constructor for every model name of the reference's registry (own implementations
    first, torchvision for the rest)."""
    if name in list_models():
        return create_model(name, **kw)
    from ..models.detection import OWN_MODELS as DET
    from ..models.vision_families import OWN_MODELS as MORE
    from ..models.vision_zoo import OWN_MODELS

    for own in (OWN_MODELS, MORE, DET):
        if name in own:
            return own[name](**kw)
    for table in (CLASSIFIERS, DETECTORS, SEGMENTERS):
        if name in table:
            return _tv(table[name], **kw)
    if name == "unet":
        return UNet(**kw)
    return create_model(name, **kw)


def available() -> list[str]:
    """Every name :func:`build` accepts."""
    from ..models.detection import OWN_MODELS as DET
    from ..models.vision_families import OWN_MODELS as MORE
    from ..models.vision_zoo import OWN_MODELS

    return sorted(set(list_models()) | set(OWN_MODELS) | set(MORE) | set(DET) | set(CLASSIFIERS) | set(DETECTORS) | set(SEGMENTERS)
                  | {"unet"})


class UNet(nn.Module):
    """Encoder-decoder with skip connections (ferrotorch-vision/src/models/unet.rs);
    torchvision has no UNet, so this one is written out."""

    def __init__(self, in_channels: int = 3, num_classes: int = 2, base: int = 32, depth: int = 4):
        super().__init__()

        def block(i, o):
            return nn.Sequential(nn.Conv2d(i, o, 3, padding=1, bias=False), nn.BatchNorm2d(o), nn.ReLU(inplace=True),
                                 nn.Conv2d(o, o, 3, padding=1, bias=False), nn.BatchNorm2d(o), nn.ReLU(inplace=True))

        chans = [base * 2 ** i for i in range(depth + 1)]
        self.down = nn.ModuleList(block(in_channels if i == 0 else chans[i - 1], chans[i]) for i in range(depth + 1))
        self.up = nn.ModuleList(nn.ConvTranspose2d(chans[i + 1], chans[i], 2, stride=2) for i in reversed(range(depth)))
        self.dec = nn.ModuleList(block(2 * chans[i], chans[i]) for i in reversed(range(depth)))
        self.head = nn.Conv2d(chans[0], num_classes, 1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        skips = []
        for i, d in enumerate(self.down):
            x = d(x if i == 0 else nn.functional.max_pool2d(x, 2))
            skips.append(x)
        skips.pop()
        for up, dec in zip(self.up, self.dec):
            x = up(x)
            s = skips.pop()
            if x.shape[-2:] != s.shape[-2:]:
                x = nn.functional.interpolate(x, size=s.shape[-2:], mode="nearest")
            x = dec(torch.cat([s, x], 1))
        return self.head(x)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)


from .io import (GaussianNoise, RandomGaussianBlur, RawImage, VisionNormalize, VisionToTensor,  # noqa: F401,E402
                 raw_image_to_tensor, read_image, read_image_as_tensor, read_image_rgba, tensor_to_raw_image,
                 vision_manual_seed, write_image, write_tensor_as_image)

from . import det_ops  # noqa: F401,E402

from .compat import *  # noqa: F401,F403,E402
from .compat import (FPN_OUT_CHANNELS, IMAGENET_MEAN, IMAGENET_STD, SSD_ANCHORS_PER_SCALE, SSD_FM_SIZES,  # noqa: F401,E402
                     SSD_TOTAL_ANCHORS, CifarSample, Detections, MaskDetections, MnistSample, ModelConstructor,
                     SsdDetections)


def __getattr__(name):
    """Constructor functions of the model zoo under the reference's names (``vision.vgg16()``,
    ``vision.retinanet_resnet50_fpn()``, ``vision.swin_tiny()`` ...), resolved through the registry on first use,
    and the detectors' post-processing helpers."""
    alias = {"swin_tiny": "swin_t"}
    if name == "mobilenet_v3_large_dilated":
        return lambda **kw: build("mobilenet_v3_large", dilated=True, **kw)
    if name == "resnet50_dilated":
        return lambda num_classes=1000, **kw: resnet50(num_classes=num_classes, replace_stride_with_dilation=(False, True, True), **kw)
    if name in ("heatmaps_to_keypoints", "paste_masks_in_image", "postprocess_detections", "postprocess_masks", "decode_per_class",
                "apply_bn_buffers_from_state_dict"):
        from ..models import detection

        return getattr(detection, name)
    target = alias.get(name, name)
    if target in available() or target in CLASSIFIERS or target in set(DETECTORS.values()) | set(SEGMENTERS.values()):
        return lambda **kw: build(target, **kw)
    raise AttributeError(name)
