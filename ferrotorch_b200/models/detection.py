"""Object detectors as this package's own modules: feature pyramid, region-proposal network, RoI
heads (boxes, masks, keypoints), Faster / Mask / Keypoint R-CNN, RetinaNet, FCOS, SSD300 and the
small YOLO of the reference.

The reference implements them in ``ferrotorch-vision/src/models/detection/`` (``fpn.rs``,
``rpn.rs``, ``faster_rcnn.rs``, ``mask_rcnn.rs``, ``keypoint_rcnn.rs``, ``retinanet.rs``,
``fcos.rs``, ``ssd.rs``, ``roi_heads_postprocess.rs``) and ``models/yolo.rs``, inference only, with
torchvision's parameter names so that torchvision checkpoints load.  The modules here keep those
names (the tests load a torchvision state dict with ``strict=True`` and compare detections), sit on
this package's own ResNet / VGG, and use the plain-torch operators of ``ops/det_ops.py`` (NMS,
RoI align, box decoding, anchors).  Like the reference's ``forward`` they take a batch
``[B, 3, H, W]`` that is already normalised and sized (H, W multiples of 32 for the pyramid
models; SSD resizes to 300 x 300 itself) and return one ``{"boxes", "scores", "labels", ...}``
dictionary per image.
"""
from __future__ import annotations

import math
from collections import OrderedDict

import torch
import torch.nn.functional as tF
from torch import nn

from ..ops.conv import convert_convs
from ..ops import det_ops as D
from .resnet import resnet50


# --------------------------------------------------------------------------- backbone + FPN
class LastLevelP6P7(nn.Module):
    def __init__(self, cin: int, cout: int):
        super().__init__()
        self.p6, self.p7 = nn.Conv2d(cin, cout, 3, 2, 1), nn.Conv2d(cout, cout, 3, 2, 1)
        self.use_p5 = cin == cout

    def forward(self, p5, c5):
        p6 = self.p6(p5 if self.use_p5 else c5)
        return p6, self.p7(tF.relu(p6))


class FeaturePyramidNetwork(nn.Module):
    """Top-down pathway with lateral 1 x 1 convolutions and 3 x 3 output convolutions; ``extra`` is
    ``"pool"`` (one more level by stride-2 subsampling) or ``"p6p7"`` (two more by strided convolutions)."""

    def __init__(self, in_channels: list[int], out_channels: int = 256, extra: str | None = "pool"):
        super().__init__()
        self.inner_blocks = nn.ModuleList(nn.Sequential(nn.Conv2d(c, out_channels, 1)) for c in in_channels)
        self.layer_blocks = nn.ModuleList(nn.Sequential(nn.Conv2d(out_channels, out_channels, 3, padding=1)) for _ in in_channels)
        self.extra = extra
        if extra == "p6p7":
            self.extra_blocks = LastLevelP6P7(out_channels, out_channels)

    def forward(self, feats: "OrderedDict[str, torch.Tensor]") -> "OrderedDict[str, torch.Tensor]":
        names, xs = list(feats.keys()), list(feats.values())
        last = self.inner_blocks[-1](xs[-1])
        outs = [self.layer_blocks[-1](last)]
        for i in range(len(xs) - 2, -1, -1):
            last = self.inner_blocks[i](xs[i]) + tF.interpolate(last, size=xs[i].shape[-2:], mode="nearest")
            outs.insert(0, self.layer_blocks[i](last))
        if self.extra == "pool":
            names.append("pool")
            outs.append(tF.max_pool2d(outs[-1], 1, 2, 0))
        elif self.extra == "p6p7":
            names += ["p6", "p7"]
            outs += list(self.extra_blocks(outs[-1], xs[-1]))
        return OrderedDict(zip(names, outs))


class ResNetFPN(nn.Module):
    """``body`` = this package's ResNet-50 without its classifier, ``fpn`` over the stages in
    ``returned_layers`` (1-based)."""

    def __init__(self, returned_layers=(1, 2, 3, 4), extra: str | None = "pool"):
        super().__init__()
        body = resnet50()
        del body.fc
        self.body = body
        self.returned = list(returned_layers)
        self.fpn = FeaturePyramidNetwork([256 * 2 ** (i - 1) for i in self.returned], 256, extra)
        self.out_channels = 256

    def forward_body(self, x) -> "OrderedDict[str, torch.Tensor]":
        """The returned stages of the ResNet body, keyed ``"0"``, ``"1"`` ... in order."""
        from .resnet import _bn

        b = self.body
        x = b.maxpool(_bn(b.conv1(x), b.bn1))
        feats = OrderedDict()
        for i, layer in enumerate((b.layer1, b.layer2, b.layer3, b.layer4), 1):
            x = layer(x)
            if i in self.returned:
                feats[str(self.returned.index(i))] = x
        return feats

    def forward(self, x):
        return self.fpn(self.forward_body(x))


def _as_batch(images) -> torch.Tensor:
    """A batch tensor as it is; a list of ``[3, H, W]`` images stacked, the smaller ones zero-padded
    at the bottom / right to the largest (rounded up to a multiple of 32 when they differ)."""
    if torch.is_tensor(images):
        return images
    hs, ws = [im.shape[-2] for im in images], [im.shape[-1] for im in images]
    if len(set(hs)) == 1 and len(set(ws)) == 1:
        return torch.stack(list(images))
    H, W = (max(hs) + 31) // 32 * 32, (max(ws) + 31) // 32 * 32
    return torch.stack([tF.pad(im, (0, W - im.shape[-1], 0, H - im.shape[-2])) for im in images])


def _permute_head_output(t: torch.Tensor, c: int) -> torch.Tensor:
    """``[N, A * c, H, W]`` -> ``[N, H * W * A, c]`` (the anchor order of the generators)."""
    n, _, h, w = t.shape
    return t.view(n, -1, c, h, w).permute(0, 3, 4, 1, 2).reshape(n, -1, c)


# --------------------------------------------------------------------------- RPN
class RPNHead(nn.Module):
    def __init__(self, in_channels: int, num_anchors: int):
        super().__init__()
        self.conv = nn.Sequential(nn.Sequential(nn.Conv2d(in_channels, in_channels, 3, padding=1), nn.ReLU(inplace=True)))
        self.cls_logits = nn.Conv2d(in_channels, num_anchors, 1)
        self.bbox_pred = nn.Conv2d(in_channels, 4 * num_anchors, 1)

    def forward(self, feats: list[torch.Tensor]):
        ts = [self.conv(f) for f in feats]
        return [self.cls_logits(t) for t in ts], [self.bbox_pred(t) for t in ts]

    def forward_level(self, x: torch.Tensor):
        """One pyramid level: ``(objectness [B, A, H, W], box deltas [B, 4 A, H, W])``."""
        t = self.conv(x)
        return self.cls_logits(t), self.bbox_pred(t)


class RegionProposalNetwork(nn.Module):
    """Objectness + box deltas per anchor; per pyramid level the ``pre_nms_top_n`` best anchors are
    decoded, clipped, filtered (size, score), suppressed per level and the best ``post_nms_top_n``
    of the image are kept."""

    def __init__(self, in_channels: int = 256, anchors: D.AnchorGenerator | None = None, pre_nms_top_n: int = 1000,
                 post_nms_top_n: int = 1000, nms_thresh: float = 0.7, score_thresh: float = 0.0, min_size: float = 1e-3,
                 head: RPNHead | None = None):
        super().__init__()
        self.anchor_generator = anchors or D.AnchorGenerator()
        self.head = head or RPNHead(in_channels, self.anchor_generator.num_anchors_per_location()[0])
        self.pre_nms_top_n, self.post_nms_top_n = pre_nms_top_n, post_nms_top_n
        self.nms_thresh, self.score_thresh, self.min_size = nms_thresh, score_thresh, min_size

    def forward(self, feats: "OrderedDict[str, torch.Tensor]", image_size: tuple[int, int]) -> list[torch.Tensor]:
        fs = list(feats.values())
        obj, deltas = self.head(fs)
        anchors = self.anchor_generator(image_size, [tuple(f.shape[-2:]) for f in fs], fs[0].dtype, fs[0].device)
        per_level = [o[0].numel() for o in obj]
        obj = torch.cat([_permute_head_output(o, 1) for o in obj], 1).squeeze(-1)            # [N, sum]
        deltas = torch.cat([_permute_head_output(d, 4) for d in deltas], 1)                    # [N, sum, 4]
        levels = torch.cat([torch.full((n,), i, dtype=torch.int64, device=obj.device) for i, n in enumerate(per_level)])
        out = []
        for n in range(obj.shape[0]):
            idx, off = [], 0
            for cnt in per_level:
                k = min(self.pre_nms_top_n, cnt)
                idx.append(obj[n, off:off + cnt].detach().topk(k)[1] + off)
                off += cnt
            idx = torch.cat(idx)
            boxes = D.decode_boxes(deltas[n, idx].detach(), anchors[idx])
            scores, lvl = torch.sigmoid(obj[n, idx].detach()), levels[idx]
            boxes = D.clip_boxes_to_image(boxes, image_size)
            keep = D.remove_small_boxes(boxes, self.min_size)
            boxes, scores, lvl = boxes[keep], scores[keep], lvl[keep]
            keep = torch.where(scores >= self.score_thresh)[0]
            boxes, scores, lvl = boxes[keep], scores[keep], lvl[keep]
            keep = D.batched_nms(boxes, scores, lvl, self.nms_thresh)[: self.post_nms_top_n]
            out.append(boxes[keep])
        return out


# --------------------------------------------------------------------------- RoI heads
class TwoMLPHead(nn.Module):
    def __init__(self, in_features: int, representation: int = 1024):
        super().__init__()
        self.fc6, self.fc7 = nn.Linear(in_features, representation), nn.Linear(representation, representation)

    def forward(self, x):
        return tF.relu(self.fc7(tF.relu(self.fc6(x.flatten(1)))))


class FastRCNNPredictor(nn.Module):
    def __init__(self, in_features: int, num_classes: int):
        super().__init__()
        self.cls_score, self.bbox_pred = nn.Linear(in_features, num_classes), nn.Linear(in_features, 4 * num_classes)

    def forward(self, x):
        x = x.flatten(1)
        return self.cls_score(x), self.bbox_pred(x)


class MaskRCNNHeads(nn.Sequential):
    """The mask branch's tower: 3 x 3 convolutions + ReLU on the 14 x 14 pooled features."""

    def __init__(self, in_channels: int, layers=(256, 256, 256, 256), dilation: int = 1):
        blocks, cin = [], in_channels
        for c in layers:
            blocks.append(nn.Sequential(nn.Conv2d(cin, c, 3, padding=dilation, dilation=dilation), nn.ReLU(inplace=True)))
            cin = c
        super().__init__(*blocks)


class MaskRCNNPredictor(nn.Sequential):
    def __init__(self, in_channels: int, dim_reduced: int, num_classes: int):
        super().__init__(OrderedDict([("conv5_mask", nn.ConvTranspose2d(in_channels, dim_reduced, 2, 2, 0)),
                                      ("relu", nn.ReLU(inplace=True)),
                                      ("mask_fcn_logits", nn.Conv2d(dim_reduced, num_classes, 1, 1, 0))]))


class KeypointRCNNPredictor(nn.Module):
    def __init__(self, in_channels: int, num_keypoints: int):
        super().__init__()
        self.kps_score_lowres = nn.ConvTranspose2d(in_channels, num_keypoints, 4, stride=2, padding=1)

    def forward(self, x):
        return tF.interpolate(self.kps_score_lowres(x), scale_factor=2.0, mode="bilinear", align_corners=False,
                              recompute_scale_factor=False)


def paste_masks_in_image(masks: torch.Tensor, boxes: torch.Tensor, image_size: tuple[int, int], padding: int = 1) -> torch.Tensor:
    """``masks [K, 1, M, M]`` (probabilities inside their boxes) -> ``[K, 1, H, W]``: every mask is
    padded by one pixel, its box grown by the same ratio, and resized to the box's integer extent."""
    K, M = masks.shape[0], masks.shape[-1]
    H, W = image_size
    out = masks.new_zeros((K, 1, H, W))
    if K == 0:
        return out
    scale = float(M + 2 * padding) / M
    masks = tF.pad(masks, (padding,) * 4)
    wh, hh = (boxes[:, 2] - boxes[:, 0]) * 0.5 * scale, (boxes[:, 3] - boxes[:, 1]) * 0.5 * scale
    xc, yc = (boxes[:, 2] + boxes[:, 0]) * 0.5, (boxes[:, 3] + boxes[:, 1]) * 0.5
    ib = torch.stack((xc - wh, yc - hh, xc + wh, yc + hh), 1).to(torch.int64).tolist()
    for i, (x0, y0, x1, y1) in enumerate(ib):
        w, h = max(x1 - x0 + 1, 1), max(y1 - y0 + 1, 1)
        m = tF.interpolate(masks[i][None], size=(h, w), mode="bilinear", align_corners=False)[0, 0]
        xa, xb, ya, yb = max(x0, 0), min(x1 + 1, W), max(y0, 0), min(y1 + 1, H)
        out[i, 0, ya:yb, xa:xb] = m[ya - y0:yb - y0, xa - x0:xb - x0]
    return out


def heatmaps_to_keypoints(maps: torch.Tensor, rois: torch.Tensor):
    """``maps [K, P, S, S]`` -> keypoints ``[K, P, 3]`` (x, y, 1) in image coordinates and their
    scores ``[K, P]``: each heat map is resized (bicubic) to its box and its arg-max taken."""
    ox, oy = rois[:, 0], rois[:, 1]
    ws, hs = (rois[:, 2] - rois[:, 0]).clamp(min=1), (rois[:, 3] - rois[:, 1]).clamp(min=1)
    wc, hc = ws.ceil(), hs.ceil()
    K, P = maps.shape[:2]
    xy = torch.zeros((K, 3, P), dtype=torch.float32, device=maps.device)
    sc = torch.zeros((K, P), dtype=torch.float32, device=maps.device)
    for i in range(K):
        rw, rh = int(wc[i].item()), int(hc[i].item())
        m = tF.interpolate(maps[i][:, None], size=(rh, rw), mode="bicubic", align_corners=False)[:, 0]
        pos = m.reshape(P, -1).argmax(1)
        xi = pos % rw
        yi = torch.div(pos - xi, rw, rounding_mode="floor")
        xy[i, 0] = (xi.float() + 0.5) * (ws[i] / rw) + ox[i]
        xy[i, 1] = (yi.float() + 0.5) * (hs[i] / rh) + oy[i]
        xy[i, 2] = 1
        sc[i] = m[torch.arange(P, device=maps.device), yi, xi]
    return xy.permute(0, 2, 1), sc


def decode_per_class(box_regression: torch.Tensor, proposals: torch.Tensor, weights=(10.0, 10.0, 5.0, 5.0)) -> torch.Tensor:
    """``box_regression [R, C * 4]`` -> boxes ``[R, C, 4]``: every proposal decoded once per class with the
    Faster R-CNN delta weights (ferrotorch-vision/src/models/detection/roi_heads_postprocess.rs)."""
    C = box_regression.shape[-1] // 4
    return D.decode_boxes(box_regression, proposals, weights).reshape(-1, C, 4)


def postprocess_detections(class_logits: torch.Tensor, box_regression: torch.Tensor, proposals: list[torch.Tensor],
                           image_size: tuple[int, int], score_thresh: float = 0.05, nms_thresh: float = 0.5,
                           detections_per_img: int = 100) -> list[dict]:
    """Second-stage outputs to detections, per image: soft-max scores, per-class boxes clipped to the image,
    background dropped, low scores and degenerate boxes removed, per-class NMS, the best
    ``detections_per_img`` kept."""
    C = class_logits.shape[-1]
    boxes = decode_per_class(box_regression, torch.cat(proposals))
    scores = tF.softmax(class_logits, -1)
    out, off = [], 0
    for p in proposals:
        b, s = D.clip_boxes_to_image(boxes[off:off + len(p)], image_size), scores[off:off + len(p)]
        off += len(p)
        labels = torch.arange(C, device=b.device).view(1, -1).expand_as(s)
        b, s, labels = b[:, 1:].reshape(-1, 4), s[:, 1:].reshape(-1), labels[:, 1:].reshape(-1)     # drop background
        keep = torch.where(s > score_thresh)[0]
        b, s, labels = b[keep], s[keep], labels[keep]
        keep = D.remove_small_boxes(b, 1e-2)
        b, s, labels = b[keep], s[keep], labels[keep]
        keep = D.batched_nms(b, s, labels, nms_thresh)[:detections_per_img]
        out.append({"boxes": b[keep], "labels": labels[keep], "scores": s[keep]})
    return out


def postprocess_masks(mask_logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """``mask_logits [R, C, M, M]`` and the predicted class of every detection -> that class's mask
    probabilities ``[R, 1, M, M]``."""
    return torch.sigmoid(mask_logits)[torch.arange(len(labels), device=mask_logits.device), labels][:, None]


def apply_bn_buffers_from_state_dict(module: nn.Module, state_dict: dict, prefix: str = "") -> int:
    """Copy the running statistics (``running_mean`` / ``running_var`` / ``num_batches_tracked``) of every batch-norm
    layer below ``module`` from a state dict; returns how many buffers were set.  (``load_state_dict`` does this
    too; the reference loads parameters and buffers in two passes.)"""
    n = 0
    with torch.no_grad():
        for name, buf in module.named_buffers():
            key = prefix + name
            if name.rsplit(".", 1)[-1] in ("running_mean", "running_var", "num_batches_tracked") and key in state_dict:
                buf.copy_(state_dict[key].to(buf.dtype))
                n += 1
    return n


class RoIHeads(nn.Module):
    """Second stage: pooled box features -> class scores and per-class boxes -> per-class NMS; then,
    on the surviving boxes, the optional mask and keypoint branches."""

    def __init__(self, num_classes: int, score_thresh: float = 0.05, nms_thresh: float = 0.5, detections_per_img: int = 100):
        super().__init__()
        self.box_roi_pool = D.MultiScaleRoIAlign(["0", "1", "2", "3"], 7, 2)
        self.box_head = TwoMLPHead(256 * 7 * 7, 1024)
        self.box_predictor = FastRCNNPredictor(1024, num_classes)
        self.score_thresh, self.nms_thresh, self.detections_per_img = score_thresh, nms_thresh, detections_per_img
        self.mask_roi_pool = self.keypoint_roi_pool = None

    def add_mask_branch(self, num_classes: int) -> None:
        self.mask_roi_pool = D.MultiScaleRoIAlign(["0", "1", "2", "3"], 14, 2)
        self.mask_head = MaskRCNNHeads(256, (256, 256, 256, 256))
        self.mask_predictor = MaskRCNNPredictor(256, 256, num_classes)

    def add_keypoint_branch(self, num_keypoints: int) -> None:
        self.keypoint_roi_pool = D.MultiScaleRoIAlign(["0", "1", "2", "3"], 14, 2)
        layers, cin = [], 256
        for _ in range(8):
            layers += [nn.Conv2d(cin, 512, 3, padding=1), nn.ReLU(inplace=True)]
            cin = 512
        self.keypoint_head = nn.Sequential(*layers)
        self.keypoint_predictor = KeypointRCNNPredictor(512, num_keypoints)

    def forward(self, feats, proposals: list[torch.Tensor], image_size: tuple[int, int]) -> list[dict]:
        x = self.box_head(self.box_roi_pool(feats, proposals, image_size))
        logits, reg = self.box_predictor(x)
        out = postprocess_detections(logits, reg, proposals, image_size, self.score_thresh, self.nms_thresh, self.detections_per_img)
        if self.mask_roi_pool is not None:
            det = [o["boxes"] for o in out]
            ml = self.mask_predictor(self.mask_head(self.mask_roi_pool(feats, det, image_size)))
            prob = postprocess_masks(ml, torch.cat([o["labels"] for o in out]))
            for o, m in zip(out, prob.split([len(d) for d in det])):
                o["masks"] = paste_masks_in_image(m, o["boxes"], image_size)
        if self.keypoint_roi_pool is not None:
            det = [o["boxes"] for o in out]
            kl = self.keypoint_predictor(self.keypoint_head(self.keypoint_roi_pool(feats, det, image_size)))
            for o, m in zip(out, kl.split([len(d) for d in det])):
                o["keypoints"], o["keypoints_scores"] = heatmaps_to_keypoints(m, o["boxes"])
        return out


class FasterRCNN(nn.Module):
    def __init__(self, num_classes: int = 91, **roi_kw):
        super().__init__()
        self.backbone = ResNetFPN((1, 2, 3, 4), "pool")
        self.rpn = RegionProposalNetwork(256)
        self.roi_heads = RoIHeads(num_classes, **roi_kw)
        convert_convs(self)

    @torch.no_grad()
    def forward(self, images) -> list[dict]:
        images = _as_batch(images)
        size = tuple(images.shape[-2:])
        feats = self.backbone(images)
        return self.roi_heads(feats, self.rpn(feats, size), size)

    # ---- pieces of the pipeline under the reference's names (faster_rcnn.rs:278-300, 470-480), for heads
    # that reuse the features without running detection twice
    @torch.no_grad()
    def forward_backbone(self, images) -> dict:
        """ResNet stages C2 .. C5 as ``{"layer1": ..., "layer4": ...}``."""
        feats = self.backbone.forward_body(_as_batch(images))
        return {"layer%d" % self.backbone.returned[int(k)]: v for k, v in feats.items()}

    @torch.no_grad()
    def forward_fpn(self, backbone_features: dict) -> dict:
        """The pyramid ``{"p2": ..., "p6": ...}`` over the output of :meth:`forward_backbone`."""
        ordered = OrderedDict((str(i), backbone_features["layer%d" % l]) for i, l in enumerate(self.backbone.returned))
        out = self.backbone.fpn(ordered)
        return {"p%d" % (i + 2): v for i, v in enumerate(out.values())}

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad)

    def num_classes(self) -> int:
        """Detection classes, background (index 0) included."""
        return self.roi_heads.box_predictor.cls_score.out_features


class MaskRCNN(FasterRCNN):
    def __init__(self, num_classes: int = 91, **roi_kw):
        super().__init__(num_classes, **roi_kw)
        self.roi_heads.add_mask_branch(num_classes)
        convert_convs(self)


class KeypointRCNN(FasterRCNN):
    def __init__(self, num_classes: int = 2, num_keypoints: int = 17, **roi_kw):
        super().__init__(num_classes, **roi_kw)
        self.roi_heads.add_keypoint_branch(num_keypoints)
        convert_convs(self)


def fasterrcnn_resnet50_fpn(num_classes: int = 91, **kw):
    return FasterRCNN(num_classes, **kw)


def maskrcnn_resnet50_fpn(num_classes: int = 91, **kw):
    return MaskRCNN(num_classes, **kw)


def keypointrcnn_resnet50_fpn(num_classes: int = 2, num_keypoints: int = 17, **kw):
    return KeypointRCNN(num_classes, num_keypoints, **kw)


# --------------------------------------------------------------------------- one-stage: RetinaNet, FCOS
def _tower(channels: int, norm: bool) -> nn.Sequential:
    layers = []
    for _ in range(4):
        if norm:
            layers += [nn.Conv2d(channels, channels, 3, padding=1), nn.GroupNorm(32, channels), nn.ReLU()]
        else:
            layers.append(nn.Sequential(nn.Conv2d(channels, channels, 3, padding=1), nn.ReLU(inplace=True)))
    return nn.Sequential(*layers)


class _ClsHead(nn.Module):
    def __init__(self, channels, num_anchors, num_classes, norm, prior=0.01):
        super().__init__()
        self.conv = _tower(channels, norm)
        self.cls_logits = nn.Conv2d(channels, num_anchors * num_classes, 3, padding=1)
        nn.init.normal_(self.cls_logits.weight, std=0.01)
        nn.init.constant_(self.cls_logits.bias, -math.log((1 - prior) / prior))
        self.k = num_classes

    def forward(self, feats):
        return torch.cat([_permute_head_output(self.cls_logits(self.conv(f)), self.k) for f in feats], 1)


class _RetinaRegHead(nn.Module):
    def __init__(self, channels, num_anchors):
        super().__init__()
        self.conv = _tower(channels, False)
        self.bbox_reg = nn.Conv2d(channels, 4 * num_anchors, 3, padding=1)

    def forward(self, feats):
        return torch.cat([_permute_head_output(self.bbox_reg(self.conv(f)), 4) for f in feats], 1)


class _FcosRegHead(nn.Module):
    def __init__(self, channels, num_anchors):
        super().__init__()
        self.conv = _tower(channels, True)
        self.bbox_reg = nn.Conv2d(channels, 4 * num_anchors, 3, padding=1)
        self.bbox_ctrness = nn.Conv2d(channels, num_anchors, 3, padding=1)

    def forward(self, feats):
        reg, ctr = [], []
        for f in feats:
            t = self.conv(f)
            reg.append(_permute_head_output(tF.relu(self.bbox_reg(t)), 4))
            ctr.append(_permute_head_output(self.bbox_ctrness(t), 1))
        return torch.cat(reg, 1), torch.cat(ctr, 1)


class _Heads(nn.Module):
    def __init__(self, cls, reg):
        super().__init__()
        self.classification_head, self.regression_head = cls, reg


def _dense_postprocess(scores_per_level, boxes_fn, per_level, K, score_thresh, topk, nms_thresh, max_det, image_size):
    """Shared tail of the one-stage detectors: per level threshold + top-k over (anchor, class)
    pairs, decode the survivors, then per-class NMS over all levels."""
    boxes, scores, labels, off = [], [], [], 0
    for lvl, cnt in enumerate(per_level):
        s = scores_per_level[off:off + cnt].flatten()
        keep = torch.where(s > score_thresh)[0]
        s, idx = s[keep].topk(min(topk, len(keep)))
        idx = keep[idx]
        a = torch.div(idx, K, rounding_mode="floor")
        boxes.append(D.clip_boxes_to_image(boxes_fn(a + off), image_size))
        scores.append(s)
        labels.append(idx % K)
        off += cnt
    boxes, scores, labels = torch.cat(boxes), torch.cat(scores), torch.cat(labels)
    keep = D.batched_nms(boxes, scores, labels, nms_thresh)[:max_det]
    return {"boxes": boxes[keep], "scores": scores[keep], "labels": labels[keep]}


class RetinaNet(nn.Module):
    def __init__(self, num_classes: int = 91, score_thresh: float = 0.05, nms_thresh: float = 0.5, detections_per_img: int = 300,
                 topk_candidates: int = 1000):
        super().__init__()
        self.backbone = ResNetFPN((2, 3, 4), "p6p7")
        sizes = tuple((x, int(x * 2 ** (1.0 / 3)), int(x * 2 ** (2.0 / 3))) for x in [32, 64, 128, 256, 512])
        self.anchor_generator = D.AnchorGenerator(sizes, ((0.5, 1.0, 2.0),) * 5)
        A = self.anchor_generator.num_anchors_per_location()[0]
        self.head = _Heads(_ClsHead(256, A, num_classes, False), _RetinaRegHead(256, A))
        self.cfg = (num_classes, score_thresh, topk_candidates, nms_thresh, detections_per_img)
        convert_convs(self)

    @torch.no_grad()
    def forward(self, images) -> list[dict]:
        images = _as_batch(images)
        size = tuple(images.shape[-2:])
        fs = list(self.backbone(images).values())
        cls, reg = self.head.classification_head(fs), self.head.regression_head(fs)
        anchors = self.anchor_generator(size, [tuple(f.shape[-2:]) for f in fs], fs[0].dtype, fs[0].device)
        A = self.anchor_generator.num_anchors_per_location()[0]
        per_level = [f.shape[-2] * f.shape[-1] * A for f in fs]
        K, st, topk, nt, md = self.cfg
        return [_dense_postprocess(torch.sigmoid(cls[n]), lambda a, n=n: D.decode_boxes(reg[n][a], anchors[a]), per_level, K,
                                   st, topk, nt, md, size) for n in range(images.shape[0])]


class FCOS(nn.Module):
    def __init__(self, num_classes: int = 91, score_thresh: float = 0.2, nms_thresh: float = 0.6, detections_per_img: int = 100,
                 topk_candidates: int = 1000):
        super().__init__()
        self.backbone = ResNetFPN((2, 3, 4), "p6p7")
        self.anchor_generator = D.AnchorGenerator(((8,), (16,), (32,), (64,), (128,)), ((1.0,),) * 5)
        self.head = _Heads(_ClsHead(256, 1, num_classes, True), _FcosRegHead(256, 1))
        self.cfg = (num_classes, score_thresh, topk_candidates, nms_thresh, detections_per_img)
        convert_convs(self)

    @torch.no_grad()
    def forward(self, images) -> list[dict]:
        images = _as_batch(images)
        size = tuple(images.shape[-2:])
        fs = list(self.backbone(images).values())
        cls = self.head.classification_head(fs)
        reg, ctr = self.head.regression_head(fs)
        anchors = self.anchor_generator(size, [tuple(f.shape[-2:]) for f in fs], fs[0].dtype, fs[0].device)
        per_level = [f.shape[-2] * f.shape[-1] for f in fs]
        K, st, topk, nt, md = self.cfg
        out = []
        for n in range(images.shape[0]):
            scores = torch.sqrt(torch.sigmoid(cls[n]) * torch.sigmoid(ctr[n]))
            out.append(_dense_postprocess(scores, lambda a, n=n: D.decode_ltrb(reg[n][a], anchors[a]), per_level, K, st, topk,
                                          nt, md, size))
        return out


def retinanet_resnet50_fpn(num_classes: int = 91, **kw):
    return RetinaNet(num_classes, **kw)


def fcos_resnet50_fpn(num_classes: int = 91, **kw):
    return FCOS(num_classes, **kw)


# --------------------------------------------------------------------------- SSD300
class SSDFeatureExtractorVGG(nn.Module):
    """VGG-16 up to conv4_3 (L2-normalised and rescaled by a learned per-channel factor), then
    conv5 + the dilated fc6 / fc7 convolutions, then four shrinking extra blocks: six maps of
    38, 19, 10, 5, 3 and 1 cells for a 300 x 300 input."""

    def __init__(self):
        super().__init__()
        from .vision_zoo import vgg16

        feats = list(vgg16().features.children())
        pools = [i for i, layer in enumerate(feats) if isinstance(layer, nn.MaxPool2d)]
        feats[pools[2]] = nn.MaxPool2d(2, 2, ceil_mode=True)
        self.scale_weight = nn.Parameter(torch.ones(512) * 20)
        self.features = nn.Sequential(*feats[:pools[3]])
        fc = nn.Sequential(nn.MaxPool2d(3, 1, 1), nn.Conv2d(512, 1024, 3, padding=6, dilation=6), nn.ReLU(inplace=True),
                           nn.Conv2d(1024, 1024, 1), nn.ReLU(inplace=True))

        def block(cin, mid, cout, **kw):
            return nn.Sequential(nn.Conv2d(cin, mid, 1), nn.ReLU(inplace=True), nn.Conv2d(mid, cout, 3, **kw), nn.ReLU(inplace=True))

        self.extra = nn.ModuleList([nn.Sequential(*feats[pools[3]:-1], fc), block(1024, 256, 512, padding=1, stride=2),
                                    block(512, 128, 256, padding=1, stride=2), block(256, 128, 256), block(256, 128, 256)])

    def forward(self, x):
        x = self.features(x)
        outs = [self.scale_weight.view(1, -1, 1, 1) * tF.normalize(x)]
        for b in self.extra:
            x = b(x)
            outs.append(x)
        return outs


class _SSDScoringHead(nn.Module):
    def __init__(self, channels, num_anchors, width):
        super().__init__()
        self.module_list = nn.ModuleList(nn.Conv2d(c, a * width, 3, padding=1) for c, a in zip(channels, num_anchors))
        self.width = width

    def forward(self, feats):
        return torch.cat([_permute_head_output(m(f), self.width) for m, f in zip(self.module_list, feats)], 1)


class SSD300(nn.Module):
    """``normalize=True`` applies the statistics of the published checkpoint (inputs in ``[0, 1]``)."""

    def __init__(self, num_classes: int = 91, score_thresh: float = 0.01, nms_thresh: float = 0.45, detections_per_img: int = 200,
                 topk_candidates: int = 400, normalize: bool = True):
        super().__init__()
        self.backbone = SSDFeatureExtractorVGG()
        self.anchor_generator = D.DefaultBoxGenerator([[2], [2, 3], [2, 3], [2, 3], [2], [2]],
                                                      scales=[0.07, 0.15, 0.33, 0.51, 0.69, 0.87, 1.05],
                                                      steps=[8, 16, 32, 64, 100, 300])
        A, ch = self.anchor_generator.num_anchors_per_location(), [512, 1024, 512, 256, 256, 256]
        self.head = _Heads(_SSDScoringHead(ch, A, num_classes), _SSDScoringHead(ch, A, 4))
        self.cfg = (num_classes, score_thresh, topk_candidates, nms_thresh, detections_per_img)
        self.normalize = normalize
        convert_convs(self)

    @torch.no_grad()
    def forward(self, images) -> list[dict]:
        images = _as_batch(images)
        if self.normalize:
            mean = images.new_tensor([0.48235, 0.45882, 0.40784]).view(1, 3, 1, 1)
            images = (images - mean) * 255.0
        if tuple(images.shape[-2:]) != (300, 300):
            images = tF.interpolate(images, size=(300, 300), mode="bilinear", align_corners=False)
        fs = self.backbone(images)
        cls, reg = self.head.classification_head(fs), self.head.regression_head(fs)
        anchors = self.anchor_generator((300, 300), [tuple(f.shape[-2:]) for f in fs], fs[0].dtype, fs[0].device)
        K, st, topk, nt, md = self.cfg
        out = []
        for n in range(images.shape[0]):
            boxes = D.clip_boxes_to_image(D.decode_boxes(reg[n], anchors, (10.0, 10.0, 5.0, 5.0)), (300, 300))
            prob = tF.softmax(cls[n], -1)
            bs, ss, ls = [], [], []
            for label in range(1, K):
                s = prob[:, label]
                keep = torch.where(s > st)[0]
                s, idx = s[keep].topk(min(topk, len(keep)))
                bs.append(boxes[keep[idx]])
                ss.append(s)
                ls.append(torch.full_like(s, label, dtype=torch.int64))
            b, s, lab = torch.cat(bs), torch.cat(ss), torch.cat(ls)
            keep = D.batched_nms(b, s, lab, nt)[:md]
            out.append({"boxes": b[keep], "scores": s[keep], "labels": lab[keep]})
        return out


def ssd300_vgg16(num_classes: int = 91, **kw):
    return SSD300(num_classes, **kw)


# --------------------------------------------------------------------------- YOLO (the reference's small one)
class _YoloStage(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, 3, 1, 1, bias=False)

    def forward(self, x):
        return tF.max_pool2d(tF.relu(self.conv(x)), 2, 2)


class Yolo(nn.Module):
    """Five ``conv 3x3 -> ReLU -> max-pool 2`` stages (3 -> 32 -> 64 -> 128 -> 256 -> 512 channels,
    416 -> 13 cells) and a 1 x 1 head with ``num_anchors * (5 + num_classes)`` outputs per cell:
    ``(x, y, w, h, objectness)`` plus class scores per anchor (ferrotorch-vision/src/models/yolo.rs;
    parameter names ``backbone.stage{1..5}.conv.weight``, ``head.weight`` / ``head.bias``)."""

    def __init__(self, num_classes: int = 80, num_anchors: int = 3):
        super().__init__()
        self.num_classes, self.num_anchors = num_classes, num_anchors
        ch = [3, 32, 64, 128, 256, 512]
        self.backbone = nn.Sequential(OrderedDict(("stage%d" % (i + 1), _YoloStage(ch[i], ch[i + 1])) for i in range(5)))
        self.head = nn.Conv2d(512, num_anchors * (5 + num_classes), 1)
        convert_convs(self)

    def forward(self, x):
        return self.head(self.backbone(x))

    def decode(self, grid: torch.Tensor, anchors_wh, image_size: tuple[int, int], conf_thresh: float = 0.25,
               nms_thresh: float = 0.45) -> list[dict]:
        """Raw grid ``[B, A * (5 + C), S, S]`` -> detections: sigmoid cell offsets, exponential sizes
        relative to ``anchors_wh`` (pixels), confidence = objectness x best class, per-class NMS."""
        B, _, Sy, Sx = grid.shape
        A, C = self.num_anchors, self.num_classes
        g = grid.view(B, A, 5 + C, Sy, Sx).permute(0, 1, 3, 4, 2)
        cy, cx = torch.meshgrid(torch.arange(Sy, device=grid.device), torch.arange(Sx, device=grid.device), indexing="ij")
        aw = torch.as_tensor(anchors_wh, dtype=grid.dtype, device=grid.device).view(1, A, 1, 1, 2)
        px = (torch.sigmoid(g[..., 0]) + cx) * (image_size[1] / Sx)
        py = (torch.sigmoid(g[..., 1]) + cy) * (image_size[0] / Sy)
        pw, ph = torch.exp(g[..., 2].clamp(max=8)) * aw[..., 0], torch.exp(g[..., 3].clamp(max=8)) * aw[..., 1]
        conf, lab = (torch.sigmoid(g[..., 4:5]) * torch.softmax(g[..., 5:], -1)).max(-1)
        boxes = torch.stack((px - pw / 2, py - ph / 2, px + pw / 2, py + ph / 2), -1)
        out = []
        for n in range(B):
            b, s, lbl = boxes[n].reshape(-1, 4), conf[n].reshape(-1), lab[n].reshape(-1)
            keep = torch.where(s > conf_thresh)[0]
            b, s, lbl = D.clip_boxes_to_image(b[keep], image_size), s[keep], lbl[keep]
            keep = D.batched_nms(b, s, lbl, nms_thresh)
            out.append({"boxes": b[keep], "scores": s[keep], "labels": lbl[keep]})
        return out


def yolo(num_classes: int = 80, **kw):
    return Yolo(num_classes, **kw)


OWN_MODELS = {"faster_rcnn": fasterrcnn_resnet50_fpn, "fasterrcnn_resnet50_fpn": fasterrcnn_resnet50_fpn,
              "mask_rcnn": maskrcnn_resnet50_fpn, "maskrcnn_resnet50_fpn": maskrcnn_resnet50_fpn,
              "keypoint_rcnn": keypointrcnn_resnet50_fpn, "keypointrcnn_resnet50_fpn": keypointrcnn_resnet50_fpn,
              "retinanet": retinanet_resnet50_fpn, "retinanet_resnet50_fpn": retinanet_resnet50_fpn,
              "fcos": fcos_resnet50_fpn, "fcos_resnet50_fpn": fcos_resnet50_fpn,
              "ssd300": ssd300_vgg16, "ssd300_vgg16": ssd300_vgg16, "yolo": yolo}


# Rust's ``parameters_mut`` / ``num_parameters`` of the reference's detection modules: a Python module hands
# out its (mutable) parameters through ``parameters()``
def _num_parameters(self) -> int:
    return sum(p.numel() for p in self.parameters() if p.requires_grad)


for _cls in (FeaturePyramidNetwork, RPNHead, RegionProposalNetwork, TwoMLPHead, MaskRCNNHeads, MaskRCNNPredictor, SSD300, RetinaNet, FCOS,
             Yolo):
    _cls.parameters_mut = nn.Module.parameters
    _cls.num_parameters = _num_parameters
