#!/usr/bin/env python
"""Object detection with this package's own detectors: build a model by its registry name, run
it on a synthetic image with a few bright rectangles, print the detections, and show the
operators underneath (anchors, NMS, RoI align).  Weights are random, so the boxes mean nothing:
the point is the API and the shapes.  Pass ``--weights file.safetensors`` (a torchvision state
dict) to load a trained detector; the parameter names are torchvision's.

    python examples/detect_objects.py [--model retinanet] [--size 128]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ferrotorch_b200 import vision  # noqa: E402
from ferrotorch_b200.ops import det_ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="retinanet", choices=["retinanet", "fcos", "faster_rcnn", "mask_rcnn", "ssd300", "yolo"])
    ap.add_argument("--size", type=int, default=128)
    ap.add_argument("--weights", default=None)
    a = ap.parse_args()
    torch.manual_seed(0)
    kw = {"score_thresh": 0.0} if a.model in ("retinanet", "fcos") else {}
    model = vision.build(a.model, num_classes=4, **kw).eval()
    if a.weights:
        from ferrotorch_b200.serialize.state import load_safetensors

        model.load_state_dict(load_safetensors(a.weights), strict=True)
    size = 416 if a.model == "yolo" else 300 if a.model == "ssd300" else a.size
    img = torch.rand(1, 3, size, size) * 0.1
    img[:, :, size // 8: size // 2, size // 8: size // 3] += 0.8          # two "objects"
    img[:, 1, size // 2: size * 7 // 8, size // 2: size * 3 // 4] += 0.6
    if a.model == "yolo":
        with torch.no_grad():
            grid = model(img)
        det = model.decode(grid, [(30, 40), (80, 60), (150, 200)], (size, size), conf_thresh=0.1)[0]
        print("grid", tuple(grid.shape))
    else:
        det = model(img)[0]
    n = len(det["boxes"])
    print("%s: %d detections, best score %.3f, labels %s" % (a.model, n, float(det["scores"][0]) if n else 0.0,
                                                             sorted(set(det["labels"].tolist()))))
    if "masks" in det:
        print("masks", tuple(det["masks"].shape))
    # the operators underneath
    anchors = det_ops.AnchorGenerator(((32,), (64,)), ((0.5, 1.0, 2.0),) * 2)((size, size), [(size // 8, size // 8), (size // 16, size // 16)])
    boxes = torch.tensor([[10.0, 10, 60, 60], [12, 12, 62, 62], [70, 70, 120, 110]])
    keep = det_ops.nms(boxes, torch.tensor([0.9, 0.8, 0.7]), 0.5)
    pooled = det_ops.roi_align(torch.rand(1, 8, size // 4, size // 4), torch.tensor([[0.0, 10, 10, 60, 60]]), 7, 0.25, 2)
    print("anchors", tuple(anchors.shape), "| nms keeps", keep.tolist(), "| roi_align", tuple(pooled.shape))


if __name__ == "__main__":
    main()
