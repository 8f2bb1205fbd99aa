"""Detection operators: box IoU, greedy non-maximum suppression (single and per-class), RoI align
with the sampling rules of the detectors' checkpoints, box coders, anchor and default-box
generators.  The NMS sweep and the fp32 host RoI align run in the native host library
(``csrc/host/det_ops.cpp``); everything has a torch formulation as well (any device, autograd).

The reference has them in ``ferrotorch-vision/src/ops/`` (``nms``, ``roi_align``, ``box_iou``),
``models/detection/anchor_utils.rs`` (``AnchorGenerator``, SSD default boxes) and
``models/detection/roi_heads_postprocess.rs`` (``decode_per_class``).  Semantics follow
torchvision's (boxes are ``x1, y1, x2, y2``; NMS keeps the higher score and drops boxes whose IoU
with a kept box is **above** the threshold; RoI align samples ``sampling_ratio^2`` points per bin,
no half-pixel shift unless ``aligned``), which the tests check against ``torchvision.ops``.
"""
from __future__ import annotations

import math

import torch

BBOX_XFORM_CLIP = math.log(1000.0 / 16)


def box_area(b: torch.Tensor) -> torch.Tensor:
    return (b[:, 2] - b[:, 0]) * (b[:, 3] - b[:, 1])


def box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Pairwise IoU ``[len(a), len(b)]``."""
    lt = torch.max(a[:, None, :2], b[None, :, :2])
    rb = torch.min(a[:, None, 2:], b[None, :, 2:])
    wh = (rb - lt).clamp(min=0)
    inter = wh[..., 0] * wh[..., 1]
    return inter / (box_area(a)[:, None] + box_area(b)[None, :] - inter)


def _enclosing_and_iou(a: torch.Tensor, b: torch.Tensor):
    iou = box_iou(a, b)
    lt = torch.min(a[:, None, :2], b[None, :, :2])
    rb = torch.max(a[:, None, 2:], b[None, :, 2:])
    return iou, lt, rb


def generalized_box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """GIoU ``[len(a), len(b)]``: IoU minus the share of the smallest enclosing box that neither box covers
    (Rezatofighi et al. 2019); in ``(-1, 1]``."""
    iou, lt, rb = _enclosing_and_iou(a, b)
    wh = (rb - lt).clamp(min=0)
    hull = wh[..., 0] * wh[..., 1]
    total = box_area(a)[:, None] + box_area(b)[None, :]
    union = total / (1 + iou)                                  # union = total - intersection, intersection = iou * union
    return iou - (hull - union) / hull


def _diou_terms(a: torch.Tensor, b: torch.Tensor, eps: float):
    iou, lt, rb = _enclosing_and_iou(a, b)
    wh = (rb - lt).clamp(min=0)
    diag = wh[..., 0] ** 2 + wh[..., 1] ** 2 + eps
    ca, cb = (a[:, :2] + a[:, 2:]) / 2, (b[:, :2] + b[:, 2:]) / 2
    dist = ((ca[:, None, :] - cb[None, :, :]) ** 2).sum(-1)
    return iou, dist / diag


def distance_box_iou(a: torch.Tensor, b: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """DIoU: IoU minus the squared centre distance over the squared diagonal of the enclosing box
    (Zheng et al. 2020)."""
    iou, penalty = _diou_terms(a, b, eps)
    return iou - penalty


def complete_box_iou(a: torch.Tensor, b: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """CIoU: DIoU minus an aspect-ratio term ``alpha * v`` with ``v = (4 / pi^2) (atan(w_b / h_b) - atan(w_a / h_a))^2``
    and ``alpha = v / (1 - IoU + v)`` (no gradient through ``alpha``)."""
    import math

    iou, penalty = _diou_terms(a, b, eps)
    wa, ha = a[:, 2] - a[:, 0], a[:, 3] - a[:, 1]
    wb, hb = b[:, 2] - b[:, 0], b[:, 3] - b[:, 1]
    v = (4 / math.pi ** 2) * (torch.atan(wa / ha)[:, None] - torch.atan(wb / hb)[None, :]) ** 2
    with torch.no_grad():
        alpha = v / (1 - iou + v + eps)
    return iou - penalty - alpha * v


def box_convert(boxes: torch.Tensor, in_fmt: str, out_fmt: str) -> torch.Tensor:
    """Between ``xyxy`` (corners), ``xywh`` (corner + size) and ``cxcywh`` (centre + size)."""
    fmts = ("xyxy", "xywh", "cxcywh")
    if in_fmt not in fmts or out_fmt not in fmts:
        raise ValueError("box_convert: formats must be among %s, got %r -> %r" % (fmts, in_fmt, out_fmt))
    if in_fmt == out_fmt:
        return boxes.clone()
    a, b, c, d = boxes.unbind(-1)
    if in_fmt == "xywh":
        a, b, c, d = a, b, a + c, b + d
    elif in_fmt == "cxcywh":
        a, b, c, d = a - c / 2, b - d / 2, a + c / 2, b + d / 2
    if out_fmt == "xywh":
        a, b, c, d = a, b, c - a, d - b
    elif out_fmt == "cxcywh":
        a, b, c, d = (a + c) / 2, (b + d) / 2, c - a, d - b
    return torch.stack((a, b, c, d), -1)


def sigmoid_focal_loss(inputs: torch.Tensor, targets: torch.Tensor, alpha: float = 0.25, gamma: float = 2.0,
                       reduction: str = "none") -> torch.Tensor:
    """Binary focal loss on logits (Lin et al. 2017): ``alpha_t (1 - p_t)^gamma BCE``; ``alpha < 0`` switches the
    class weighting off."""
    p = torch.sigmoid(inputs)
    ce = torch.nn.functional.binary_cross_entropy_with_logits(inputs, targets, reduction="none")
    p_t = p * targets + (1 - p) * (1 - targets)
    loss = ce * (1 - p_t) ** gamma
    if alpha >= 0:
        loss = (alpha * targets + (1 - alpha) * (1 - targets)) * loss
    if reduction == "mean":
        return loss.mean()
    if reduction == "sum":
        return loss.sum()
    if reduction != "none":
        raise ValueError("sigmoid_focal_loss: reduction must be none, mean or sum, got %r" % reduction)
    return loss


focal_loss = sigmoid_focal_loss


def roi_pool(feat: torch.Tensor, rois: torch.Tensor, output_size: int | tuple[int, int], spatial_scale: float = 1.0) -> torch.Tensor:
    """RoI max pooling (Fast R-CNN): the box, rounded to feature cells, is cut into ``ph x pw`` bins (integer
    edges: floor of the start, ceil of the end) and every bin gives its maximum; empty bins give zero.
    ``rois [K, 5]`` = (batch index, x1, y1, x2, y2), or a list with one ``[k, 4]`` tensor per image."""
    if not torch.is_tensor(rois):
        rois = torch.cat([torch.cat([b.new_full((len(b), 1), i), b], 1) for i, b in enumerate(rois)])
    ph, pw = (output_size, output_size) if isinstance(output_size, int) else output_size
    N, C, H, W = feat.shape
    out = feat.new_zeros((rois.shape[0], C, ph, pw))
    import math

    def rnd(v: float) -> int:                                  # halves away from zero, as C's round()
        return int(math.floor(abs(v) + 0.5)) * (1 if v >= 0 else -1)

    r = rois.detach().cpu().double().tolist()
    for k in range(rois.shape[0]):
        n = int(r[k][0])
        x1, y1, x2, y2 = (rnd(r[k][j] * spatial_scale) for j in range(1, 5))
        rw, rh = max(x2 - x1 + 1, 1), max(y2 - y1 + 1, 1)
        for i in range(ph):
            hs = min(max(math.floor(i * rh / ph) + y1, 0), H)
            he = min(max(math.ceil((i + 1) * rh / ph) + y1, 0), H)
            for j in range(pw):
                ws = min(max(math.floor(j * rw / pw) + x1, 0), W)
                we = min(max(math.ceil((j + 1) * rw / pw) + x1, 0), W)
                if he > hs and we > ws:
                    out[k, :, i, j] = feat[n, :, hs:he, ws:we].amax((-2, -1))
    return out


def _host_lib():
    """The native host library with the prototypes of its detection entry points set (``None`` when
    it cannot be built or loaded)."""
    import ctypes

    from .. import _native

    lib = _native.host(required=False)
    if lib is not None and not getattr(lib, "_ftd_ready", False):
        vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
        lib.ftd_nms.restype, lib.ftd_nms.argtypes = ll, [vp, ll, cf, vp]
        lib.ftd_roi_align.restype = ci
        lib.ftd_roi_align.argtypes = [vp, ci, ci, ci, ci, vp, ll, ci, ci, cf, ci, ci, vp]
        lib._ftd_ready = True
    return lib


def nms_torch(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """NMS in torch operations: one IoU matrix, then a sequential sweep over the boxes in score
    order on a boolean "suppressed" vector (the sweep is inherently serial: a box is kept only if
    no *kept* box before it overlaps it)."""
    if boxes.numel() == 0:
        return torch.empty((0,), dtype=torch.int64, device=boxes.device)
    order = scores.argsort(descending=True, stable=True)
    b = boxes[order].float()
    over = (box_iou(b, b) > iou_threshold).cpu()
    n = b.shape[0]
    dead = torch.zeros(n, dtype=torch.bool)
    keep = []
    for i in range(n):
        if dead[i]:
            continue
        keep.append(i)
        dead |= over[i]
    return order[torch.tensor(keep, dtype=torch.int64, device=boxes.device)]


def nms(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """Indices of the kept boxes, highest score first.  The boxes are sorted on their own device and
    the sweep runs in the native host library (``csrc/host/det_ops.cpp``: a candidate is compared
    only with the boxes kept so far); :func:`nms_torch` is the fallback without the library."""
    if boxes.numel() == 0:
        return torch.empty((0,), dtype=torch.int64, device=boxes.device)
    lib = _host_lib()
    if lib is None:
        return nms_torch(boxes, scores, iou_threshold)
    order = scores.argsort(descending=True, stable=True)
    b = boxes[order].detach().to("cpu", torch.float32).contiguous()
    keep = torch.empty(b.shape[0], dtype=torch.int64)
    n = lib.ftd_nms(b.data_ptr(), b.shape[0], float(iou_threshold), keep.data_ptr())
    if n < 0:
        raise RuntimeError("ftd_nms failed (%d)" % n)
    return order[keep[:n].to(boxes.device)]


def batched_nms(boxes: torch.Tensor, scores: torch.Tensor, idxs: torch.Tensor, iou_threshold: float) -> torch.Tensor:
    """NMS inside each group of ``idxs`` (class or pyramid level): groups are moved apart by more
    than the largest coordinate so that boxes of different groups never overlap."""
    if boxes.numel() == 0:
        return torch.empty((0,), dtype=torch.int64, device=boxes.device)
    offsets = idxs.to(boxes) * (boxes.max() + 1)
    return nms(boxes + offsets[:, None], scores, iou_threshold)


def clip_boxes_to_image(boxes: torch.Tensor, size: tuple[int, int]) -> torch.Tensor:
    h, w = size
    x = boxes[..., 0::2].clamp(0, w)
    y = boxes[..., 1::2].clamp(0, h)
    return torch.stack((x[..., 0], y[..., 0], x[..., 1], y[..., 1]), -1)


def remove_small_boxes(boxes: torch.Tensor, min_size: float) -> torch.Tensor:
    ws, hs = boxes[:, 2] - boxes[:, 0], boxes[:, 3] - boxes[:, 1]
    return torch.where((ws >= min_size) & (hs >= min_size))[0]


# --------------------------------------------------------------------------- box coders
def decode_boxes(deltas: torch.Tensor, anchors: torch.Tensor, weights=(1.0, 1.0, 1.0, 1.0),
                 clip: float = BBOX_XFORM_CLIP) -> torch.Tensor:
    """``(dx, dy, dw, dh)`` relative to ``anchors`` -> boxes.  ``deltas [N, 4 * C]`` decodes C boxes
    per anchor (per-class regression); ``dw / dh`` are clamped from above only."""
    anchors = anchors.to(deltas.dtype)
    w, h = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
    cx, cy = anchors[:, 0] + 0.5 * w, anchors[:, 1] + 0.5 * h
    wx, wy, ww, wh = weights
    dx, dy = deltas[:, 0::4] / wx, deltas[:, 1::4] / wy
    dw, dh = (deltas[:, 2::4] / ww).clamp(max=clip), (deltas[:, 3::4] / wh).clamp(max=clip)
    pcx, pcy = dx * w[:, None] + cx[:, None], dy * h[:, None] + cy[:, None]
    pw, ph = torch.exp(dw) * w[:, None], torch.exp(dh) * h[:, None]
    out = torch.stack((pcx - 0.5 * pw, pcy - 0.5 * ph, pcx + 0.5 * pw, pcy + 0.5 * ph), 2)
    return out.flatten(1)


def decode_ltrb(ltrb: torch.Tensor, anchors: torch.Tensor) -> torch.Tensor:
    """FCOS: distances (left, top, right, bottom) from the anchor centre in units of the anchor size."""
    cx, cy = 0.5 * (anchors[:, 0] + anchors[:, 2]), 0.5 * (anchors[:, 1] + anchors[:, 3])
    w, h = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
    d = ltrb * torch.stack((w, h, w, h), 1)
    return torch.stack((cx - d[:, 0], cy - d[:, 1], cx + d[:, 2], cy + d[:, 3]), 1)


# --------------------------------------------------------------------------- RoI align
def _bilinear(feat: torch.Tensor, y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``feat [C, H, W]`` sampled at ``y, x [...]`` with the edge rules of the RoI-align kernels:
    a point more than one pixel outside contributes 0, coordinates are clamped to ``[0, size-1]``."""
    C, H, W = feat.shape
    outside = (y < -1.0) | (y > H) | (x < -1.0) | (x > W)
    y, x = y.clamp(min=0), x.clamp(min=0)
    y0, x0 = y.floor().long(), x.floor().long()
    top, left = y0 >= H - 1, x0 >= W - 1
    y0, x0 = torch.where(top, torch.full_like(y0, H - 1), y0), torch.where(left, torch.full_like(x0, W - 1), x0)
    y1, x1 = torch.where(top, y0, y0 + 1), torch.where(left, x0, x0 + 1)
    y, x = torch.where(top, y0.to(y.dtype), y), torch.where(left, x0.to(x.dtype), x)
    ly, lx = y - y0, x - x0
    hy, hx = 1 - ly, 1 - lx
    flat = feat.reshape(C, H * W)
    g = lambda yy, xx: flat[:, (yy * W + xx).reshape(-1)].reshape((C,) + tuple(y.shape))  # noqa: E731
    val = g(y0, x0) * (hy * hx) + g(y0, x1) * (hy * lx) + g(y1, x0) * (ly * hx) + g(y1, x1) * (ly * lx)
    return val.masked_fill(outside, 0)


def roi_align_torch(feat: torch.Tensor, rois: torch.Tensor, output_size: int | tuple[int, int], spatial_scale: float = 1.0,
                    sampling_ratio: int = 2, aligned: bool = False) -> torch.Tensor:
    """RoI align in torch operations (any device, differentiable in ``feat``)."""
    ph, pw = (output_size, output_size) if isinstance(output_size, int) else output_size
    assert sampling_ratio > 0, "adaptive sampling (sampling_ratio <= 0) is not implemented"
    K, s = rois.shape[0], sampling_ratio
    out = feat.new_zeros((K, feat.shape[1], ph, pw))
    if K == 0:
        return out
    off = 0.5 if aligned else 0.0
    x1, y1 = rois[:, 1] * spatial_scale - off, rois[:, 2] * spatial_scale - off
    x2, y2 = rois[:, 3] * spatial_scale - off, rois[:, 4] * spatial_scale - off
    rw, rh = x2 - x1, y2 - y1
    if not aligned:
        rw, rh = rw.clamp(min=1.0), rh.clamp(min=1.0)
    bw, bh = rw / pw, rh / ph
    iy = (torch.arange(ph * s, device=feat.device, dtype=rois.dtype) + 0.5) / s       # sample rows in bin units
    ix = (torch.arange(pw * s, device=feat.device, dtype=rois.dtype) + 0.5) / s
    ys = y1[:, None] + iy[None, :] * bh[:, None]                                       # [K, ph*s]
    xs = x1[:, None] + ix[None, :] * bw[:, None]                                       # [K, pw*s]
    batch = rois[:, 0].long()
    for b in batch.unique().tolist():
        sel = torch.where(batch == b)[0]
        yy = ys[sel][:, :, None].expand(-1, -1, pw * s)
        xx = xs[sel][:, None, :].expand(-1, ph * s, -1)
        v = _bilinear(feat[b], yy, xx)                                                 # [C, k, ph*s, pw*s]
        v = v.reshape(v.shape[0], len(sel), ph, s, pw, s).mean((3, 5))
        out[sel] = v.permute(1, 0, 2, 3).to(out.dtype)
    return out


def roi_align(feat: torch.Tensor, rois: torch.Tensor, output_size: int | tuple[int, int], spatial_scale: float = 1.0,
              sampling_ratio: int = 2, aligned: bool = False) -> torch.Tensor:
    """``feat [N, C, H, W]``, ``rois [K, 5]`` (batch index, x1, y1, x2, y2 in image coordinates) ->
    ``[K, C, ph, pw]``: every output bin is the mean of ``sampling_ratio^2`` bilinear samples.
    fp32 host tensors outside autograd go through the native library (``ftd_roi_align``), everything
    else through :func:`roi_align_torch`."""
    if not torch.is_tensor(rois):                       # one [k, 4] tensor per image -> [K, 5] with the image index
        rois = torch.cat([torch.cat([b.new_full((len(b), 1), i), b], 1) for i, b in enumerate(rois)])
    lib = _host_lib() if (not feat.is_cuda and feat.dtype == torch.float32 and rois.shape[0] > 0
                          and not (feat.requires_grad and torch.is_grad_enabled())) else None
    if lib is None:
        return roi_align_torch(feat, rois, output_size, spatial_scale, sampling_ratio, aligned)
    ph, pw = (output_size, output_size) if isinstance(output_size, int) else output_size
    f, r = feat.detach().contiguous(), rois.detach().to(torch.float32).contiguous()
    out = torch.empty((r.shape[0], f.shape[1], ph, pw), dtype=torch.float32)
    rc = lib.ftd_roi_align(f.data_ptr(), f.shape[0], f.shape[1], f.shape[2], f.shape[3], r.data_ptr(), r.shape[0], ph, pw,
                           float(spatial_scale), int(sampling_ratio), int(bool(aligned)), out.data_ptr())
    if rc != 0:
        raise RuntimeError("ftd_roi_align failed (%d)" % rc)
    return out


class MultiScaleRoIAlign:
    """RoI align over a feature pyramid: a box of area ``a`` goes to level
    ``floor(4 + log2(sqrt(a) / 224))`` clamped to the pyramid (FPN paper, eq. 1)."""

    def __init__(self, levels, output_size: int, sampling_ratio: int = 2, canonical_scale: int = 224, canonical_level: int = 4):
        self.levels, self.output_size, self.sampling_ratio = list(levels), output_size, sampling_ratio
        self.s0, self.k0 = canonical_scale, canonical_level

    def __call__(self, feats: dict, boxes: list[torch.Tensor], image_size: tuple[int, int]) -> torch.Tensor:
        fs = [feats[k] for k in self.levels]
        scales = [2.0 ** round(math.log2(f.shape[-2] / image_size[0])) for f in fs]
        rois = torch.cat([torch.cat([b.new_full((len(b), 1), i), b], 1) for i, b in enumerate(boxes)])
        if len(fs) == 1:
            return roi_align(fs[0], rois, self.output_size, scales[0], self.sampling_ratio)
        kmin, kmax = -math.log2(scales[0]), -math.log2(scales[-1])
        area = torch.cat([box_area(b) for b in boxes])
        lvl = torch.floor(self.k0 + torch.log2(area.sqrt() / self.s0) + 1e-6).clamp(kmin, kmax) - kmin
        out = fs[0].new_zeros((len(rois), fs[0].shape[1], self.output_size, self.output_size))
        for i, (f, sc) in enumerate(zip(fs, scales)):
            sel = torch.where(lvl == i)[0]
            if len(sel):
                out[sel] = roi_align(f, rois[sel], self.output_size, sc, self.sampling_ratio)
        return out


# --------------------------------------------------------------------------- anchors
class AnchorGenerator:
    """Anchors of ``sizes[l] x aspect_ratios[l]`` at every cell of pyramid level ``l``, in image
    coordinates; the cell stride is ``image size // feature size``."""

    def __init__(self, sizes=((32,), (64,), (128,), (256,), (512,)), aspect_ratios=((0.5, 1.0, 2.0),) * 5):
        self.sizes, self.aspect_ratios = sizes, aspect_ratios

    def num_anchors_per_location(self) -> list[int]:
        return [len(s) * len(a) for s, a in zip(self.sizes, self.aspect_ratios)]

    # ---- the reference's entry points (ferrotorch-vision/src/models/detection/anchor_utils.rs:50-230)
    @classmethod
    def default_fasterrcnn(cls) -> "AnchorGenerator":
        """Sizes 32 .. 512, one per pyramid level p2 .. p6, aspect ratios 0.5 / 1 / 2."""
        return cls()

    CANONICAL_STRIDES = (4, 8, 16, 32, 64)

    def generate_anchors(self, level: int, grid_size: tuple[int, int], stride: int | None = None, dtype=torch.float32, device="cpu"
                         ) -> torch.Tensor:
        """Anchors of one level on a ``(h, w)`` grid with the level's canonical square stride (4, 8, ...
        for p2, p3, ...), ``[h * w * A, 4]``."""
        s = stride if stride is not None else self.CANONICAL_STRIDES[level]
        fh, fw = grid_size
        one = AnchorGenerator((self.sizes[level],), (self.aspect_ratios[level],))
        return one((fh * s, fw * s), [(fh, fw)], dtype, device)

    def generate_anchors_for_image(self, level: int, grid_size: tuple[int, int], image_size: tuple[int, int], dtype=torch.float32,
                                   device="cpu") -> torch.Tensor:
        """The same with strides taken from the actual image: ``image_h // grid_h`` and ``image_w // grid_w``
        (what ``__call__`` does for every level), which differs from the canonical stride at the coarse
        levels of images whose size is not a multiple of 64."""
        one = AnchorGenerator((self.sizes[level],), (self.aspect_ratios[level],))
        return one(tuple(image_size), [tuple(grid_size)], dtype, device)

    @staticmethod
    def _cell(scales, ratios, dtype, device):
        scales = torch.as_tensor(scales, dtype=dtype, device=device)
        h_r = torch.as_tensor(ratios, dtype=dtype, device=device).sqrt()
        ws, hs = ((1 / h_r)[:, None] * scales[None, :]).reshape(-1), (h_r[:, None] * scales[None, :]).reshape(-1)
        return (torch.stack([-ws, -hs, ws, hs], 1) / 2).round()

    def __call__(self, image_size: tuple[int, int], feature_sizes: list[tuple[int, int]], dtype=torch.float32,
                 device="cpu") -> torch.Tensor:
        out = []
        for (fh, fw), s, a in zip(feature_sizes, self.sizes, self.aspect_ratios):
            sy, sx = image_size[0] // fh, image_size[1] // fw
            ys = torch.arange(fh, dtype=torch.int32, device=device) * sy
            xs = torch.arange(fw, dtype=torch.int32, device=device) * sx
            yy, xx = torch.meshgrid(ys, xs, indexing="ij")
            shifts = torch.stack((xx.reshape(-1), yy.reshape(-1), xx.reshape(-1), yy.reshape(-1)), 1)
            out.append((shifts[:, None, :] + self._cell(s, a, dtype, device)[None]).reshape(-1, 4))
        return torch.cat(out)


class DefaultBoxGenerator:
    """SSD default boxes: per feature map ``k`` the scales ``s_k`` and ``sqrt(s_k s_k+1)`` at aspect
    ratio 1 plus ``s_k`` at the ratios ``r`` and ``1/r``, centred on the cells, clipped to ``[0, 1]``
    and returned in pixels (``x1, y1, x2, y2``)."""

    def __init__(self, aspect_ratios, min_ratio: float = 0.15, max_ratio: float = 0.9, scales=None, steps=None, clip: bool = True):
        self.aspect_ratios, self.steps, self.clip = aspect_ratios, steps, clip
        n = len(aspect_ratios)
        if scales is None:
            scales = [min_ratio + (max_ratio - min_ratio) * k / (n - 1.0) for k in range(n)] + [1.0] if n > 1 else [min_ratio, max_ratio]
        self.scales = scales

    def num_anchors_per_location(self) -> list[int]:
        return [2 + 2 * len(r) for r in self.aspect_ratios]

    def __call__(self, image_size: tuple[int, int], feature_sizes: list[tuple[int, int]], dtype=torch.float32,
                 device="cpu") -> torch.Tensor:
        out = []
        for k, (fh, fw) in enumerate(feature_sizes):
            if self.steps is not None:
                y_f, x_f = image_size[0] / self.steps[k], image_size[1] / self.steps[k]
            else:
                y_f, x_f = fh, fw
            cy = (torch.arange(fh, dtype=dtype, device=device) + 0.5) / y_f
            cx = (torch.arange(fw, dtype=dtype, device=device) + 0.5) / x_f
            yy, xx = torch.meshgrid(cy, cx, indexing="ij")
            s, s1 = self.scales[k], math.sqrt(self.scales[k] * self.scales[k + 1])
            wh = [[s, s], [s1, s1]]
            for r in self.aspect_ratios[k]:
                q = math.sqrt(r)
                wh += [[s * q, s / q], [s / q, s * q]]
            wh = torch.as_tensor(wh, dtype=dtype, device=device)
            if self.clip:
                wh = wh.clamp(0, 1)
            centres = torch.stack((xx.reshape(-1), yy.reshape(-1)), 1)
            boxes = torch.cat((centres[:, None, :].expand(-1, len(wh), -1), wh[None].expand(len(centres), -1, -1)), 2)
            out.append(boxes.reshape(-1, 4))
        b = torch.cat(out)                                             # cx, cy, w, h in [0, 1]
        xyxy = torch.cat((b[:, :2] - 0.5 * b[:, 2:], b[:, :2] + 0.5 * b[:, 2:]), 1)
        return xyxy * torch.as_tensor([image_size[1], image_size[0]] * 2, dtype=dtype, device=device)


def roi_align_with_aligned(feat, rois, output_size, spatial_scale: float = 1.0, sampling_ratio: int = 2, aligned: bool = True):
    """:func:`roi_align` with the half-pixel shift as an explicit argument (default on)."""
    return roi_align(feat, rois, output_size, spatial_scale, sampling_ratio, aligned)
