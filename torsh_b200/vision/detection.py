"""Object detection: anchor generation, box coding, a feature pyramid, RetinaNet- and SSD-style detectors over any
backbone that returns a list of feature maps, YOLO-style grid decoding, and the shared post-processing (score threshold,
per-class NMS, top-k). Reference: crates/torsh-vision/src/models/detection.rs (YOLOv5, RetinaNet, SSD, Detection,
BoundingBox).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from . import box_iou, nms


@dataclass
class BoundingBox:
    x1: float
    y1: float
    x2: float
    y2: float

    def area(self) -> float:
        return max(self.x2 - self.x1, 0.0) * max(self.y2 - self.y1, 0.0)

    def center(self) -> tuple[float, float]:
        return (0.5 * (self.x1 + self.x2), 0.5 * (self.y1 + self.y2))


@dataclass
class Detection:
    box: BoundingBox
    score: float
    label: int


class AnchorGenerator:
    """Anchors ``[sum_l H_l * W_l * A, 4]`` (x1, y1, x2, y2) for feature maps with the given strides."""

    def __init__(self, sizes=(32, 64, 128, 256, 512), ratios=(0.5, 1.0, 2.0), scales=(1.0, 2 ** (1 / 3), 2 ** (2 / 3))):
        self.sizes, self.ratios, self.scales = sizes, ratios, scales

    @property
    def num_anchors(self) -> int:
        return len(self.ratios) * len(self.scales)

    def cell_anchors(self, size: float) -> torch.Tensor:
        out = []
        for r in self.ratios:
            for s in self.scales:
                area = (size * s) ** 2
                w = math.sqrt(area / r)
                h = w * r
                out.append([-w / 2, -h / 2, w / 2, h / 2])
        return torch.tensor(out)

    def __call__(self, feature_shapes, strides) -> torch.Tensor:
        all_a = []
        for (h, w), stride, size in zip(feature_shapes, strides, self.sizes):
            ys = (torch.arange(h) + 0.5) * stride
            xs = (torch.arange(w) + 0.5) * stride
            cy, cx = torch.meshgrid(ys, xs, indexing="ij")
            ctr = torch.stack([cx, cy, cx, cy], -1).reshape(-1, 1, 4)
            all_a.append((ctr + self.cell_anchors(size)[None]).reshape(-1, 4))
        return torch.cat(all_a)


class BoxCoder:
    """(dx, dy, dw, dh) regression targets relative to anchors, with the usual weights and a clamp on dw / dh."""

    def __init__(self, weights=(1.0, 1.0, 1.0, 1.0), clip: float = math.log(1000.0 / 16)):
        self.w, self.clip = weights, clip

    def encode(self, boxes, anchors):
        aw, ah = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
        ax, ay = anchors[:, 0] + 0.5 * aw, anchors[:, 1] + 0.5 * ah
        bw, bh = boxes[:, 2] - boxes[:, 0], boxes[:, 3] - boxes[:, 1]
        bx, by = boxes[:, 0] + 0.5 * bw, boxes[:, 1] + 0.5 * bh
        return torch.stack([self.w[0] * (bx - ax) / aw, self.w[1] * (by - ay) / ah, self.w[2] * torch.log(bw / aw),
                            self.w[3] * torch.log(bh / ah)], -1)

    def decode(self, deltas, anchors):
        aw, ah = anchors[:, 2] - anchors[:, 0], anchors[:, 3] - anchors[:, 1]
        ax, ay = anchors[:, 0] + 0.5 * aw, anchors[:, 1] + 0.5 * ah
        dx, dy = deltas[..., 0] / self.w[0], deltas[..., 1] / self.w[1]
        dw, dh = (deltas[..., 2] / self.w[2]).clamp(max=self.clip), (deltas[..., 3] / self.w[3]).clamp(max=self.clip)
        cx, cy, w, h = ax + dx * aw, ay + dy * ah, aw * torch.exp(dw), ah * torch.exp(dh)
        return torch.stack([cx - 0.5 * w, cy - 0.5 * h, cx + 0.5 * w, cy + 0.5 * h], -1)


def match_anchors(anchors, gt_boxes, fg_iou: float = 0.5, bg_iou: float = 0.4):
    """Index of the matched ground-truth box per anchor: >= 0 foreground, -1 background, -2 ignored (between thresholds)."""
    if gt_boxes.numel() == 0:
        return torch.full((anchors.shape[0],), -1, dtype=torch.long)
    iou = box_iou(anchors, gt_boxes)
    best, idx = iou.max(1)
    out = torch.where(best >= fg_iou, idx, torch.full_like(idx, -2))
    out[best < bg_iou] = -1
    out[iou.argmax(0)] = torch.arange(gt_boxes.shape[0])             # every ground-truth box keeps its best anchor
    return out


def postprocess(boxes, scores, score_thresh: float = 0.05, iou_thresh: float = 0.5, top_k: int = 100, image_size=None) -> list[Detection]:
    """``boxes`` [N, 4], ``scores`` [N, C]: threshold, per-class NMS, highest ``top_k``."""
    if image_size is not None:
        h, w = image_size
        boxes = torch.stack([boxes[:, 0].clamp(0, w), boxes[:, 1].clamp(0, h), boxes[:, 2].clamp(0, w), boxes[:, 3].clamp(0, h)], -1)
    dets = []
    for c in range(scores.shape[1]):
        m = scores[:, c] > score_thresh
        if not m.any():
            continue
        b, s = boxes[m], scores[m, c]
        keep = nms(b, s, iou_thresh)
        dets += [Detection(BoundingBox(*b[i].tolist()), float(s[i]), c) for i in keep.tolist()]
    dets.sort(key=lambda d: -d.score)
    return dets[:top_k]


class FeaturePyramid(nn.Module):
    """Top-down pathway with lateral 1x1 convolutions and 3x3 output convolutions; two extra stride-2 levels."""

    def __init__(self, in_channels, out_channels: int = 256, extra_levels: int = 2):
        super().__init__()
        self.lateral = nn.ModuleList(nn.Conv2d(c, out_channels, 1) for c in in_channels)
        self.output = nn.ModuleList(nn.Conv2d(out_channels, out_channels, 3, padding=1) for _ in in_channels)
        self.extra = nn.ModuleList(nn.Conv2d(out_channels, out_channels, 3, stride=2, padding=1) for _ in range(extra_levels))

    def forward(self, feats):
        lat = [l(f) for l, f in zip(self.lateral, feats)]
        for i in range(len(lat) - 2, -1, -1):
            lat[i] = lat[i] + nn.functional.interpolate(lat[i + 1], size=lat[i].shape[-2:], mode="nearest")
        outs = [o(x) for o, x in zip(self.output, lat)]
        x = outs[-1]
        for e in self.extra:
            x = e(torch.relu(x) if e is not self.extra[0] else x)
            outs.append(x)
        return outs


class _Head(nn.Module):
    def __init__(self, channels: int, out_per_anchor: int, num_anchors: int, depth: int = 4, prior: float | None = None):
        super().__init__()
        layers = []
        for _ in range(depth):
            layers += [nn.Conv2d(channels, channels, 3, padding=1), nn.ReLU(inplace=True)]
        self.tower = nn.Sequential(*layers)
        self.out = nn.Conv2d(channels, num_anchors * out_per_anchor, 3, padding=1)
        self.k = out_per_anchor
        if prior is not None:                      # focal-loss initialisation: every anchor starts as background
            nn.init.constant_(self.out.bias, -math.log((1 - prior) / prior))

    def forward(self, feats):
        outs = []
        for f in feats:
            y = self.out(self.tower(f))
            n, _, h, w = y.shape
            outs.append(y.permute(0, 2, 3, 1).reshape(n, -1, self.k))
        return torch.cat(outs, 1)


class TinyBackbone(nn.Module):
    """Three stride-8 / 16 / 32 feature maps from a small convolutional stack (for tests and as a template)."""

    def __init__(self, width: int = 32):
        super().__init__()
        def block(i, o, s): return nn.Sequential(nn.Conv2d(i, o, 3, s, 1), nn.BatchNorm2d(o), nn.ReLU(inplace=True))
        self.stem = nn.Sequential(block(3, width, 2), block(width, width, 2))
        self.c3, self.c4, self.c5 = block(width, width * 2, 2), block(width * 2, width * 4, 2), block(width * 4, width * 8, 2)
        self.out_channels = [width * 2, width * 4, width * 8]
        self.strides = [8, 16, 32]

    def forward(self, x):
        x = self.stem(x)
        c3 = self.c3(x)
        c4 = self.c4(c3)
        return [c3, c4, self.c5(c4)]


class RetinaNet(nn.Module):
    """Backbone -> FPN -> shared classification / regression towers; focal loss + smooth-L1 training loss."""

    def __init__(self, backbone: nn.Module, num_classes: int, fpn_channels: int = 256, anchors: AnchorGenerator | None = None, head_depth: int = 4):
        super().__init__()
        self.backbone, self.num_classes = backbone, num_classes
        self.fpn = FeaturePyramid(backbone.out_channels, fpn_channels)
        self.anchor_gen = anchors or AnchorGenerator()
        a = self.anchor_gen.num_anchors
        self.cls_head = _Head(fpn_channels, num_classes, a, head_depth, prior=0.01)
        self.box_head = _Head(fpn_channels, 4, a, head_depth)
        self.coder = BoxCoder()
        self.strides = list(backbone.strides) + [backbone.strides[-1] * 2 ** (i + 1) for i in range(len(self.fpn.extra))]

    def forward(self, images):
        feats = self.fpn(self.backbone(images))
        anchors = self.anchor_gen([f.shape[-2:] for f in feats], self.strides).to(images.device)
        return self.cls_head(feats), self.box_head(feats), anchors

    def loss(self, images, targets, alpha: float = 0.25, gamma: float = 2.0):
        """``targets``: list of dicts with ``boxes`` [G, 4] and ``labels`` [G]."""
        from ..nn.losses import focal_loss
        cls, reg, anchors = self(images)
        cls_loss = reg_loss = 0.0
        for i, t in enumerate(targets):
            m = match_anchors(anchors, t["boxes"])
            fg, valid = m >= 0, m != -2
            onehot = torch.zeros_like(cls[i])
            onehot[fg, t["labels"][m[fg]]] = 1.0
            nfg = max(int(fg.sum()), 1)
            cls_loss = cls_loss + focal_loss(cls[i][valid], onehot[valid], alpha, gamma, "sum") / nfg
            if fg.any():
                tgt = self.coder.encode(t["boxes"][m[fg]], anchors[fg])
                reg_loss = reg_loss + nn.functional.smooth_l1_loss(reg[i][fg], tgt, beta=1 / 9, reduction="sum") / nfg
        n = len(targets)
        return {"classification": cls_loss / n, "regression": reg_loss / n}

    @torch.no_grad()
    def detect(self, images, score_thresh: float = 0.05, iou_thresh: float = 0.5, top_k: int = 100) -> list[list[Detection]]:
        cls, reg, anchors = self(images)
        out = []
        for i in range(images.shape[0]):
            boxes = self.coder.decode(reg[i], anchors)
            out.append(postprocess(boxes, torch.sigmoid(cls[i]), score_thresh, iou_thresh, top_k, images.shape[-2:]))
        return out


class SSD(nn.Module):
    """Single-shot detector: one 3x3 prediction layer per feature map (softmax over classes + background)."""

    def __init__(self, backbone: nn.Module, num_classes: int, anchors: AnchorGenerator | None = None):
        super().__init__()
        self.backbone, self.num_classes = backbone, num_classes
        self.anchor_gen = anchors or AnchorGenerator(sizes=(32, 64, 128), ratios=(0.5, 1.0, 2.0), scales=(1.0, 1.26))
        a = self.anchor_gen.num_anchors
        self.cls = nn.ModuleList(nn.Conv2d(c, a * (num_classes + 1), 3, padding=1) for c in backbone.out_channels)
        self.reg = nn.ModuleList(nn.Conv2d(c, a * 4, 3, padding=1) for c in backbone.out_channels)
        self.coder = BoxCoder(weights=(10.0, 10.0, 5.0, 5.0))

    def forward(self, images):
        feats = self.backbone(images)
        n = images.shape[0]
        cls = torch.cat([c(f).permute(0, 2, 3, 1).reshape(n, -1, self.num_classes + 1) for c, f in zip(self.cls, feats)], 1)
        reg = torch.cat([r(f).permute(0, 2, 3, 1).reshape(n, -1, 4) for r, f in zip(self.reg, feats)], 1)
        anchors = self.anchor_gen([f.shape[-2:] for f in feats], self.backbone.strides).to(images.device)
        return cls, reg, anchors

    @torch.no_grad()
    def detect(self, images, score_thresh: float = 0.3, iou_thresh: float = 0.45, top_k: int = 100):
        cls, reg, anchors = self(images)
        return [postprocess(self.coder.decode(reg[i], anchors), torch.softmax(cls[i], -1)[:, 1:], score_thresh, iou_thresh, top_k,
                            images.shape[-2:]) for i in range(images.shape[0])]


def decode_yolo_grid(pred: torch.Tensor, anchors_wh, stride: int) -> tuple[torch.Tensor, torch.Tensor]:
    """YOLOv5 decoding of one scale: ``pred`` [N, A, H, W, 5 + C] raw outputs -> (boxes [N, A*H*W, 4] xyxy in pixels,
    scores [N, A*H*W, C] = objectness x class probability)."""
    n, a, h, w, k = pred.shape
    p = torch.sigmoid(pred)
    gy, gx = torch.meshgrid(torch.arange(h, device=pred.device), torch.arange(w, device=pred.device), indexing="ij")
    cx = (p[..., 0] * 2 - 0.5 + gx) * stride
    cy = (p[..., 1] * 2 - 0.5 + gy) * stride
    awh = torch.as_tensor(anchors_wh, dtype=pred.dtype, device=pred.device).reshape(1, a, 1, 1, 2)
    wh = (p[..., 2:4] * 2) ** 2 * awh
    boxes = torch.stack([cx - wh[..., 0] / 2, cy - wh[..., 1] / 2, cx + wh[..., 0] / 2, cy + wh[..., 1] / 2], -1)
    return boxes.reshape(n, -1, 4), (p[..., 4:5] * p[..., 5:]).reshape(n, -1, k - 5)


def retinanet_tiny(num_classes: int) -> RetinaNet:
    return RetinaNet(TinyBackbone(16), num_classes, fpn_channels=32, anchors=AnchorGenerator(sizes=(16, 32, 64, 128, 256)), head_depth=1)


def ssd_tiny(num_classes: int) -> SSD:
    return SSD(TinyBackbone(16), num_classes)
