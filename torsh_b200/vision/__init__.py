"""Vision utilities (``crates/torsh-vision``): tensor transforms and augmentations, box ops (IoU, NMS), synthetic
image dataset for benchmarks. Transforms operate on ``[C, H, W]`` or ``[N, C, H, W]`` float tensors on any device."""
from __future__ import annotations

import math
import random

import torch
import torch.nn.functional as F


class Compose:
    def __init__(self, transforms): self.transforms = list(transforms)
    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class Normalize:
    def __init__(self, mean, std):
        self.mean, self.std = torch.tensor(mean).view(-1, 1, 1), torch.tensor(std).view(-1, 1, 1)
    def __call__(self, x): return (x - self.mean.to(x)) / self.std.to(x)


class Resize:
    def __init__(self, size, mode="bilinear"): self.size, self.mode = (size, size) if isinstance(size, int) else tuple(size), mode
    def __call__(self, x):
        b = x.dim() == 3
        y = F.interpolate(x[None] if b else x, size=self.size, mode=self.mode, align_corners=False if self.mode != "nearest" else None)
        return y[0] if b else y


class CenterCrop:
    def __init__(self, size): self.size = (size, size) if isinstance(size, int) else tuple(size)
    def __call__(self, x):
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = (h - th) // 2, (w - tw) // 2
        return x[..., i:i + th, j:j + tw]


class RandomCrop(CenterCrop):
    def __init__(self, size, padding=0):
        super().__init__(size); self.padding = padding
    def __call__(self, x):
        if self.padding:
            x = F.pad(x, [self.padding] * 4)
        h, w = x.shape[-2:]
        th, tw = self.size
        i, j = random.randint(0, h - th), random.randint(0, w - tw)
        return x[..., i:i + th, j:j + tw]


class RandomHorizontalFlip:
    def __init__(self, p=0.5): self.p = p
    def __call__(self, x): return x.flip(-1) if random.random() < self.p else x


class RandomVerticalFlip(RandomHorizontalFlip):
    def __call__(self, x): return x.flip(-2) if random.random() < self.p else x


class ColorJitter:
    def __init__(self, brightness=0.0, contrast=0.0, saturation=0.0):
        self.b, self.c, self.s = brightness, contrast, saturation
    def __call__(self, x):
        if self.b: x = x * (1 + random.uniform(-self.b, self.b))
        if self.c:
            m = x.mean((-3, -2, -1), keepdim=True)
            x = (x - m) * (1 + random.uniform(-self.c, self.c)) + m
        if self.s:
            g = x.mean(-3, keepdim=True)
            x = (x - g) * (1 + random.uniform(-self.s, self.s)) + g
        return x.clamp(0, 1)


class RandomErasing:
    def __init__(self, p=0.5, scale=(0.02, 0.33)): self.p, self.scale = p, scale
    def __call__(self, x):
        if random.random() >= self.p:
            return x
        h, w = x.shape[-2:]
        a = random.uniform(*self.scale) * h * w
        eh, ew = min(h, int(math.sqrt(a))), min(w, int(math.sqrt(a)))
        i, j = random.randint(0, h - eh), random.randint(0, w - ew)
        x = x.clone(); x[..., i:i + eh, j:j + ew] = 0
        return x


def mixup(x, y, alpha=0.2):
    lam = random.betavariate(alpha, alpha) if alpha > 0 else 1.0
    perm = torch.randperm(x.shape[0], device=x.device)
    return lam * x + (1 - lam) * x[perm], y, y[perm], lam


def cutmix(x, y, alpha=1.0):
    lam = random.betavariate(alpha, alpha)
    perm = torch.randperm(x.shape[0], device=x.device)
    h, w = x.shape[-2:]
    r = math.sqrt(1 - lam)
    ch, cw = int(h * r), int(w * r)
    cy, cx = random.randint(0, h), random.randint(0, w)
    y0, y1, x0, x1 = max(cy - ch // 2, 0), min(cy + ch // 2, h), max(cx - cw // 2, 0), min(cx + cw // 2, w)
    x = x.clone(); x[..., y0:y1, x0:x1] = x[perm][..., y0:y1, x0:x1]
    return x, y, y[perm], 1 - (y1 - y0) * (x1 - x0) / (h * w)


def box_area(b): return (b[:, 2] - b[:, 0]).clamp(min=0) * (b[:, 3] - b[:, 1]).clamp(min=0)


def box_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    lt, rb = torch.max(a[:, None, :2], b[None, :, :2]), torch.min(a[:, None, 2:], b[None, :, 2:])
    inter = (rb - lt).clamp(min=0).prod(-1)
    return inter / (box_area(a)[:, None] + box_area(b)[None] - inter).clamp(min=1e-12)


def nms(boxes: torch.Tensor, scores: torch.Tensor, iou_threshold: float = 0.5) -> torch.Tensor:
    order, keep = scores.argsort(descending=True), []
    while order.numel():
        i = order[0]; keep.append(i.item())
        if order.numel() == 1:
            break
        rest = order[1:]
        order = rest[box_iou(boxes[i][None], boxes[rest])[0] <= iou_threshold]
    return torch.tensor(keep, dtype=torch.long, device=boxes.device)


class SyntheticImageDataset(torch.utils.data.Dataset):
    """N(0,1) pixels, uniform labels (the ResNet benchmark data)."""
    def __init__(self, length=1024, shape=(3, 224, 224), num_classes=1000, seed=0):
        self.n, self.shape, self.c, self.seed = length, shape, num_classes, seed
    def __len__(self): return self.n
    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 7919 + i)
        return torch.randn(self.shape, generator=g), int(torch.randint(0, self.c, (1,), generator=g))
