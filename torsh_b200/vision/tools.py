"""Vision tooling (``crates/torsh-vision/src``): drawing and grids, annotation sessions with COCO export and an SVG / HTML viewer
(``interactive.rs``, ``utils/``), further attribution methods (``explainability.rs``), tiled processing of large images, buffer
pools and batch-size estimation (``memory.rs``), device / precision policy (``hardware.rs``), video clips with temporal
transforms, dense optical flow, flow-based interpolation, shot detection, stabilisation and animated PNG output
(``video.rs``, ``streaming.rs``) and transform throughput benchmarks (``benchmarks.rs``)."""
from __future__ import annotations

import html
import json
import math
import struct
import time
import zlib
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.nn.functional as F
from torch import nn

_PALETTE = torch.tensor([[230, 25, 75], [60, 180, 75], [255, 225, 25], [0, 130, 200], [245, 130, 48], [145, 30, 180], [70, 240, 240], [240, 50, 230], [210, 245, 60], [0, 128, 128]], dtype=torch.uint8)


# ================================================================================================ drawing
def _as_rgb_u8(img: torch.Tensor) -> torch.Tensor:
    img = img.clone()
    if img.is_floating_point():
        img = (img.clamp(0, 1) * 255).round().to(torch.uint8)
    return img.expand(3, -1, -1).clone() if img.shape[0] == 1 else img


def draw_boxes(img: torch.Tensor, boxes: torch.Tensor, colors: torch.Tensor | None = None, width: int = 1, fill_alpha: float = 0.0) -> torch.Tensor:
    """``[3, H, W]`` image with ``xyxy`` boxes drawn (outline of ``width`` pixels, optional translucent fill)."""
    out = _as_rgb_u8(img)
    H, W = out.shape[-2:]
    for i, b in enumerate(boxes.round().long().tolist()):
        c = (colors[i] if colors is not None else _PALETTE[i % len(_PALETTE)]).to(torch.uint8)[:, None, None]
        x0, y0, x1, y1 = max(b[0], 0), max(b[1], 0), min(b[2], W - 1), min(b[3], H - 1)
        if x1 < x0 or y1 < y0:
            continue
        if fill_alpha:
            region = out[:, y0:y1 + 1, x0:x1 + 1].float()
            out[:, y0:y1 + 1, x0:x1 + 1] = (region * (1 - fill_alpha) + c.float() * fill_alpha).round().to(torch.uint8)
        for w in range(width):
            ya, yb, xa, xb = min(y0 + w, y1), max(y1 - w, y0), min(x0 + w, x1), max(x1 - w, x0)
            out[:, ya, x0:x1 + 1], out[:, yb, x0:x1 + 1], out[:, y0:y1 + 1, xa], out[:, y0:y1 + 1, xb] = c[:, 0], c[:, 0], c[:, 0], c[:, 0]
    return out


def draw_keypoints(img: torch.Tensor, points: torch.Tensor, radius: int = 2, connections: Sequence[tuple[int, int]] = (), color=(255, 0, 0)) -> torch.Tensor:
    out = _as_rgb_u8(img)
    H, W = out.shape[-2:]
    c = torch.tensor(color, dtype=torch.uint8)[:, None]
    yy, xx = torch.meshgrid(torch.arange(H), torch.arange(W), indexing="ij")
    for a, b in connections:
        n = int(max((points[a] - points[b]).abs().max().item(), 1)) * 2
        t = torch.linspace(0, 1, n)[:, None]
        line = (points[a][None] * (1 - t) + points[b][None] * t).round().long()
        ok = (line[:, 0] >= 0) & (line[:, 0] < W) & (line[:, 1] >= 0) & (line[:, 1] < H)
        out[:, line[ok, 1], line[ok, 0]] = c
    for p in points:
        m = (xx - p[0]) ** 2 + (yy - p[1]) ** 2 <= radius ** 2
        out[:, m] = c
    return out


def draw_segmentation_masks(img: torch.Tensor, masks: torch.Tensor, alpha: float = 0.5, colors: torch.Tensor | None = None) -> torch.Tensor:
    out = _as_rgb_u8(img).float()
    for i, m in enumerate(masks.bool()):
        c = (colors[i] if colors is not None else _PALETTE[i % len(_PALETTE)]).float()[:, None]
        out[:, m] = out[:, m] * (1 - alpha) + c * alpha
    return out.round().to(torch.uint8)


def make_grid(images: torch.Tensor | Sequence[torch.Tensor], nrow: int = 8, padding: int = 2, pad_value: float = 0.0, normalize: bool = False) -> torch.Tensor:
    imgs = torch.stack(list(images)) if not isinstance(images, torch.Tensor) else images
    if normalize:
        lo, hi = imgs.amin((1, 2, 3), keepdim=True), imgs.amax((1, 2, 3), keepdim=True)
        imgs = (imgs - lo) / (hi - lo).clamp_min(1e-12)
    n, c, h, w = imgs.shape
    cols = min(nrow, n); rows = math.ceil(n / cols)
    grid = torch.full((c, rows * (h + padding) + padding, cols * (w + padding) + padding), pad_value, dtype=imgs.dtype)
    for i in range(n):
        r, col = divmod(i, cols)
        y, x = padding + r * (h + padding), padding + col * (w + padding)
        grid[:, y:y + h, x:x + w] = imgs[i]
    return grid


# ================================================================================================ annotation sessions
@dataclass
class Annotation:
    id: int
    kind: str                                                                        # "box", "point", "polygon"
    label: str
    coords: list
    score: float | None = None
    attributes: dict = field(default_factory=dict)


class AnnotationSession:
    """Editable annotations of one image with undo, label statistics, COCO export and an SVG overlay for viewing."""

    def __init__(self, width: int, height: int, image_name: str = "image"): self.w, self.h, self.name, self.items, self._next, self._undo = width, height, image_name, {}, 1, []

    def add(self, kind: str, label: str, coords: Sequence[float], **kw) -> int:
        if kind == "box" and not (len(coords) == 4 and coords[2] > coords[0] and coords[3] > coords[1]):
            raise ValueError("a box is x0, y0, x1, y1 with positive size")
        if kind == "polygon" and (len(coords) < 6 or len(coords) % 2):
            raise ValueError("a polygon needs at least three x, y pairs")
        a = Annotation(self._next, kind, label, list(coords), **kw)
        self.items[a.id] = a; self._next += 1; self._undo.append(("remove", a.id))
        return a.id

    def remove(self, ann_id: int): a = self.items.pop(ann_id); self._undo.append(("restore", a))
    def relabel(self, ann_id: int, label: str): self._undo.append(("relabel", ann_id, self.items[ann_id].label)); self.items[ann_id].label = label
    def move(self, ann_id: int, dx: float, dy: float):
        a = self.items[ann_id]; self._undo.append(("coords", ann_id, list(a.coords)))
        a.coords = [v + (dx if i % 2 == 0 else dy) for i, v in enumerate(a.coords)]

    def undo(self) -> bool:
        if not self._undo:
            return False
        op = self._undo.pop()
        if op[0] == "remove":
            self.items.pop(op[1], None)
        elif op[0] == "restore":
            self.items[op[1].id] = op[1]
        elif op[0] == "relabel":
            self.items[op[1]].label = op[2]
        else:
            self.items[op[1]].coords = op[2]
        return True

    def statistics(self) -> dict:
        from collections import Counter
        boxes = [a for a in self.items.values() if a.kind == "box"]
        areas = [(a.coords[2] - a.coords[0]) * (a.coords[3] - a.coords[1]) for a in boxes]
        return {"count": len(self.items), "labels": dict(Counter(a.label for a in self.items.values())), "kinds": dict(Counter(a.kind for a in self.items.values())), "mean_box_area": sum(areas) / len(areas) if areas else 0.0,
                "coverage": min(1.0, sum(areas) / (self.w * self.h))}

    @staticmethod
    def _poly_area(c): xs, ys = c[0::2], c[1::2]; return abs(sum(xs[i] * ys[(i + 1) % len(xs)] - xs[(i + 1) % len(xs)] * ys[i] for i in range(len(xs)))) / 2

    def to_coco(self, image_id: int = 1) -> dict:
        cats = {l: i + 1 for i, l in enumerate(sorted({a.label for a in self.items.values()}))}
        anns = []
        for a in self.items.values():
            d = {"id": a.id, "image_id": image_id, "category_id": cats[a.label], "iscrowd": 0}
            if a.kind == "box":
                x0, y0, x1, y1 = a.coords
                d.update(bbox=[x0, y0, x1 - x0, y1 - y0], area=(x1 - x0) * (y1 - y0))
            elif a.kind == "polygon":
                xs, ys = a.coords[0::2], a.coords[1::2]
                d.update(segmentation=[a.coords], bbox=[min(xs), min(ys), max(xs) - min(xs), max(ys) - min(ys)], area=self._poly_area(a.coords))
            else:
                d.update(keypoints=[a.coords[0], a.coords[1], 2], num_keypoints=1)
            if a.score is not None:
                d["score"] = a.score
            anns.append(d)
        return {"images": [{"id": image_id, "file_name": self.name, "width": self.w, "height": self.h}], "categories": [{"id": i, "name": l} for l, i in cats.items()], "annotations": anns}

    @classmethod
    def from_coco(cls, coco: dict) -> "AnnotationSession":
        im = coco["images"][0]
        s = cls(im["width"], im["height"], im["file_name"])
        names = {c["id"]: c["name"] for c in coco["categories"]}
        for a in coco["annotations"]:
            if "segmentation" in a:
                s.add("polygon", names[a["category_id"]], a["segmentation"][0], score=a.get("score"))
            elif "bbox" in a:
                x, y, w, h = a["bbox"]; s.add("box", names[a["category_id"]], [x, y, x + w, y + h], score=a.get("score"))
            else:
                s.add("point", names[a["category_id"]], a["keypoints"][:2], score=a.get("score"))
        s._undo.clear()
        return s

    def to_svg(self, image_href: str | None = None) -> str:
        labels = sorted({a.label for a in self.items.values()})
        col = lambda l: "#%02x%02x%02x" % tuple(_PALETTE[labels.index(l) % len(_PALETTE)].tolist())
        parts = [f'<svg xmlns="http://www.w3.org/2000/svg" viewBox="0 0 {self.w} {self.h}" width="{self.w}" height="{self.h}">']
        if image_href:
            parts.append(f'<image href="{html.escape(image_href)}" width="{self.w}" height="{self.h}"/>')
        for a in self.items.values():
            c, tip = col(a.label), html.escape(a.label + (f" {a.score:.2f}" if a.score is not None else ""))
            if a.kind == "box":
                x0, y0, x1, y1 = a.coords
                parts.append(f'<rect x="{x0}" y="{y0}" width="{x1 - x0}" height="{y1 - y0}" fill="none" stroke="{c}" stroke-width="2"><title>{tip}</title></rect><text x="{x0 + 2}" y="{y0 + 12}" fill="{c}" font-size="11">{tip}</text>')
            elif a.kind == "polygon":
                pts = " ".join(f"{x},{y}" for x, y in zip(a.coords[0::2], a.coords[1::2]))
                parts.append(f'<polygon points="{pts}" fill="{c}" fill-opacity="0.3" stroke="{c}"><title>{tip}</title></polygon>')
            else:
                parts.append(f'<circle cx="{a.coords[0]}" cy="{a.coords[1]}" r="3" fill="{c}"><title>{tip}</title></circle>')
        return "".join(parts) + "</svg>"


def html_gallery(sessions: Sequence[AnnotationSession], title: str = "Annotations", hrefs: Sequence[str] | None = None) -> str:
    cells = "".join(f"<figure>{s.to_svg(hrefs[i] if hrefs else None)}<figcaption>{html.escape(s.name)}: {s.statistics()['count']} annotations</figcaption></figure>" for i, s in enumerate(sessions))
    return f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(title)}</title><style>figure{{display:inline-block;margin:8px;border:1px solid #999}}</style></head><body><h1>{html.escape(title)}</h1>{cells}</body></html>"


# ================================================================================================ attribution
def occlusion_sensitivity(model: nn.Module, x: torch.Tensor, target: int, patch: int = 4, stride: int | None = None, baseline: float = 0.0, batch: int = 64) -> torch.Tensor:
    """Drop of the target score when a patch is replaced by ``baseline``, averaged over the patches covering each pixel."""
    stride = stride or patch
    _, H, W = x.shape
    model.eval()
    with torch.no_grad():
        ref = model(x[None])[0, target]
        heat, cnt, jobs = torch.zeros(H, W), torch.zeros(H, W), [(y, xx) for y in range(0, H - patch + 1, stride) for xx in range(0, W - patch + 1, stride)]
        for s in range(0, len(jobs), batch):
            chunk = jobs[s:s + batch]
            xs = x[None].repeat(len(chunk), 1, 1, 1)
            for i, (y, xx) in enumerate(chunk):
                xs[i, :, y:y + patch, xx:xx + patch] = baseline
            drop = ref - model(xs)[:, target]
            for (y, xx), d in zip(chunk, drop):
                heat[y:y + patch, xx:xx + patch] += d; cnt[y:y + patch, xx:xx + patch] += 1
    return heat / cnt.clamp_min(1)


def smooth_grad(model: nn.Module, x: torch.Tensor, target: int, samples: int = 16, noise: float = 0.1, generator: torch.Generator | None = None) -> torch.Tensor:
    """Mean absolute input gradient over noisy copies of the input (noise scaled by the input's range)."""
    model.eval()
    sigma = noise * float(x.max() - x.min())
    xs = (x[None] + sigma * torch.randn(samples, *x.shape, generator=generator)).requires_grad_(True)
    model(xs)[:, target].sum().backward()
    return xs.grad.abs().mean(0).sum(0)


def attention_rollout(attentions: Sequence[torch.Tensor], discard_ratio: float = 0.0) -> torch.Tensor:
    """Combines per-layer attention ``[heads, tokens, tokens]`` into input attribution: average heads, add the identity for
    the residual path, renormalise rows and multiply through the layers."""
    n = attentions[0].shape[-1]
    roll = torch.eye(n, dtype=attentions[0].dtype)
    for a in attentions:
        m = a.mean(0)
        if discard_ratio:
            flat = m.flatten()
            k = int(flat.numel() * discard_ratio)
            if k:
                idx = flat.topk(k, largest=False).indices
                flat = flat.clone(); flat[idx[idx != 0]] = 0
                m = flat.view_as(m)
        m = m + torch.eye(n, dtype=m.dtype)
        roll = (m / m.sum(-1, keepdim=True)) @ roll
    return roll


def activation_maximization(model: nn.Module, shape: Sequence[int], unit: Callable[[torch.Tensor], torch.Tensor], steps: int = 100, lr: float = 0.1, l2: float = 1e-3, generator: torch.Generator | None = None) -> torch.Tensor:
    """Input that maximises ``unit(model(x))`` by gradient ascent with an L2 penalty (what a unit responds to)."""
    model.eval()
    x = (0.01 * torch.randn(1, *shape, generator=generator)).requires_grad_(True)
    opt = torch.optim.Adam([x], lr=lr)
    for _ in range(steps):
        opt.zero_grad(); (-unit(model(x)).sum() + l2 * x.pow(2).sum()).backward(); opt.step()
    return x.detach()[0]


# ================================================================================================ memory
class TiledProcessor:
    """Applies a shape-preserving (or integer-upscaling) function to a large image tile by tile: tiles overlap by ``overlap``
    pixels and are blended with a linear ramp, so that no seam shows and peak memory is that of one tile."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], tile: int = 256, overlap: int = 16, scale: int = 1): self.fn, self.tile, self.overlap, self.scale = fn, tile, overlap, scale

    def __call__(self, img: torch.Tensor) -> torch.Tensor:
        C, H, W = img.shape
        s, step = self.scale, self.tile - self.overlap
        out, weight = None, torch.zeros(1, H * s, W * s, dtype=torch.float32)
        ys = sorted({min(y, max(H - self.tile, 0)) for y in range(0, max(H - self.overlap, 1), step)})
        xs = sorted({min(x, max(W - self.tile, 0)) for x in range(0, max(W - self.overlap, 1), step)})
        self.tiles = 0
        for y in ys:
            for x in xs:
                t = self.fn(img[None, :, y:y + self.tile, x:x + self.tile])[0].float()
                th, tw = t.shape[-2:]
                ramp = lambda n, first, last: torch.minimum(torch.ones(n) if first else (torch.arange(n) + 1).float() / (self.overlap * s + 1), torch.ones(n) if last else (n - torch.arange(n)).float() / (self.overlap * s + 1)).clamp(max=1)
                wy, wx = ramp(th, y == 0, y + self.tile >= H), ramp(tw, x == 0, x + self.tile >= W)
                w = wy[:, None] * wx[None]
                if out is None:
                    out = torch.zeros(t.shape[0], H * s, W * s, dtype=torch.float32)
                out[:, y * s:y * s + th, x * s:x * s + tw] += t * w
                weight[:, y * s:y * s + th, x * s:x * s + tw] += w
                self.tiles += 1
        return (out / weight.clamp_min(1e-12)).to(img.dtype if img.is_floating_point() else torch.float32)


class ImageBufferPool:
    """Reusable image buffers keyed by shape and dtype (avoids an allocation per frame in a pipeline)."""

    def __init__(self, max_per_key: int = 4): self.free, self.max, self.hits, self.misses = {}, max_per_key, 0, 0
    def acquire(self, shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
        key = (tuple(shape), dtype, str(device))
        lst = self.free.get(key)
        if lst:
            self.hits += 1
            return lst.pop()
        self.misses += 1
        return torch.empty(shape, dtype=dtype, device=device)
    def release(self, t: torch.Tensor):
        lst = self.free.setdefault((tuple(t.shape), t.dtype, str(t.device)), [])
        if len(lst) < self.max:
            lst.append(t)
    def bytes_held(self) -> int: return sum(t.numel() * t.element_size() for l in self.free.values() for t in l)


def estimate_batch_memory(model: nn.Module, example: torch.Tensor, training: bool = True) -> dict:
    """Bytes per sample of activations (every leaf module's output, kept for backward when training) plus the fixed cost
    of parameters, gradients and Adam state."""
    acts, hooks = [], []
    for m in model.modules():
        if not list(m.children()):
            hooks.append(m.register_forward_hook(lambda mod, i, o: acts.append(o.numel() * o.element_size()) if isinstance(o, torch.Tensor) else None))
    with torch.no_grad():
        model(example[:1])
    for h in hooks:
        h.remove()
    params = sum(p.numel() * p.element_size() for p in model.parameters())
    per_sample = sum(acts) if training else max(acts, default=0) * 2
    return {"per_sample_bytes": per_sample + example[:1].numel() * example.element_size(), "fixed_bytes": params * (4 if training else 1), "parameters_bytes": params}


def auto_batch_size(model: nn.Module, example: torch.Tensor, memory_budget: int, training: bool = True, multiple_of: int = 8, safety: float = 0.9) -> int:
    est = estimate_batch_memory(model, example, training)
    n = int((memory_budget * safety - est["fixed_bytes"]) // est["per_sample_bytes"])
    return max(1, n // multiple_of * multiple_of) if n >= multiple_of else max(1, n)


# ================================================================================================ device / precision policy
@dataclass
class HardwarePolicy:
    device: str
    dtype: torch.dtype
    channels_last: bool
    autocast: bool

    @classmethod
    def detect(cls, prefer_bf16: bool = True) -> "HardwarePolicy":
        if torch.cuda.is_available():
            return cls("cuda", torch.bfloat16 if prefer_bf16 else torch.float16, True, True)
        return cls("cpu", torch.float32, False, False)

    def prepare(self, model: nn.Module) -> nn.Module:
        model = model.to(self.device)
        if self.dtype != torch.float32:
            model = model.to(self.dtype)
        return model.to(memory_format=torch.channels_last) if self.channels_last else model

    def prepare_input(self, x: torch.Tensor) -> torch.Tensor:
        x = x.to(self.device, self.dtype if x.is_floating_point() else None, non_blocking=True)
        return x.contiguous(memory_format=torch.channels_last) if self.channels_last and x.dim() == 4 else x


# ================================================================================================ video
@dataclass
class VideoClip:
    frames: torch.Tensor                                                              # [T, C, H, W]
    fps: float = 30.0

    @property
    def duration(self): return len(self.frames) / self.fps
    def subclip(self, start: float, end: float) -> "VideoClip": return VideoClip(self.frames[int(round(start * self.fps)):int(round(end * self.fps))], self.fps)
    def subsample(self, step: int) -> "VideoClip": return VideoClip(self.frames[::step], self.fps / step)
    def reverse(self) -> "VideoClip": return VideoClip(self.frames.flip(0), self.fps)
    def speed(self, factor: float) -> "VideoClip":
        idx = torch.arange(0, len(self.frames), factor).long().clamp(max=len(self.frames) - 1)
        return VideoClip(self.frames[idx], self.fps)
    def resample_fps(self, fps: float) -> "VideoClip":
        n = max(1, int(round(self.duration * fps)))
        idx = (torch.arange(n) * self.fps / fps).round().long().clamp(max=len(self.frames) - 1)
        return VideoClip(self.frames[idx], fps)
    def temporal_crop(self, length: int, generator: torch.Generator | None = None) -> "VideoClip":
        s = int(torch.randint(0, len(self.frames) - length + 1, (1,), generator=generator))
        return VideoClip(self.frames[s:s + length], self.fps)
    def map(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "VideoClip": return VideoClip(torch.stack([fn(f) for f in self.frames]), self.fps)


def _gray(f: torch.Tensor) -> torch.Tensor: return f.float().mean(0) if f.dim() == 3 else f.float()


def _gradients(a: torch.Tensor, b: torch.Tensor):
    kx = torch.tensor([[-1.0, 1.0], [-1.0, 1.0]]) * 0.25
    ky = torch.tensor([[-1.0, -1.0], [1.0, 1.0]]) * 0.25
    kt = torch.ones(2, 2) * 0.25
    conv = lambda t, k: F.conv2d(F.pad(t[None, None], (0, 1, 0, 1), mode="replicate"), k[None, None])[0, 0]
    return conv(a, kx) + conv(b, kx), conv(a, ky) + conv(b, ky), conv(b, kt) - conv(a, kt)


def horn_schunck(a: torch.Tensor, b: torch.Tensor, alpha: float = 1.0, iters: int = 100) -> torch.Tensor:
    """Dense optical flow ``[2, H, W]`` (x and y displacement in pixels) from brightness constancy plus a smoothness term."""
    ga, gb = _gray(a), _gray(b)
    ix, iy, it = _gradients(ga, gb)
    u, v = torch.zeros_like(ga), torch.zeros_like(ga)
    k = torch.tensor([[1 / 12, 1 / 6, 1 / 12], [1 / 6, 0, 1 / 6], [1 / 12, 1 / 6, 1 / 12]])[None, None]
    avg = lambda t: F.conv2d(F.pad(t[None, None], (1, 1, 1, 1), mode="replicate"), k)[0, 0]
    for _ in range(iters):
        ub, vb = avg(u), avg(v)
        d = (ix * ub + iy * vb + it) / (alpha ** 2 + ix ** 2 + iy ** 2)
        u, v = ub - ix * d, vb - iy * d
    return torch.stack([u, v])


def lucas_kanade(a: torch.Tensor, b: torch.Tensor, window: int = 7, levels: int = 3) -> torch.Tensor:
    """Dense pyramidal Lucas-Kanade: per pixel least squares over a window, refined from coarse to fine."""
    ga, gb = _gray(a), _gray(b)
    pyr = [(ga, gb)]
    for _ in range(levels - 1):
        pyr.append(tuple(F.avg_pool2d(t[None, None], 2)[0, 0] for t in pyr[-1]))
    flow = torch.zeros(2, *pyr[-1][0].shape)
    box = lambda t: F.avg_pool2d(F.pad(t[None, None], (window // 2,) * 4, mode="replicate"), window, stride=1)[0, 0]
    for la, lb in reversed(pyr):
        if flow.shape[-2:] != la.shape:
            flow = 2 * F.interpolate(flow[None], size=la.shape, mode="bilinear", align_corners=False)[0]
        warped = warp_by_flow(lb[None], flow)[0]
        ix, iy, it = _gradients(la, warped)
        a11, a12, a22, b1, b2 = box(ix * ix), box(ix * iy), box(iy * iy), -box(ix * it), -box(iy * it)
        det = a11 * a22 - a12 * a12
        ok = det.abs() > 1e-6
        du = torch.where(ok, (a22 * b1 - a12 * b2) / det.clamp_min(1e-12).where(det > 0, det.clamp_max(-1e-12)), torch.zeros_like(det))
        dv = torch.where(ok, (a11 * b2 - a12 * b1) / det.clamp_min(1e-12).where(det > 0, det.clamp_max(-1e-12)), torch.zeros_like(det))
        flow = flow + torch.stack([du, dv])
    return flow


def warp_by_flow(img: torch.Tensor, flow: torch.Tensor) -> torch.Tensor:
    """Samples ``img [C, H, W]`` at ``(x + u, y + v)``: with the flow from frame a to frame b, warping b gives a."""
    C, H, W = img.shape
    yy, xx = torch.meshgrid(torch.arange(H, dtype=torch.float32), torch.arange(W, dtype=torch.float32), indexing="ij")
    gx, gy = (xx + flow[0]) / max(W - 1, 1) * 2 - 1, (yy + flow[1]) / max(H - 1, 1) * 2 - 1
    return F.grid_sample(img[None].float(), torch.stack([gx, gy], -1)[None], mode="bilinear", padding_mode="border", align_corners=True)[0]


def interpolate_frames(a: torch.Tensor, b: torch.Tensor, t: float = 0.5, flow: torch.Tensor | None = None) -> torch.Tensor:
    """Frame at time ``t`` between ``a`` and ``b``: both are warped part of the way along the flow and cross-faded."""
    flow = lucas_kanade(a, b) if flow is None else flow
    fa, fb = warp_by_flow(a.float(), -t * flow), warp_by_flow(b.float(), (1 - t) * flow)
    return (1 - t) * fa + t * fb


def detect_shots(frames: torch.Tensor, bins: int = 16, threshold: float = 0.4) -> list[int]:
    """Indices at which a new shot starts: histogram distance between consecutive frames above ``threshold`` (and a local
    maximum, so a gradual change fires once)."""
    g = frames.float().mean(1) if frames.dim() == 4 else frames.float()
    g = g / g.max().clamp_min(1e-12)
    hists = torch.stack([torch.histc(f, bins, 0.0, 1.0) / f.numel() for f in g])
    d = 0.5 * (hists[1:] - hists[:-1]).abs().sum(1)
    return [i + 1 for i in range(len(d)) if d[i] > threshold and (i == 0 or d[i] >= d[i - 1]) and (i == len(d) - 1 or d[i] > d[i + 1])]


def phase_correlation(a: torch.Tensor, b: torch.Tensor) -> tuple[int, int]:
    """Integer translation ``(dx, dy)`` that moves ``a`` onto ``b`` from the peak of the normalised cross-power spectrum."""
    fa, fb = torch.fft.fft2(_gray(a)), torch.fft.fft2(_gray(b))
    r = fb * fa.conj()
    c = torch.fft.ifft2(r / r.abs().clamp_min(1e-12)).real
    idx = int(c.argmax())
    dy, dx = divmod(idx, c.shape[1])
    H, W = c.shape
    return (dx - W if dx > W // 2 else dx), (dy - H if dy > H // 2 else dy)


def stabilize(frames: torch.Tensor, smoothing: int = 5) -> tuple[torch.Tensor, torch.Tensor]:
    """Removes camera shake: the accumulated inter-frame translation is smoothed with a moving average and every frame is
    shifted by the difference between the smooth and the actual path.  Returns the frames and the corrections applied."""
    steps = torch.tensor([[0, 0]] + [list(phase_correlation(frames[i], frames[i + 1])) for i in range(len(frames) - 1)], dtype=torch.float32)
    path = steps.cumsum(0)
    k = torch.ones(1, 1, smoothing) / smoothing
    pad = smoothing // 2
    smooth = F.conv1d(F.pad(path.T[:, None], (pad, pad), mode="replicate"), k)[:, 0].T
    corr = (smooth - path).round().long()
    out = torch.stack([torch.roll(f, shifts=(int(c[1]), int(c[0])), dims=(-2, -1)) for f, c in zip(frames, corr)])
    return out, corr


def encode_apng(frames: torch.Tensor, fps: float = 10.0, loops: int = 0) -> bytes:
    """Animated PNG from ``[T, C, H, W]`` uint8 (or float in ``[0, 1]``) frames with one or three channels: a standard PNG of the
    first frame plus ``acTL`` / ``fcTL`` / ``fdAT`` chunks, so that any PNG reader shows at least the first frame."""
    if frames.is_floating_point():
        frames = (frames.clamp(0, 1) * 255).round().to(torch.uint8)
    T, C, H, W = frames.shape
    chunk = lambda tag, data: struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    def raw(f): return zlib.compress(b"".join(b"\x00" + row.tobytes() for row in f.permute(1, 2, 0).contiguous().numpy()), 6)
    out = [b"\x89PNG\r\n\x1a\n", chunk(b"IHDR", struct.pack(">IIBBBBB", W, H, 8, 0 if C == 1 else 2, 0, 0, 0)), chunk(b"acTL", struct.pack(">II", T, loops))]
    den = 1000
    num, seq = int(round(den / fps)), 0
    for i, f in enumerate(frames):
        out.append(chunk(b"fcTL", struct.pack(">IIIIIHHBB", seq, W, H, 0, 0, num, den, 0, 0))); seq += 1
        if i == 0:
            out.append(chunk(b"IDAT", raw(f)))
        else:
            out.append(chunk(b"fdAT", struct.pack(">I", seq) + raw(f))); seq += 1
    out.append(chunk(b"IEND", b""))
    return b"".join(out)


def decode_apng(data: bytes) -> tuple[torch.Tensor, float]:
    """Frames and frame rate of a file written by :func:`encode_apng` (full-frame, non-interlaced, filter type 0)."""
    pos, frames, W = 8, [], None
    delay = (1, 10)
    while pos < len(data):
        (n,), tag = struct.unpack(">I", data[pos:pos + 4]), data[pos + 4:pos + 8]
        body = data[pos + 8:pos + 8 + n]
        if zlib.crc32(tag + body) & 0xFFFFFFFF != struct.unpack(">I", data[pos + 8 + n:pos + 12 + n])[0]:
            raise ValueError(f"bad CRC in {tag!r} chunk")
        if tag == b"IHDR":
            W, H, _, ctype = struct.unpack(">IIBB", body[:10]); C = 1 if ctype == 0 else 3
        elif tag == b"fcTL":
            delay = struct.unpack(">HH", body[20:24])
        elif tag in (b"IDAT", b"fdAT"):
            rawb = zlib.decompress(body if tag == b"IDAT" else body[4:])
            rows = torch.frombuffer(bytearray(rawb), dtype=torch.uint8).reshape(H, 1 + W * C)[:, 1:]
            frames.append(rows.reshape(H, W, C).permute(2, 0, 1).clone())
        pos += 12 + n
    return torch.stack(frames), delay[1] / delay[0]


# ================================================================================================ benchmarks
def benchmark_transforms(transforms: dict[str, Callable[[torch.Tensor], torch.Tensor]], image: torch.Tensor, iterations: int = 20) -> dict:
    rows = {}
    for name, fn in transforms.items():
        fn(image)
        t0 = time.perf_counter()
        for _ in range(iterations):
            out = fn(image)
        dt = (time.perf_counter() - t0) / iterations
        rows[name] = {"ms": dt * 1e3, "images_per_s": 1 / dt, "megapixels_per_s": image.shape[-1] * image.shape[-2] / dt / 1e6, "output_shape": tuple(out.shape)}
    return rows
