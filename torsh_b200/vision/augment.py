"""Augmentation policies (``crates/torsh-vision/src/transforms/{automated,sophisticated,mixing}.rs``,
``advanced_transforms.rs``, ``self_supervised.rs``): the primitive operation table shared by AutoAugment and RandAugment,
AugMix, GridMask, Mosaic, noise / cutout / random affine transforms, and the two-view generators of SimCLR, BYOL, MoCo,
SwAV and DINO.  Operations take ``[C, H, W]`` images in ``[0, 1]``; every random choice comes from the object's own
``torch.Generator`` so a seed reproduces the stream."""
from __future__ import annotations

import math

import torch

from . import ops as V


def _posterize(x, bits): q = 2 ** (8 - int(bits)); return torch.floor(x * 255 / q) * q / 255
def _solarize(x, thr): return torch.where(x >= thr, 1 - x, x)
def _autocontrast(x): lo, hi = x.amin((-2, -1), keepdim=True), x.amax((-2, -1), keepdim=True); return torch.where(hi > lo, (x - lo) / (hi - lo).clamp(min=1e-12), x)
def _sharpness(x, f): return (x + (f - 1) * (x - V.box_blur(x, 3))).clamp(0, 1)


def _affine(x, **kw): return V.warp_affine(x, V.affine_grid_matrix(**kw))


#: name -> (function(image, magnitude value), range of the value at magnitudes 0..1, whether the sign is random)
OPS = {
    "identity": (lambda x, v: x, (0, 0), False),
    "shear_x": (lambda x, v: _affine(x, shear=(v, 0.0)), (0, 17.0), True),
    "shear_y": (lambda x, v: _affine(x, shear=(0.0, v)), (0, 17.0), True),
    "translate_x": (lambda x, v: _affine(x, translate=(v, 0.0)), (0, 0.6), True),
    "translate_y": (lambda x, v: _affine(x, translate=(0.0, v)), (0, 0.6), True),
    "rotate": (lambda x, v: V.rotate(x, v), (0, 30.0), True),
    "brightness": (lambda x, v: V.adjust_brightness(x, 1 + v), (0, 0.9), True),
    "color": (lambda x, v: V.adjust_saturation(x, 1 + v), (0, 0.9), True),
    "contrast": (lambda x, v: V.adjust_contrast(x, 1 + v), (0, 0.9), True),
    "sharpness": (lambda x, v: _sharpness(x, 1 + v), (0, 0.9), True),
    "posterize": (lambda x, v: _posterize(x, round(v)), (8, 4), False),
    "solarize": (lambda x, v: _solarize(x, v), (1.0, 0.0), False),
    "autocontrast": (lambda x, v: _autocontrast(x), (0, 0), False),
    "equalize": (lambda x, v: V.histogram_equalization(x), (0, 0), False),
    "invert": (lambda x, v: 1 - x, (0, 0), False),
}


class _Random:
    def __init__(self, seed=0): self.gen = torch.Generator().manual_seed(seed)
    def rand(self): return float(torch.rand((), generator=self.gen))
    def randint(self, n): return int(torch.randint(0, n, (), generator=self.gen))
    def uniform(self, lo, hi): return lo + (hi - lo) * self.rand()

    def apply_op(self, x, name, magnitude):
        fn, (lo, hi), signed = OPS[name]
        v = lo + (hi - lo) * magnitude
        if signed and self.rand() < 0.5:
            v = -v
        return fn(x, v)


class RandAugment(_Random):
    """``n`` operations drawn uniformly from the table, all at magnitude ``m / 30``."""

    def __init__(self, n=2, m=9, ops=None, seed=0):
        super().__init__(seed)
        self.n, self.m, self.ops = n, m, list(ops or [k for k in OPS if k != "invert"])
        self.last = []

    def __call__(self, x):
        self.last = [self.ops[self.randint(len(self.ops))] for _ in range(self.n)]
        for name in self.last:
            x = self.apply_op(x, name, self.m / 30)
        return x


class AutoAugment(_Random):
    """A policy is a list of sub-policies ``[(op, probability, magnitude 0..9), (op, probability, magnitude)]``; one
    sub-policy is drawn per image.  ``imagenet`` and ``cifar10`` are shortened forms of the published policies."""

    POLICIES = {
        "imagenet": [[("posterize", 0.4, 8), ("rotate", 0.6, 9)], [("solarize", 0.6, 5), ("autocontrast", 0.6, 5)],
                     [("equalize", 0.8, 8), ("equalize", 0.6, 3)], [("posterize", 0.6, 7), ("posterize", 0.6, 6)],
                     [("equalize", 0.4, 7), ("solarize", 0.2, 4)], [("rotate", 0.8, 8), ("color", 0.4, 0)],
                     [("color", 0.6, 4), ("contrast", 1.0, 8)], [("shear_x", 0.6, 5), ("equalize", 1.0, 9)]],
        "cifar10": [[("invert", 0.1, 7), ("contrast", 0.2, 6)], [("rotate", 0.7, 2), ("translate_x", 0.3, 9)],
                    [("sharpness", 0.8, 1), ("sharpness", 0.9, 3)], [("shear_y", 0.5, 8), ("translate_y", 0.7, 9)],
                    [("autocontrast", 0.5, 8), ("equalize", 0.9, 2)], [("color", 0.4, 3), ("brightness", 0.6, 7)]],
    }

    def __init__(self, policy="imagenet", seed=0):
        super().__init__(seed)
        self.policies = self.POLICIES[policy] if isinstance(policy, str) else policy

    def __call__(self, x):
        for name, p, mag in self.policies[self.randint(len(self.policies))]:
            if self.rand() < p:
                x = self.apply_op(x, name, mag / 9)
        return x


class AugMix(_Random):
    """Convex mixture (Dirichlet weights) of ``width`` short chains of operations, blended with the original image by a
    Beta-distributed weight; the output stays close to the input while covering many corruptions."""

    def __init__(self, width=3, depth=-1, severity=3, alpha=1.0, seed=0):
        super().__init__(seed)
        self.width, self.depth, self.severity, self.alpha = width, depth, severity, alpha
        self.ops = ["autocontrast", "equalize", "posterize", "rotate", "solarize", "shear_x", "shear_y", "translate_x", "translate_y"]

    def __call__(self, x):
        w = torch.distributions.Dirichlet(torch.full((self.width,), self.alpha)).sample().tolist() if self.width > 1 else [1.0]
        torch.manual_seed(self.randint(1 << 30))
        m = float(torch.distributions.Beta(self.alpha, self.alpha).sample())
        mix = torch.zeros_like(x)
        for wi in w:
            chain = x
            for _ in range(self.depth if self.depth > 0 else 1 + self.randint(3)):
                chain = self.apply_op(chain, self.ops[self.randint(len(self.ops))], self.severity / 10)
            mix = mix + wi * chain
        return ((1 - m) * x + m * mix).clamp(0, 1)


class GridMask(_Random):
    """Removes a regular grid of squares: period ``d`` drawn from ``d_range``, kept fraction ``ratio`` of each period."""

    def __init__(self, d_range=(8, 16), ratio=0.5, prob=1.0, seed=0):
        super().__init__(seed)
        self.d_range, self.ratio, self.prob = d_range, ratio, prob

    def mask(self, h, w):
        d = self.d_range[0] + self.randint(self.d_range[1] - self.d_range[0] + 1)
        keep = max(1, int(d * self.ratio))
        oy, ox = self.randint(d), self.randint(d)
        ys, xs = (torch.arange(h) + oy) % d, (torch.arange(w) + ox) % d
        return ~((ys[:, None] >= keep) & (xs[None, :] >= keep))

    def __call__(self, x):
        if self.rand() >= self.prob:
            return x
        return x * self.mask(*x.shape[-2:]).to(x)


class Mosaic(_Random):
    """Four images around a random centre on a ``size x size`` canvas; boxes (``xyxy``) are moved with their image and
    clipped, and boxes that shrink below ``min_box`` pixels are dropped."""

    def __init__(self, size=64, min_box=2, seed=0):
        super().__init__(seed)
        self.size, self.min_box = size, min_box

    def __call__(self, images, boxes=None):
        s = self.size
        cx, cy = int(self.uniform(0.25, 0.75) * s), int(self.uniform(0.25, 0.75) * s)
        canvas = torch.zeros(images[0].shape[0], s, s)
        out_boxes, out_src = [], []
        cells = [(0, 0, cx, cy), (cx, 0, s, cy), (0, cy, cx, s), (cx, cy, s, s)]
        for i, (img, (x0, y0, x1, y1)) in enumerate(zip(images, cells)):
            h, w = y1 - y0, x1 - x0
            ih, iw = img.shape[-2:]
            canvas[:, y0:y1, x0:x1] = V.resize(img, (h, w))
            if boxes is not None and len(boxes[i]):
                b = boxes[i] * torch.tensor([w / iw, h / ih, w / iw, h / ih]) + torch.tensor([x0, y0, x0, y0])
                b = V.clip_bbox(b, s, s)
                keep = V.filter_boxes_by_size(b, self.min_box)
                out_boxes.append(b[keep])
                out_src += [i] * len(keep)
        return (canvas, torch.cat(out_boxes) if out_boxes else torch.zeros(0, 4), torch.tensor(out_src)) if boxes is not None else canvas


def add_noise(x, kind="gaussian", amount=0.05, generator=None):
    g = generator
    if kind == "gaussian":
        return (x + amount * torch.randn(x.shape, generator=g)).clamp(0, 1)
    if kind == "salt_pepper":
        r = torch.rand(x.shape[-2:], generator=g)
        return torch.where(r < amount / 2, torch.zeros_like(x), torch.where(r > 1 - amount / 2, torch.ones_like(x), x))
    if kind == "speckle":
        return (x * (1 + amount * torch.randn(x.shape, generator=g))).clamp(0, 1)
    if kind == "poisson":
        return (torch.poisson(x.clamp(min=0) / amount, generator=g) * amount).clamp(0, 1)
    raise ValueError(f"unknown noise {kind!r}")


def cutout(x, size, generator=None, fill=0.0):
    h, w = x.shape[-2:]
    cy, cx = int(torch.randint(0, h, (), generator=generator)), int(torch.randint(0, w, (), generator=generator))
    out = x.clone()
    out[..., max(cy - size // 2, 0):cy + (size + 1) // 2, max(cx - size // 2, 0):cx + (size + 1) // 2] = fill
    return out


class RandomAffine(_Random):
    def __init__(self, degrees=15.0, translate=0.1, scale=(0.9, 1.1), shear=5.0, seed=0):
        super().__init__(seed)
        self.degrees, self.translate, self.scale, self.shear = degrees, translate, scale, shear

    def params(self):
        return dict(angle=self.uniform(-self.degrees, self.degrees), translate=(2 * self.uniform(-self.translate, self.translate), 2 * self.uniform(-self.translate, self.translate)),
                    scale=self.uniform(*self.scale), shear=(self.uniform(-self.shear, self.shear), 0.0))

    def __call__(self, x): return _affine(x, **self.params())


class RandomResizedCrop(_Random):
    def __init__(self, size, scale=(0.08, 1.0), ratio=(3 / 4, 4 / 3), seed=0):
        super().__init__(seed)
        self.size, self.scale, self.ratio = (size, size) if isinstance(size, int) else size, scale, ratio

    def __call__(self, x):
        h, w = x.shape[-2:]
        for _ in range(10):
            area = self.uniform(*self.scale) * h * w
            r = math.exp(self.uniform(math.log(self.ratio[0]), math.log(self.ratio[1])))
            cw, ch = int(round(math.sqrt(area * r))), int(round(math.sqrt(area / r)))
            if 0 < cw <= w and 0 < ch <= h:
                t, l = self.randint(h - ch + 1), self.randint(w - cw + 1)
                return V.resize(x[..., t:t + ch, l:l + cw], self.size)
        return V.resize(V.center_crop(x, (min(h, w), min(h, w))), self.size)


class _SSLView(_Random):
    """Crop -> flip -> colour jitter (with probability) -> grayscale (with probability) -> blur -> solarise."""

    def __init__(self, size, scale, jitter, p_jitter, p_gray, p_blur, p_solar, seed):
        super().__init__(seed)
        self.crop = RandomResizedCrop(size, scale, seed=seed + 1)
        self.jitter, self.p_jitter, self.p_gray, self.p_blur, self.p_solar = jitter, p_jitter, p_gray, p_blur, p_solar

    def __call__(self, x):
        x = self.crop(x)
        if self.rand() < 0.5:
            x = x.flip(-1)
        if self.rand() < self.p_jitter:
            b, c, s, h = self.jitter
            x = V.adjust_brightness(x, 1 + self.uniform(-b, b))
            x = V.adjust_contrast(x, 1 + self.uniform(-c, c))
            x = V.adjust_saturation(x, 1 + self.uniform(-s, s))
            x = V.adjust_hue(x, self.uniform(-h, h))
        if self.rand() < self.p_gray:
            x = V.rgb_to_grayscale(x).expand_as(x)
        if self.rand() < self.p_blur:
            x = V.gaussian_blur(x, self.uniform(0.1, 2.0))
        if self.rand() < self.p_solar:
            x = _solarize(x, 0.5)
        return x.clamp(0, 1)


class SimCLRAugmentation:
    """Two views from the same recipe (strong colour jitter, grayscale 0.2, blur 0.5)."""

    def __init__(self, size=32, strength=1.0, seed=0):
        j = (0.8 * strength, 0.8 * strength, 0.8 * strength, 0.2 * strength)
        self.views = [_SSLView(size, (0.08, 1.0), j, 0.8, 0.2, 0.5, 0.0, seed), _SSLView(size, (0.08, 1.0), j, 0.8, 0.2, 0.5, 0.0, seed + 100)]

    def generate_pair(self, x): return self.views[0](x), self.views[1](x)


class BYOLAugmentation(SimCLRAugmentation):
    """Asymmetric views: the first always blurs, the second rarely blurs and sometimes solarises."""

    def __init__(self, size=32, seed=0):
        j = (0.4, 0.4, 0.2, 0.1)
        self.views = [_SSLView(size, (0.08, 1.0), j, 0.8, 0.2, 1.0, 0.0, seed), _SSLView(size, (0.08, 1.0), j, 0.8, 0.2, 0.1, 0.2, seed + 100)]


class MoCoAugmentation(SimCLRAugmentation):
    def __init__(self, size=32, seed=0):
        j = (0.4, 0.4, 0.4, 0.1)
        self.views = [_SSLView(size, (0.2, 1.0), j, 0.8, 0.2, 0.5, 0.0, seed), _SSLView(size, (0.2, 1.0), j, 0.8, 0.2, 0.5, 0.0, seed + 100)]


class SwAVAugmentation:
    """Multi-crop: ``n_global`` large crops and ``n_local`` small, lower-resolution crops."""

    def __init__(self, global_size=32, local_size=16, n_global=2, n_local=4, seed=0):
        j = (0.8, 0.8, 0.8, 0.2)
        self.views = [_SSLView(global_size, (0.14, 1.0), j, 0.8, 0.2, 0.5, 0.0, seed + i) for i in range(n_global)]
        self.views += [_SSLView(local_size, (0.05, 0.14), j, 0.8, 0.2, 0.5, 0.0, seed + 50 + i) for i in range(n_local)]

    def generate_views(self, x): return [v(x) for v in self.views]


class DINOAugmentation(SwAVAugmentation):
    """Multi-crop with the asymmetric blur / solarise settings on the two global views."""

    def __init__(self, global_size=32, local_size=16, n_local=6, seed=0):
        j = (0.4, 0.4, 0.2, 0.1)
        self.views = [_SSLView(global_size, (0.4, 1.0), j, 0.8, 0.2, 1.0, 0.0, seed), _SSLView(global_size, (0.4, 1.0), j, 0.8, 0.2, 0.1, 0.2, seed + 1)]
        self.views += [_SSLView(local_size, (0.05, 0.4), j, 0.8, 0.2, 0.5, 0.0, seed + 50 + i) for i in range(n_local)]


def nt_xent_loss(z1, z2, temperature=0.5):
    """The SimCLR objective: each embedding's positive is the other view of the same image, all others are negatives."""
    z = torch.nn.functional.normalize(torch.cat([z1, z2]), dim=1)
    n = z1.shape[0]
    sim = z @ z.t() / temperature
    sim.fill_diagonal_(float("-inf"))
    target = torch.cat([torch.arange(n, 2 * n), torch.arange(0, n)]).to(z.device)
    return torch.nn.functional.cross_entropy(sim, target)


def byol_loss(p_online, z_target):
    return (2 - 2 * (torch.nn.functional.normalize(p_online, dim=1) * torch.nn.functional.normalize(z_target.detach(), dim=1)).sum(1)).mean()
