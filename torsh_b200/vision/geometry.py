"""Geometric vision, binary features, transform classes and image loading helpers
(``crates/torsh-vision/src/{scirs2_integration,feature_detection_advanced,spatial/matching,spatial/transforms,
transforms/color,transforms/random,transforms/registry,self_supervised,utils/performance}.rs`` and
``models/advanced_cnns.rs``): Hough transforms for lines and circles, BRIEF-style binary descriptors with a brute-force
Hamming matcher, rigid alignment (Kabsch), iterative closest point, intensity-based image registration, camera pose from
point correspondences, EfficientNetV2 with fused MBConv blocks, class-style transforms with a registry, and an LRU image
cache with a background prefetcher.

Voting, matching and alignment are dense tensor operations (``index_add_``, ``cdist``-like XOR popcounts, batched SVD), so
they run unchanged on a GPU."""
from __future__ import annotations

import math
import threading
from collections import OrderedDict
from typing import Callable, Sequence

import torch
from torch import nn

from . import ops as V

__all__ = [
    "hough_lines", "hough_circles", "HoughLine", "Circle", "brief_descriptors", "hamming_distance", "BruteForceMatcher",
    "FeatureMatch", "kabsch", "icp", "ImageRegistrar", "PoseEstimator", "FusedMBConv", "EfficientNetV2", "Grayscale",
    "RandomGrayscale", "GaussianBlur", "Solarize", "BrightnessAdjust", "ContrastAdjust", "Pad", "Rotation", "RandomRotation",
    "MixUp", "TransformRegistry", "ImageCache", "ImagePrefetcher", "BatchImageLoader",
]


# ================================================================================================ Hough transforms
class HoughLine(tuple):
    """``(rho, theta, votes)``: the line ``x cos(theta) + y sin(theta) = rho``."""
    __slots__ = ()
    rho = property(lambda s: s[0]); theta = property(lambda s: s[1]); votes = property(lambda s: s[2])


class Circle(tuple):
    __slots__ = ()
    cx = property(lambda s: s[0]); cy = property(lambda s: s[1]); radius = property(lambda s: s[2]); votes = property(lambda s: s[3])


def _peaks(acc: torch.Tensor, count: int, min_votes: float, nms: int) -> list[tuple]:
    pooled = torch.nn.functional.max_pool2d(acc[None, None], 2 * nms + 1, 1, nms)[0, 0]
    cand = (acc == pooled) & (acc >= min_votes)
    idx = cand.nonzero()
    order = acc[cand].argsort(descending=True)[:count]
    return [tuple(idx[i].tolist()) + (float(acc[tuple(idx[i])]),) for i in order]


def hough_lines(edges: torch.Tensor, n_theta: int = 180, rho_res: float = 1.0, max_lines: int = 10, min_votes: float | None = None, nms: int = 5) -> list[HoughLine]:
    """Every edge pixel votes for all ``(rho, theta)`` it lies on; votes are accumulated with one ``index_add_``."""
    h, w = edges.shape
    ys, xs = edges.nonzero(as_tuple=True)
    theta = torch.arange(n_theta, dtype=torch.float64, device=edges.device) * math.pi / n_theta
    diag = math.hypot(h, w)
    n_rho = int(2 * diag / rho_res) + 1
    rho = xs.double()[:, None] * theta.cos()[None] + ys.double()[:, None] * theta.sin()[None]
    r_idx = ((rho + diag) / rho_res).round().long().clamp(0, n_rho - 1)
    acc = torch.zeros(n_rho * n_theta, dtype=torch.float32, device=edges.device)
    acc.index_add_(0, (r_idx * n_theta + torch.arange(n_theta, device=edges.device)[None]).reshape(-1), torch.ones(r_idx.numel(), device=edges.device))
    acc = acc.view(n_rho, n_theta)
    mv = min_votes if min_votes is not None else 0.3 * float(acc.max())
    return [HoughLine((r * rho_res - diag, float(theta[t]), v)) for r, t, v in _peaks(acc, max_lines, mv, nms)]


def hough_circles(edges: torch.Tensor, radii: Sequence[int], max_circles: int = 5, min_fraction: float = 0.5, n_angles: int = 90) -> list[Circle]:
    """For every radius, edge pixels vote for centres on the circle around them; a centre needs ``min_fraction`` of the
    possible votes."""
    h, w = edges.shape
    ys, xs = edges.nonzero(as_tuple=True)
    ang = torch.arange(n_angles, dtype=torch.float64, device=edges.device) * 2 * math.pi / n_angles
    found = []
    for r in radii:
        cx = (xs.double()[:, None] - r * ang.cos()[None]).round().long()
        cy = (ys.double()[:, None] - r * ang.sin()[None]).round().long()
        ok = (cx >= 0) & (cx < w) & (cy >= 0) & (cy < h)
        acc = torch.zeros(h * w, dtype=torch.float32, device=edges.device)
        acc.index_add_(0, (cy * w + cx)[ok], torch.ones(int(ok.sum()), device=edges.device))
        acc = acc.view(h, w)
        possible = min(n_angles, 2 * math.pi * r) * 1.0
        for y, x, v in _peaks(acc, max_circles, min_fraction * possible, max(2, int(r) // 2)):
            found.append(Circle((x, y, r, v / possible)))
    found.sort(key=lambda c: -c.votes)
    kept = []
    for c in found:
        if all(math.hypot(c.cx - k.cx, c.cy - k.cy) > 0.5 * min(c.radius, k.radius) or abs(c.radius - k.radius) > 0.3 * k.radius for k in kept):
            kept.append(c)
    return kept[:max_circles]


# ================================================================================================ binary descriptors
def _brief_pattern(bits: int, patch: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(bits, 4, generator=g) * patch / 5).round().clamp(-(patch // 2), patch // 2).long()


def brief_descriptors(img: torch.Tensor, keypoints: torch.Tensor, bits: int = 256, patch: int = 31, sigma: float = 2.0, seed: int = 0, oriented: bool = False) -> torch.Tensor:
    """Binary intensity-comparison descriptors packed into bytes ``(N, bits / 8)``.  ``keypoints`` are ``(N, 2)`` ``(x, y)``;
    the image is smoothed first; with ``oriented`` the sampling pattern is rotated by the patch's intensity-centroid angle
    (the ORB construction), which makes the descriptor rotation invariant."""
    g = V.gaussian_blur(img[None, None].float(), sigma)[0, 0]
    h, w = g.shape
    pat = _brief_pattern(bits, patch, seed).to(img.device).float()
    kp = keypoints.float()
    if oriented:
        r = patch // 2
        dy, dx = torch.meshgrid(torch.arange(-r, r + 1, device=img.device), torch.arange(-r, r + 1, device=img.device), indexing="ij")
        inside = (dx ** 2 + dy ** 2 <= r * r)
        px = (kp[:, 0].long()[:, None] + dx[inside][None]).clamp(0, w - 1)
        py = (kp[:, 1].long()[:, None] + dy[inside][None]).clamp(0, h - 1)
        vals = g[py, px]
        ang = torch.atan2((vals * dy[inside][None]).sum(1), (vals * dx[inside][None]).sum(1))
    else:
        ang = torch.zeros(len(kp), device=img.device)
    c, s = ang.cos()[:, None], ang.sin()[:, None]
    def sample(ox, oy):
        x = (kp[:, 0:1] + c * ox[None] - s * oy[None]).round().long().clamp(0, w - 1)
        y = (kp[:, 1:2] + s * ox[None] + c * oy[None]).round().long().clamp(0, h - 1)
        return g[y, x]
    bitsv = (sample(pat[:, 0], pat[:, 1]) < sample(pat[:, 2], pat[:, 3])).to(torch.uint8)
    weights = (2 ** torch.arange(8, device=img.device)).to(torch.uint8)
    return (bitsv.view(len(kp), bits // 8, 8) * weights).sum(-1).to(torch.uint8)


_POPCOUNT = torch.tensor([bin(i).count("1") for i in range(256)], dtype=torch.int16)


def hamming_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """All-pairs Hamming distance between packed descriptors ``(N, B)`` and ``(M, B)``."""
    x = torch.bitwise_xor(a[:, None, :], b[None, :, :]).long()
    return _POPCOUNT.to(a.device)[x].sum(-1)


class FeatureMatch(tuple):
    __slots__ = ()
    query = property(lambda s: s[0]); train = property(lambda s: s[1]); distance = property(lambda s: s[2])


class BruteForceMatcher:
    """Nearest neighbour under Hamming (uint8 descriptors) or Euclidean distance with Lowe's ratio test and optional
    mutual-consistency check."""
    def __init__(self, ratio: float = 0.8, cross_check: bool = True, max_distance: float | None = None): self.ratio, self.cross, self.max_d = ratio, cross_check, max_distance
    def match(self, d1: torch.Tensor, d2: torch.Tensor) -> list[FeatureMatch]:
        dist = hamming_distance(d1, d2).float() if d1.dtype == torch.uint8 else torch.cdist(d1.float(), d2.float())
        k = min(2, dist.shape[1])
        best = dist.topk(k, dim=1, largest=False)
        ok = torch.ones(len(d1), dtype=torch.bool, device=d1.device)
        if k == 2:
            ok &= best.values[:, 0] < self.ratio * best.values[:, 1].clamp(min=1e-12)
        if self.cross:
            ok &= dist.argmin(0)[best.indices[:, 0]] == torch.arange(len(d1), device=d1.device)
        if self.max_d is not None:
            ok &= best.values[:, 0] <= self.max_d
        return [FeatureMatch((int(i), int(best.indices[i, 0]), float(best.values[i, 0]))) for i in ok.nonzero().flatten()]


# ================================================================================================ alignment
def kabsch(src: torch.Tensor, dst: torch.Tensor, weights: torch.Tensor | None = None, with_scale: bool = False):
    """Least-squares rigid (optionally similarity) transform ``dst ~ s R src + t`` by SVD, with reflection guard."""
    w = torch.ones(len(src), dtype=src.dtype, device=src.device) if weights is None else weights
    w = w / w.sum()
    mu_s, mu_d = (w[:, None] * src).sum(0), (w[:, None] * dst).sum(0)
    xs, xd = src - mu_s, dst - mu_d
    u, sv, vt = torch.linalg.svd((w[:, None] * xd).T @ xs)
    d = torch.ones(src.shape[1], dtype=src.dtype, device=src.device)
    d[-1] = torch.sign(torch.linalg.det(u @ vt))
    rot = u @ torch.diag(d) @ vt
    scale = (sv * d).sum() / (w[:, None] * xs ** 2).sum() if with_scale else torch.ones((), dtype=src.dtype, device=src.device)
    return rot, mu_d - scale * rot @ mu_s, scale


def icp(src: torch.Tensor, dst: torch.Tensor, iters: int = 50, tol: float = 1e-8, trim: float = 1.0):
    """Point-to-point iterative closest point; ``trim < 1`` keeps only that fraction of the closest pairs per iteration
    (robust to partial overlap).  Returns rotation, translation and the RMS residual history."""
    dim = src.shape[1]
    rot, t = torch.eye(dim, dtype=src.dtype, device=src.device), torch.zeros(dim, dtype=src.dtype, device=src.device)
    hist = []
    for _ in range(iters):
        cur = src @ rot.T + t
        d, nn_idx = torch.cdist(cur, dst).min(1)
        keep = d.argsort()[: max(dim + 1, int(trim * len(src)))]
        hist.append(float(d[keep].pow(2).mean().sqrt()))
        r_step, t_step, _ = kabsch(cur[keep], dst[nn_idx[keep]])
        rot, t = r_step @ rot, r_step @ t + t_step
        if len(hist) > 1 and abs(hist[-2] - hist[-1]) < tol:
            break
    return rot, t, hist


class ImageRegistrar:
    """Intensity-based registration of ``moving`` onto ``fixed`` with an affine (or translation-only) model: Gauss-Newton
    on the sum of squared differences over a coarse-to-fine pyramid (inverse-compositional Lucas-Kanade)."""
    def __init__(self, model: str = "affine", levels: int = 3, iters: int = 30): self.model, self.levels, self.iters = model, levels, iters

    @staticmethod
    def _warp(img, p):
        h, w = img.shape
        ys, xs = torch.meshgrid(torch.arange(h, dtype=img.dtype), torch.arange(w, dtype=img.dtype), indexing="ij")
        x2 = (1 + p[0]) * xs + p[2] * ys + p[4]
        y2 = p[1] * xs + (1 + p[3]) * ys + p[5]
        grid = torch.stack([2 * x2 / (w - 1) - 1, 2 * y2 / (h - 1) - 1], -1)[None]
        return torch.nn.functional.grid_sample(img[None, None], grid, align_corners=True, padding_mode="border")[0, 0]

    def register(self, fixed: torch.Tensor, moving: torch.Tensor) -> dict:
        fixed, moving = fixed.double(), moving.double()
        p = torch.zeros(6, dtype=torch.float64)
        for lvl in reversed(range(self.levels)):
            f = torch.nn.functional.avg_pool2d(fixed[None, None], 2 ** lvl)[0, 0] if lvl else fixed
            m = torch.nn.functional.avg_pool2d(moving[None, None], 2 ** lvl)[0, 0] if lvl else moving
            h, w = f.shape
            ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float64), torch.arange(w, dtype=torch.float64), indexing="ij")
            gy, gx = torch.gradient(f)
            if self.model == "affine":
                J = torch.stack([gx * xs, gy * xs, gx * ys, gy * ys, gx, gy], -1).reshape(-1, 6)
            else:
                J = torch.stack([gx, gy], -1).reshape(-1, 2)
            Hinv = torch.linalg.inv(J.T @ J + 1e-9 * torch.eye(J.shape[1], dtype=torch.float64))
            for _ in range(self.iters):
                err = (self._warp(m, p) - f).reshape(-1)
                dp = Hinv @ (J.T @ err)
                full = torch.zeros(6, dtype=torch.float64)
                if self.model == "affine":
                    full = dp
                else:
                    full[4:] = dp
                # inverse composition: p <- p o dp^-1
                A = torch.tensor([[1 + p[0], p[2], p[4]], [p[1], 1 + p[3], p[5]], [0, 0, 1]], dtype=torch.float64)
                D = torch.tensor([[1 + full[0], full[2], full[4]], [full[1], 1 + full[3], full[5]], [0, 0, 1]], dtype=torch.float64)
                C = A @ torch.linalg.inv(D)
                p = torch.stack([C[0, 0] - 1, C[1, 0], C[0, 1], C[1, 1] - 1, C[0, 2], C[1, 2]])
                if float(dp.norm()) < 1e-6:
                    break
            if lvl:
                p = p.clone()
                p[4:] *= 2
        matrix = torch.tensor([[1 + p[0], p[2], p[4]], [p[1], 1 + p[3], p[5]]], dtype=torch.float64)
        aligned = self._warp(moving, p)
        return {"matrix": matrix, "aligned": aligned, "rmse": float((aligned - fixed).pow(2).mean().sqrt())}


class PoseEstimator:
    """Camera pose from 3-D / 2-D correspondences: direct linear transform on normalised image coordinates, projection of
    the 3x3 block onto a rotation, and the mean reprojection error in pixels."""
    def __init__(self, intrinsics: torch.Tensor): self.K = intrinsics.double()

    def estimate(self, points3d: torch.Tensor, points2d: torch.Tensor) -> dict:
        X, uv = points3d.double(), points2d.double()
        n = len(X)
        xn = (torch.linalg.inv(self.K) @ torch.cat([uv, torch.ones(n, 1, dtype=torch.float64)], 1).T).T
        Xh = torch.cat([X, torch.ones(n, 1, dtype=torch.float64)], 1)
        z = torch.zeros(n, 4, dtype=torch.float64)
        A = torch.cat([torch.cat([Xh, z, -xn[:, 0:1] * Xh], 1), torch.cat([z, Xh, -xn[:, 1:2] * Xh], 1)])
        P = torch.linalg.svd(A)[2][-1].reshape(3, 4)
        if float((P @ Xh.T)[2].mean()) < 0:
            P = -P
        u, s, vt = torch.linalg.svd(P[:, :3])
        R = u @ vt
        if float(torch.linalg.det(R)) < 0:
            R, P = -R, -P
        t = P[:, 3] / s.mean()
        return {"rotation": R, "translation": t, "reprojection_error": float((self.project(X, R, t) - uv).norm(dim=1).mean())}

    def project(self, X, R, t) -> torch.Tensor:
        cam = X.double() @ R.T + t
        pix = (self.K @ (cam / cam[:, 2:3]).T).T
        return pix[:, :2]


# ================================================================================================ EfficientNetV2
class _SE(nn.Module):
    def __init__(self, ch, reduced):
        super().__init__()
        self.fc1, self.fc2 = nn.Conv2d(ch, reduced, 1), nn.Conv2d(reduced, ch, 1)
    def forward(self, x): return x * torch.sigmoid(self.fc2(nn.functional.silu(self.fc1(x.mean((2, 3), keepdim=True)))))


class FusedMBConv(nn.Module):
    """The expansion 1x1 and depthwise 3x3 of MBConv replaced by one dense 3x3 (a single GEMM-shaped convolution that keeps
    the tensor cores busy in the early, high-resolution stages); ``fused=False`` gives the classic MBConv with SE."""
    def __init__(self, cin: int, cout: int, expand: int, stride: int, fused: bool = True, se_ratio: float = 0.25, drop_path: float = 0.0):
        super().__init__()
        mid = cin * expand
        self.residual, self.drop = stride == 1 and cin == cout, drop_path
        bn_act = lambda c: [nn.BatchNorm2d(c), nn.SiLU()]
        if fused:
            layers = [nn.Conv2d(cin, mid, 3, stride, 1, bias=False), *bn_act(mid)]
            if expand != 1:
                layers += [nn.Conv2d(mid, cout, 1, bias=False), nn.BatchNorm2d(cout)]
        else:
            layers = [nn.Conv2d(cin, mid, 1, bias=False), *bn_act(mid), nn.Conv2d(mid, mid, 3, stride, 1, groups=mid, bias=False), *bn_act(mid),
                      _SE(mid, max(1, int(cin * se_ratio))), nn.Conv2d(mid, cout, 1, bias=False), nn.BatchNorm2d(cout)]
        self.block = nn.Sequential(*layers)
    def forward(self, x):
        out = self.block(x)
        if not self.residual:
            return out
        if self.training and self.drop > 0:
            keep = (torch.rand(len(x), 1, 1, 1, device=x.device) >= self.drop).to(x.dtype) / (1 - self.drop)
            out = out * keep
        return x + out


class EfficientNetV2(nn.Module):
    """Stage table ``(expand, channels, layers, stride, fused)``; ``variant='s'`` is the published small model (~21.5 M
    parameters at 1000 classes)."""
    STAGES = {"s": [(1, 24, 2, 1, True), (4, 48, 4, 2, True), (4, 64, 4, 2, True), (4, 128, 6, 2, False), (6, 160, 9, 1, False), (6, 256, 15, 2, False)],
              "tiny": [(1, 16, 1, 1, True), (2, 24, 2, 2, True), (2, 32, 2, 2, False)]}
    def __init__(self, num_classes: int = 1000, variant: str = "s", drop_path: float = 0.0, head_dim: int = 1280):
        super().__init__()
        stages = self.STAGES[variant]
        stem = stages[0][1]
        layers = [nn.Conv2d(3, stem, 3, 2, 1, bias=False), nn.BatchNorm2d(stem), nn.SiLU()]
        total, k, cin = sum(s[2] for s in stages), 0, stem
        for expand, ch, n, stride, fused in stages:
            for i in range(n):
                layers.append(FusedMBConv(cin, ch, expand, stride if i == 0 else 1, fused, drop_path=drop_path * k / total))
                cin, k = ch, k + 1
        self.features = nn.Sequential(*layers, nn.Conv2d(cin, head_dim, 1, bias=False), nn.BatchNorm2d(head_dim), nn.SiLU())
        self.classifier = nn.Linear(head_dim, num_classes)
    def forward(self, x): return self.classifier(self.features(x).mean((2, 3)))


# ================================================================================================ transform classes
class Grayscale:
    def __init__(self, num_output_channels: int = 1): self.c = num_output_channels
    def __call__(self, x): return V.rgb_to_grayscale(x).expand(*x.shape[:-3], self.c, *x.shape[-2:]) if self.c > 1 else V.rgb_to_grayscale(x)
class _Rand:
    def __init__(self, p: float = 0.5, seed: int | None = None): self.p, self.gen = p, None if seed is None else torch.Generator().manual_seed(seed)
    def _hit(self) -> bool: return float(torch.rand((), generator=self.gen)) < self.p
    def _uniform(self, lo, hi) -> float: return lo + (hi - lo) * float(torch.rand((), generator=self.gen))
class RandomGrayscale(_Rand):
    def __call__(self, x): return Grayscale(x.shape[-3])(x) if self._hit() else x
class GaussianBlur(_Rand):
    def __init__(self, sigma=(0.1, 2.0), p: float = 1.0, seed: int | None = None):
        super().__init__(p, seed)
        self.sigma = sigma if isinstance(sigma, (tuple, list)) else (sigma, sigma)
    def __call__(self, x): return V.gaussian_blur(x, self._uniform(*self.sigma)) if self._hit() else x
class Solarize(_Rand):
    def __init__(self, threshold: float = 0.5, p: float = 1.0, seed: int | None = None):
        super().__init__(p, seed)
        self.t = threshold
    def __call__(self, x): return torch.where(x >= self.t, 1 - x, x) if self._hit() else x
class BrightnessAdjust:
    def __init__(self, factor: float): self.f = factor
    def __call__(self, x): return V.adjust_brightness(x, self.f)
class ContrastAdjust:
    def __init__(self, factor: float): self.f = factor
    def __call__(self, x): return V.adjust_contrast(x, self.f)
class Pad:
    def __init__(self, padding, mode: str = "constant", value: float = 0.0):
        p = (padding,) * 4 if isinstance(padding, int) else tuple(padding)
        self.p, self.mode, self.value = (p[0], p[0], p[1], p[1]) if len(p) == 2 else p, mode, value
    def __call__(self, x): return V.pad(x, self.p, self.mode, self.value)
class Rotation:
    def __init__(self, degrees: float): self.deg = degrees
    def __call__(self, x): return V.rotate(x, self.deg)
class RandomRotation(_Rand):
    def __init__(self, degrees, seed: int | None = None):
        super().__init__(1.0, seed)
        self.range = (-degrees, degrees) if not isinstance(degrees, (tuple, list)) else tuple(degrees)
    def __call__(self, x):
        self.last_angle = self._uniform(*self.range)
        return V.rotate(x, self.last_angle)
class MixUp(_Rand):
    """Batch transform: convex combination of the batch with a permutation of itself, labels mixed the same way."""
    def __init__(self, alpha: float = 0.2, num_classes: int | None = None, seed: int | None = None):
        super().__init__(1.0, seed)
        self.alpha, self.nc = alpha, num_classes
    def __call__(self, x, y):
        gam = torch._standard_gamma(torch.tensor([self.alpha, self.alpha], dtype=torch.float64), generator=self.gen)     # Beta(a, a) from two gammas
        lam = float(gam[0] / gam.sum().clamp(min=1e-300))
        perm = torch.randperm(len(x), generator=self.gen)
        yo = torch.nn.functional.one_hot(y, self.nc or int(y.max()) + 1).to(x.dtype) if y.dtype == torch.long else y
        self.last_lambda = lam
        return lam * x + (1 - lam) * x[perm], lam * yo + (1 - lam) * yo[perm]


class TransformRegistry:
    """Name -> transform class with keyword construction, so that pipelines can be described in configuration files:
    ``build([{"name": "GaussianBlur", "sigma": 1.0}, "Grayscale"])`` returns a composed callable."""
    def __init__(self, defaults: bool = True):
        self._t = {}
        if defaults:
            for cls in (Grayscale, RandomGrayscale, GaussianBlur, Solarize, BrightnessAdjust, ContrastAdjust, Pad, Rotation, RandomRotation):
                self._t[cls.__name__] = cls
    def register(self, name: str, factory: Callable | None = None):
        def deco(f):
            self._t[name] = f
            return f
        return deco(factory) if factory is not None else deco
    def names(self) -> list[str]: return sorted(self._t)
    def create(self, name: str, **kw):
        if name not in self._t:
            raise KeyError(f"unknown transform {name!r}; known: {self.names()}")
        return self._t[name](**kw)
    def build(self, spec: Sequence) -> Callable:
        steps = [self.create(s) if isinstance(s, str) else self.create(**{"name": s["name"]}, **{k: v for k, v in s.items() if k != "name"}) for s in spec]
        def run(x):
            for s in steps:
                x = s(x)
            return x
        run.steps = steps
        return run


# ================================================================================================ loading helpers
class ImageCache:
    """LRU cache of decoded images bounded by bytes."""
    def __init__(self, capacity_bytes: int = 256 << 20): self.cap, self.used, self.data, self.hits, self.misses, self.lock = capacity_bytes, 0, OrderedDict(), 0, 0, threading.Lock()
    def get(self, key, loader: Callable[[], torch.Tensor]) -> torch.Tensor:
        with self.lock:
            if key in self.data:
                self.hits += 1
                self.data.move_to_end(key)
                return self.data[key]
            self.misses += 1
        img = loader()
        size = img.numel() * img.element_size()
        with self.lock:
            if size <= self.cap and key not in self.data:
                self.data[key] = img
                self.used += size
                while self.used > self.cap:
                    _, old = self.data.popitem(last=False)
                    self.used -= old.numel() * old.element_size()
        return img
    def hit_rate(self) -> float: return self.hits / max(self.hits + self.misses, 1)


class ImagePrefetcher:
    """Loads the next ``depth`` items of a key sequence on background threads while the consumer works on the current one;
    iteration yields ``(key, image)`` in order."""
    def __init__(self, keys: Sequence, loader: Callable, depth: int = 4, workers: int = 2): self.keys, self.loader, self.depth, self.workers = list(keys), loader, depth, workers
    def __iter__(self):
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(self.workers) as pool:
            pending = OrderedDict()
            it = iter(self.keys)
            def fill():
                while len(pending) < self.depth:
                    k = next(it, None)
                    if k is None:
                        return
                    pending[k] = pool.submit(self.loader, k)
            fill()
            while pending:
                k, fut = pending.popitem(last=False)
                fill()
                yield k, fut.result()


class BatchImageLoader:
    """Batches of stacked images (all resized to ``size``) from keys through a cache and a prefetcher."""
    def __init__(self, keys: Sequence, loader: Callable, batch_size: int, size: tuple[int, int] | None = None, cache: ImageCache | None = None, depth: int = 8):
        self.keys, self.loader, self.bs, self.size, self.cache, self.depth = list(keys), loader, batch_size, size, cache, depth
    def _load(self, k):
        img = self.cache.get(k, lambda: self.loader(k)) if self.cache else self.loader(k)
        return V.resize(img, self.size) if self.size and tuple(img.shape[-2:]) != tuple(self.size) else img
    def __iter__(self):
        buf = []
        for _, img in ImagePrefetcher(self.keys, self._load, self.depth):
            buf.append(img)
            if len(buf) == self.bs:
                yield torch.stack(buf)
                buf = []
        if buf:
            yield torch.stack(buf)
    def __len__(self): return math.ceil(len(self.keys) / self.bs)
