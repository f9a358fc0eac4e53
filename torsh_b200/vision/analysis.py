"""Classical image analysis (``crates/torsh-vision/src/{segmentation_advanced,feature_detection_advanced,streaming,viz3d}.rs``
and ``spatial/{structures,matching,interpolation,distance}.rs``):

* segmentation: connected components, seeded region growing, marker watershed, binary graph cut (max-flow);
* features: Harris / Shi-Tomasi corners, multi-scale detection, gradient-histogram descriptors, brute-force matching
  with ratio and cross checks, RANSAC filtering with a fitted homography, normalised cross-correlation template matching;
* spatial: k-d tree neighbour queries, IoU / distance object tracker, lens distortion correction, flow warping,
  scattered-data interpolation, patch and image similarity search;
* streaming: bounded frame queue with drop policy, preprocessing, batching, latency statistics and quality adaptation;
* 3-D: point clouds (voxel down-sampling, normals, filters), meshes (cube / sphere, normals, area, volume), boxes.
"""
from __future__ import annotations

import heapq
import math
import time
from collections import deque
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from . import ops as V


# ================================================================================================ segmentation
def connected_components(mask: torch.Tensor, connectivity: int = 4) -> tuple[torch.Tensor, int]:
    """Labels of a 2-D boolean mask (0 = background) by iterated minimum-label propagation (vectorised; converges in at
    most the longest path inside a component)."""
    h, w = mask.shape
    lab = torch.where(mask, torch.arange(1, h * w + 1, device=mask.device).reshape(h, w), torch.zeros(h, w, dtype=torch.long, device=mask.device))
    big = h * w + 1
    k = 3
    while True:
        cur = torch.where(mask, lab, torch.full_like(lab, big)).float()[None, None]
        if connectivity == 8:
            nxt = -F.max_pool2d(-cur, k, 1, 1)
        else:
            p = F.pad(cur, (1, 1, 1, 1), value=float(big))
            nxt = torch.minimum(torch.minimum(torch.minimum(p[..., 1:-1, :-2], p[..., 1:-1, 2:]), torch.minimum(p[..., :-2, 1:-1], p[..., 2:, 1:-1])), cur)
        nxt = torch.where(mask, nxt[0, 0].long(), torch.zeros_like(lab))
        if torch.equal(nxt, lab):
            break
        lab = nxt
    ids = lab.unique()
    ids = ids[ids > 0]
    remap = torch.zeros(big + 1, dtype=torch.long, device=mask.device)
    remap[ids] = torch.arange(1, len(ids) + 1, device=mask.device)
    return remap[lab], len(ids)


def region_growing(img: torch.Tensor, seeds, threshold: float = 0.1, connectivity: int = 4, adaptive: bool = True) -> torch.Tensor:
    """Grows one region per seed ``(y, x)``: a neighbour joins when it differs from the region mean (``adaptive``) or the
    seed value by at most ``threshold``.  Returns labels (0 = unassigned, i + 1 = seed i)."""
    g = img.squeeze().double().cpu().numpy()
    h, w = g.shape
    lab = np.zeros((h, w), np.int64)
    nb = [(-1, 0), (1, 0), (0, -1), (0, 1)] + ([(-1, -1), (-1, 1), (1, -1), (1, 1)] if connectivity == 8 else [])
    for i, (sy, sx) in enumerate(seeds):
        if lab[sy, sx]:
            continue
        ref, n, q = g[sy, sx], 1, deque([(sy, sx)])
        lab[sy, sx] = i + 1
        while q:
            y, x = q.popleft()
            for dy, dx in nb:
                yy, xx = y + dy, x + dx
                if 0 <= yy < h and 0 <= xx < w and not lab[yy, xx] and abs(g[yy, xx] - ref) <= threshold:
                    lab[yy, xx] = i + 1
                    q.append((yy, xx))
                    if adaptive:
                        ref, n = (ref * n + g[yy, xx]) / (n + 1), n + 1
    return torch.from_numpy(lab)


def watershed(img: torch.Tensor, markers: torch.Tensor | None = None, connectivity: int = 4, min_distance: int = 3) -> torch.Tensor:
    """Priority flood of a height map from labelled markers (Meyer's algorithm).  Without markers, the local minima of the
    smoothed image (at least ``min_distance`` apart) are used."""
    g = img.squeeze().double().cpu().numpy()
    h, w = g.shape
    if markers is None:
        sm = V.gaussian_blur(img.reshape(1, h, w).float(), 1.0)
        mn = (-F.max_pool2d(-sm[None], 2 * min_distance + 1, 1, min_distance)[0] == sm)[0]
        markers, _ = connected_components(mn, 8)
    lab = markers.cpu().numpy().astype(np.int64).copy()
    nb = [(-1, 0), (1, 0), (0, -1), (0, 1)] + ([(-1, -1), (-1, 1), (1, -1), (1, 1)] if connectivity == 8 else [])
    heap, order = [], 0
    for y, x in zip(*np.nonzero(lab)):
        heapq.heappush(heap, (g[y, x], order, y, x))
        order += 1
    while heap:
        _, _, y, x = heapq.heappop(heap)
        for dy, dx in nb:
            yy, xx = y + dy, x + dx
            if 0 <= yy < h and 0 <= xx < w and not lab[yy, xx]:
                lab[yy, xx] = lab[y, x]
                heapq.heappush(heap, (max(g[yy, xx], g[y, x]), order, yy, xx))
                order += 1
    return torch.from_numpy(lab)


def graph_cuts(img: torch.Tensor, fg_seeds: torch.Tensor, bg_seeds: torch.Tensor, lam: float = 20.0, sigma: float = 0.1, bins: int = 16) -> torch.Tensor:
    """Binary segmentation by minimum cut: unary terms from seed intensity histograms, pairwise terms
    ``lam * exp(-(Ip - Iq)^2 / (2 sigma^2))`` on the 4-neighbour grid, seeds pinned.  Solved with scipy's max-flow on
    integer capacities; the source side of the cut is the foreground."""
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import breadth_first_order, maximum_flow
    g = img.squeeze().double().cpu().numpy()
    h, w = g.shape
    n, src, snk, scale = h * w, h * w, h * w + 1, 1000
    fg, bg = fg_seeds.cpu().numpy().astype(bool), bg_seeds.cpu().numpy().astype(bool)
    idx = np.clip((g * bins).astype(int), 0, bins - 1)
    hist = lambda m: (np.bincount(idx[m], minlength=bins) + 1.0) / (m.sum() + bins)
    pf, pb = hist(fg)[idx], hist(bg)[idx]
    cap_s, cap_t = -np.log(pb), -np.log(pf)                                # source link pays when the pixel ends up background
    cap_s[fg], cap_t[fg] = 1e6, 0
    cap_s[bg], cap_t[bg] = 0, 1e6
    rows, cols, caps = [], [], []
    pid = np.arange(n).reshape(h, w)
    for a, b, d in ((pid[:, :-1], pid[:, 1:], g[:, :-1] - g[:, 1:]), (pid[:-1], pid[1:], g[:-1] - g[1:])):
        wgt = lam * np.exp(-d ** 2 / (2 * sigma ** 2))
        rows += [a.ravel(), b.ravel()]; cols += [b.ravel(), a.ravel()]; caps += [wgt.ravel(), wgt.ravel()]
    rows += [np.full(n, src), pid.ravel()]; cols += [pid.ravel(), np.full(n, snk)]; caps += [cap_s.ravel(), cap_t.ravel()]
    cap = csr_matrix((np.round(np.concatenate(caps) * scale).astype(np.int32), (np.concatenate(rows), np.concatenate(cols))), shape=(n + 2, n + 2))
    flow = maximum_flow(cap, src, snk).flow
    residual = cap - flow
    residual.data = np.maximum(residual.data, 0)
    residual.eliminate_zeros()
    reach = breadth_first_order(residual, src, directed=True, return_predecessors=False)
    out = np.zeros(n + 2, bool)
    out[reach] = True
    return torch.from_numpy(out[:n].reshape(h, w))


# ================================================================================================ features
@dataclass
class Keypoints:
    xy: torch.Tensor            # [N, 2] (x, y)
    response: torch.Tensor      # [N]
    scale: torch.Tensor         # [N]


def corner_response(img: torch.Tensor, sigma: float = 1.5, k: float = 0.04, kind: str = "harris") -> torch.Tensor:
    """Structure-tensor corner measure of a ``[1, H, W]`` image: Harris ``det - k trace^2`` or Shi-Tomasi minimum eigenvalue."""
    gx, gy = V.sobel(img)
    a, b, c = V.gaussian_blur(gx * gx, sigma), V.gaussian_blur(gy * gy, sigma), V.gaussian_blur(gx * gy, sigma)
    if kind == "harris":
        return a * b - c * c - k * (a + b) ** 2
    return (a + b) / 2 - torch.sqrt(((a - b) / 2) ** 2 + c * c)


def detect_corners(img: torch.Tensor, max_points: int = 200, quality: float = 0.01, min_distance: int = 3, kind: str = "harris", border: int = 4) -> Keypoints:
    r = corner_response(img, kind=kind)[0]
    peak = (F.max_pool2d(r[None, None], 2 * min_distance + 1, 1, min_distance)[0, 0] == r) & (r > quality * r.max())
    peak[:border] = peak[-border:] = False
    peak[:, :border] = peak[:, -border:] = False
    ys, xs = peak.nonzero(as_tuple=True)
    order = r[ys, xs].argsort(descending=True)[:max_points]
    return Keypoints(torch.stack([xs[order], ys[order]], 1).float(), r[ys, xs][order], torch.ones(len(order)))


def detect_multiscale(img: torch.Tensor, levels: int = 3, scale_factor: float = 1.5, **kw) -> Keypoints:
    """Corners on an image pyramid, reported in base-image coordinates with the level's scale."""
    pts, resp, scl, cur, s = [], [], [], img, 1.0
    for _ in range(levels):
        kp = detect_corners(cur, **kw)
        pts.append(kp.xy * s); resp.append(kp.response); scl.append(torch.full((len(kp.xy),), s))
        s *= scale_factor
        cur = V.resize(img, (max(int(img.shape[-2] / s), 16), max(int(img.shape[-1] / s), 16)))
    return Keypoints(torch.cat(pts), torch.cat(resp), torch.cat(scl))


def describe(img: torch.Tensor, kp: Keypoints, patch: int = 16, cells: int = 4, bins: int = 8) -> torch.Tensor:
    """SIFT-like descriptor: a ``patch x patch`` window (scaled by the key point's scale) split into ``cells x cells`` cells
    of ``bins`` orientation histograms weighted by gradient magnitude; L2-normalised, clipped at 0.2, re-normalised."""
    gx, gy = V.sobel(V.gaussian_blur(img, 1.0))
    mag, ang = torch.sqrt(gx * gx + gy * gy)[0], (torch.atan2(gy, gx)[0] + math.pi) / (2 * math.pi)
    h, w = mag.shape
    t = (torch.arange(patch) + 0.5) / patch * 2 - 1
    base = torch.stack(torch.meshgrid(t, t, indexing="xy"), -1)                                        # [patch, patch, 2]
    half = kp.scale[:, None, None, None] * patch / 2
    centre = kp.xy[:, None, None, :]
    px = centre + base[None] * half
    grid = torch.stack([(2 * px[..., 0] + 1) / w - 1, (2 * px[..., 1] + 1) / h - 1], -1)
    n = len(kp.xy)
    samp = lambda m: F.grid_sample(m[None, None].expand(n, 1, h, w), grid, mode="bilinear", padding_mode="border", align_corners=False)[:, 0]
    m, a = samp(mag), samp(ang)
    b = (a * bins).long().clamp(0, bins - 1)
    cs = patch // cells
    one = F.one_hot(b, bins).float() * m[..., None]                                                     # [N, p, p, bins]
    desc = one.reshape(n, cells, cs, cells, cs, bins).sum((2, 4)).reshape(n, -1)
    desc = F.normalize(desc, dim=1).clamp(max=0.2)
    return F.normalize(desc, dim=1)


def match_features(d1: torch.Tensor, d2: torch.Tensor, ratio: float = 0.8, cross_check: bool = True, metric: str = "l2") -> torch.Tensor:
    """Index pairs ``[M, 2]``: nearest neighbour in ``d2`` for each row of ``d1`` that passes Lowe's ratio test (and is
    mutual when ``cross_check``)."""
    dist = torch.cdist(d1, d2) if metric == "l2" else 1 - F.normalize(d1, dim=1) @ F.normalize(d2, dim=1).t()
    if d2.shape[0] < 2:
        return torch.zeros(0, 2, dtype=torch.long)
    two = dist.topk(2, dim=1, largest=False)
    ok = two.values[:, 0] < ratio * two.values[:, 1]
    if cross_check:
        ok &= dist.argmin(0)[two.indices[:, 0]] == torch.arange(len(d1))
    i = ok.nonzero().flatten()
    return torch.stack([i, two.indices[i, 0]], 1)


def fit_homography(src: torch.Tensor, dst: torch.Tensor) -> torch.Tensor:
    """Direct linear transform with Hartley normalisation; maps ``src`` (x, y) to ``dst``."""
    def norm(p):
        c, s = p.mean(0), math.sqrt(2) / (p - p.mean(0)).norm(dim=1).mean().clamp(min=1e-12)
        t = torch.tensor([[s, 0, -s * c[0]], [0, s, -s * c[1]], [0, 0, 1.0]], dtype=torch.float64)
        return (p.double() * s - s * c.double()), t
    a, ta = norm(src)
    b, tb = norm(dst)
    x, y, u, v = a[:, 0], a[:, 1], b[:, 0], b[:, 1]
    z, o = torch.zeros_like(x), torch.ones_like(x)
    rows = torch.cat([torch.stack([-x, -y, -o, z, z, z, u * x, u * y, u], 1), torch.stack([z, z, z, -x, -y, -o, v * x, v * y, v], 1)])
    hm = torch.linalg.svd(rows).Vh[-1].reshape(3, 3)
    hm = torch.linalg.inv(tb) @ hm @ ta
    return (hm / hm[2, 2]).float()


def apply_homography(hm, pts):
    p = torch.cat([pts, torch.ones(len(pts), 1)], 1) @ hm.t()
    return p[:, :2] / p[:, 2:3]


def ransac_homography(src: torch.Tensor, dst: torch.Tensor, threshold: float = 2.0, iters: int = 500, seed: int = 0):
    """Best homography by random 4-point samples; returns ``(H refit on the inliers, inlier mask)``."""
    g = torch.Generator().manual_seed(seed)
    best = torch.zeros(len(src), dtype=torch.bool)
    for _ in range(iters):
        pick = torch.randperm(len(src), generator=g)[:4]
        try:
            hm = fit_homography(src[pick], dst[pick])
        except Exception:
            continue
        err = (apply_homography(hm, src) - dst).norm(dim=1)
        inl = err < threshold
        if inl.sum() > best.sum():
            best = inl
    return (fit_homography(src[best], dst[best]) if best.sum() >= 4 else None), best


def match_template(img: torch.Tensor, template: torch.Tensor) -> torch.Tensor:
    """Zero-mean normalised cross-correlation map ``[H - h + 1, W - w + 1]`` of single-channel tensors (values in [-1, 1])."""
    i, t = img.reshape(1, 1, *img.shape[-2:]).float(), template.reshape(1, 1, *template.shape[-2:]).float()
    n = t.shape[-1] * t.shape[-2]
    t0 = t - t.mean()
    ones = torch.ones_like(t)
    s1, s2 = F.conv2d(i, ones), F.conv2d(i * i, ones)
    num = F.conv2d(i, t0)
    den = torch.sqrt((s2 - s1 * s1 / n).clamp(min=1e-12) * (t0 * t0).sum())
    return (num / den)[0, 0]


class TemplateMatcher:
    def __init__(self, threshold: float = 0.8):
        self.threshold, self.templates = threshold, {}

    def add_template(self, name, template): self.templates[name] = template

    def match_templates(self, img) -> list[dict]:
        out = []
        for name, t in self.templates.items():
            r = match_template(img, t)
            peak = (F.max_pool2d(r[None, None], 5, 1, 2)[0, 0] == r) & (r >= self.threshold)
            for y, x in peak.nonzero().tolist():
                out.append({"template": name, "x": x, "y": y, "score": float(r[y, x])})
        return sorted(out, key=lambda m: -m["score"])


# ================================================================================================ spatial
class KDTree:
    """Static k-d tree over ``[N, D]`` points with k-nearest and radius queries (median splits, array storage)."""

    def __init__(self, points: torch.Tensor, leaf_size: int = 8):
        self.pts = points.double().cpu().numpy()
        self.leaf = leaf_size
        self.root = self._build(np.arange(len(self.pts)), 0)

    def _build(self, idx, depth):
        if len(idx) <= self.leaf:
            return ("leaf", idx)
        ax = depth % self.pts.shape[1]
        order = idx[np.argsort(self.pts[idx, ax], kind="stable")]
        mid = len(order) // 2
        return ("node", ax, self.pts[order[mid], ax], self._build(order[:mid], depth + 1), self._build(order[mid:], depth + 1))

    def find_neighbors(self, q, k: int = 1):
        q = np.asarray(q, dtype=np.float64)
        heap: list = []                                                      # max-heap of (-dist2, index)
        def visit(node):
            if node[0] == "leaf":
                for i in node[1]:
                    d = float(((self.pts[i] - q) ** 2).sum())
                    if len(heap) < k:
                        heapq.heappush(heap, (-d, int(i)))
                    elif d < -heap[0][0]:
                        heapq.heapreplace(heap, (-d, int(i)))
                return
            _, ax, split, lo, hi = node
            near, far = (lo, hi) if q[ax] < split else (hi, lo)
            visit(near)
            if len(heap) < k or (q[ax] - split) ** 2 < -heap[0][0]:
                visit(far)
        visit(self.root)
        out = sorted((-d, i) for d, i in heap)
        return [i for _, i in out], [math.sqrt(d) for d, _ in out]

    def query_region(self, q, radius: float):
        q, out = np.asarray(q, dtype=np.float64), []
        def visit(node):
            if node[0] == "leaf":
                out.extend(int(i) for i in node[1] if ((self.pts[i] - q) ** 2).sum() <= radius ** 2)
                return
            _, ax, split, lo, hi = node
            if q[ax] - radius < split:
                visit(lo)
            if q[ax] + radius >= split:
                visit(hi)
        visit(self.root)
        return sorted(out)


class SpatialObjectTracker:
    """Greedy IoU association of detections (``xyxy``) to tracks; unmatched detections open tracks, tracks unseen for
    ``max_age`` frames close.  Keeps every track's trajectory of box centres."""

    def __init__(self, iou_threshold: float = 0.3, max_age: int = 3):
        self.thr, self.max_age, self.tracks, self.next_id, self.frame = iou_threshold, max_age, {}, 0, 0
        self.finished: dict[int, list] = {}

    def track_objects(self, boxes: torch.Tensor) -> list[int]:
        from . import box_iou
        self.frame += 1
        ids = [-1] * len(boxes)
        live = list(self.tracks)
        if live and len(boxes):
            iou = box_iou(torch.stack([self.tracks[t]["box"] for t in live]), boxes)
            while True:
                v, flat = iou.flatten().max(0)
                if v < self.thr:
                    break
                ti, di = divmod(int(flat), len(boxes))
                ids[di] = live[ti]
                iou[ti, :], iou[:, di] = -1, -1
        for di, b in enumerate(boxes):
            if ids[di] < 0:
                ids[di] = self.next_id
                self.tracks[self.next_id] = {"trajectory": []}
                self.next_id += 1
            t = self.tracks[ids[di]]
            t["box"], t["seen"] = b, self.frame
            t["trajectory"].append(((b[0] + b[2]).item() / 2, (b[1] + b[3]).item() / 2))
        for tid in [t for t, v in self.tracks.items() if self.frame - v["seen"] > self.max_age]:
            self.finished[tid] = self.tracks.pop(tid)["trajectory"]
        return ids

    def get_trajectory(self, tid): return self.tracks[tid]["trajectory"] if tid in self.tracks else self.finished.get(tid)


def radial_distort_grid(h, w, k1: float, k2: float = 0.0, device=None):
    ys, xs = torch.meshgrid(torch.linspace(-1, 1, h, device=device), torch.linspace(-1, 1, w, device=device), indexing="ij")
    r2 = xs * xs + ys * ys
    f = 1 + k1 * r2 + k2 * r2 * r2
    return torch.stack([xs * f, ys * f], -1)


def correct_radial_distortion(img: torch.Tensor, k1: float, k2: float = 0.0) -> torch.Tensor:
    """Resamples an image taken through a lens with radial coefficients ``k1, k2`` (barrel: ``k1 < 0``, pincushion:
    ``k1 > 0``) at the distorted position of every undistorted pixel."""
    x4, lead = V._as4(img)
    grid = radial_distort_grid(*x4.shape[-2:], k1, k2, img.device).expand(x4.shape[0], -1, -1, -1)
    o = F.grid_sample(x4, grid, mode="bilinear", padding_mode="zeros", align_corners=True)
    return o.reshape(*lead, *o.shape[1:])


def warp_by_flow(img: torch.Tensor, flow: torch.Tensor) -> torch.Tensor:
    """Backward warp: output pixel ``p`` reads ``img[p + flow[p]]``; ``flow``: ``[2, H, W]`` (dx, dy) in pixels."""
    x4, lead = V._as4(img)
    h, w = x4.shape[-2:]
    ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float32, device=img.device), torch.arange(w, dtype=torch.float32, device=img.device), indexing="ij")
    px, py = xs + flow[0], ys + flow[1]
    grid = torch.stack([(2 * px + 1) / w - 1, (2 * py + 1) / h - 1], -1).expand(x4.shape[0], -1, -1, -1)
    o = F.grid_sample(x4, grid, mode="bilinear", padding_mode="border", align_corners=False)
    return o.reshape(*lead, *o.shape[1:])


def interpolate_frames(a: torch.Tensor, b: torch.Tensor, flow_ab: torch.Tensor, t: float = 0.5) -> torch.Tensor:
    """Intermediate frame at time ``t`` from two frames and the flow ``a -> b`` (linear motion, blended backward warps)."""
    return (1 - t) * warp_by_flow(a, -t * flow_ab) + t * warp_by_flow(b, (1 - t) * flow_ab)


def smooth_flow_field(flow: torch.Tensor, sigma: float = 1.5) -> torch.Tensor: return V.gaussian_blur(flow[None], sigma)[0]


def interpolate_to_grid(points: torch.Tensor, values: torch.Tensor, h: int, w: int, method: str = "idw", power: float = 2.0, k: int = 4) -> torch.Tensor:
    """Scattered samples at ``points`` (x, y) onto an ``h x w`` grid: ``nearest`` or inverse-distance weighting of the
    ``k`` nearest samples."""
    ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float32), torch.arange(w, dtype=torch.float32), indexing="ij")
    d = torch.cdist(torch.stack([xs.flatten(), ys.flatten()], 1), points.float())
    if method == "nearest":
        return values[d.argmin(1)].reshape(h, w)
    near = d.topk(min(k, len(points)), dim=1, largest=False)
    wgt = 1 / near.values.clamp(min=1e-6) ** power
    exact = near.values[:, 0] < 1e-6
    out = (wgt * values[near.indices]).sum(1) / wgt.sum(1)
    return torch.where(exact, values[near.indices[:, 0]], out).reshape(h, w)


def interpolate_image_gaps(img: torch.Tensor, valid: torch.Tensor, iters: int = 200) -> torch.Tensor:
    """Fills invalid pixels: a first guess by front propagation of neighbour averages, then Jacobi relaxation of the
    Laplace equation inside the holes (each hole pixel becomes the mean of its four neighbours); valid pixels unchanged."""
    x, m = img.clone() * valid, valid.float()
    k = torch.ones(3, 3)
    while m.min() == 0:
        num, den = V.conv2d_per_channel(x, k, "zeros"), V.conv2d_per_channel(m, k, "zeros")
        fill = (m == 0) & (den > 0)
        if not fill.any():
            break
        x = torch.where(fill, num / den.clamp(min=1e-12), x)
        m = torch.where(fill, torch.ones_like(m), m)
    cross = torch.tensor([[0.0, 1, 0], [1, 0, 1], [0, 1, 0]]) / 4
    for _ in range(iters):
        x = torch.where(valid, img, V.conv2d_per_channel(x, cross, "replicate"))
    return x


def compute_image_similarity(a: torch.Tensor, b: torch.Tensor, metric: str = "ssim") -> float:
    if metric == "mse":
        return float(((a - b) ** 2).mean())
    if metric == "psnr":
        return float(10 * torch.log10(1 / ((a - b) ** 2).mean().clamp(min=1e-12)))
    if metric == "ncc":
        a0, b0 = a - a.mean(), b - b.mean()
        return float((a0 * b0).sum() / (a0.norm() * b0.norm()).clamp(min=1e-12))
    mu_a, mu_b = V.gaussian_blur(a, 1.5), V.gaussian_blur(b, 1.5)
    va, vb, cab = V.gaussian_blur(a * a, 1.5) - mu_a ** 2, V.gaussian_blur(b * b, 1.5) - mu_b ** 2, V.gaussian_blur(a * b, 1.5) - mu_a * mu_b
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    return float((((2 * mu_a * mu_b + c1) * (2 * cab + c2)) / ((mu_a ** 2 + mu_b ** 2 + c1) * (va + vb + c2))).mean())


def find_similar_images(query: torch.Tensor, gallery: torch.Tensor, k: int = 3, size: int = 16):
    """Nearest gallery images by cosine similarity of down-sampled, standardised thumbnails."""
    thumb = lambda x: F.normalize(V.zscore(V.resize(x, (size, size)), per_channel=False).flatten(-3), dim=-1)
    sim = thumb(gallery) @ thumb(query)
    top = sim.topk(min(k, len(gallery)))
    return top.indices.tolist(), top.values.tolist()


def find_similar_patches(img: torch.Tensor, patch: torch.Tensor, k: int = 3):
    r = match_template(img, patch)
    top = r.flatten().topk(k)
    return [(int(i) % r.shape[1], int(i) // r.shape[1]) for i in top.indices], top.values.tolist()


# ================================================================================================ streaming
@dataclass
class Frame:
    data: torch.Tensor
    index: int
    timestamp: float


class FramePreprocessor:
    def __init__(self, resize=None, grayscale=False, normalize=None):
        self.resize, self.grayscale, self.normalize = resize, grayscale, normalize

    def preprocess(self, x):
        if self.resize:
            x = V.resize(x, self.resize)
        if self.grayscale and x.shape[-3] == 3:
            x = V.rgb_to_grayscale(x)
        if self.normalize:
            x = V.normalize(x, *self.normalize)
        return x


class StreamProcessor:
    """Bounded frame queue (``drop_oldest`` or ``drop_newest`` when full), per-frame processing with latency records, batches
    of ``batch_size``, and a resolution ladder that steps down when the mean latency exceeds the frame budget and back up
    when there is headroom."""

    def __init__(self, fn, target_fps: float = 30.0, buffer_size: int = 8, batch_size: int = 1, drop_policy: str = "drop_oldest",
                 preprocessor: FramePreprocessor | None = None, resolutions=((64, 64), (48, 48), (32, 32)), clock=time.perf_counter):
        self.fn, self.budget, self.cap, self.batch, self.policy = fn, 1.0 / target_fps, buffer_size, batch_size, drop_policy
        self.pre, self.resolutions, self.level, self.clock = preprocessor or FramePreprocessor(), list(resolutions), 0, clock
        self.queue: deque[Frame] = deque()
        self.times: deque[float] = deque(maxlen=30)
        self.received = self.dropped = self.processed = 0

    def push_frame(self, data) -> bool:
        self.received += 1
        if len(self.queue) >= self.cap:
            self.dropped += 1
            if self.policy == "drop_newest":
                return False
            self.queue.popleft()
        self.queue.append(Frame(data, self.received - 1, self.clock()))
        return True

    def is_full(self): return len(self.queue) >= self.cap
    def is_empty(self): return not self.queue
    def __len__(self): return len(self.queue)

    def process_available(self) -> list:
        out = []
        while len(self.queue) >= self.batch:
            frames = [self.queue.popleft() for _ in range(self.batch)]
            t0 = self.clock()
            self.pre.resize = self.resolutions[self.level]
            batch = torch.stack([self.pre.preprocess(f.data) for f in frames])
            res = self.fn(batch)
            dt = (self.clock() - t0) / self.batch
            self.times.append(dt)
            self.processed += self.batch
            out.append({"indices": [f.index for f in frames], "result": res, "latency": dt, "resolution": self.resolutions[self.level]})
            self._adapt()
        return out

    def flush(self):
        b, self.batch = self.batch, 1
        out = self.process_available()
        self.batch = b
        return out

    def _adapt(self):
        if len(self.times) < 3:
            return
        mean = sum(self.times) / len(self.times)
        if mean > self.budget and self.level < len(self.resolutions) - 1:
            self.level += 1
            self.times.clear()
        elif mean < 0.5 * self.budget and self.level > 0:
            self.level -= 1
            self.times.clear()

    def is_realtime(self): return bool(self.times) and sum(self.times) / len(self.times) <= self.budget

    def stats(self):
        t = list(self.times)
        return {"received": self.received, "dropped": self.dropped, "processed": self.processed, "queue": len(self.queue),
                "mean_latency": sum(t) / len(t) if t else 0.0, "fps": len(t) / sum(t) if t and sum(t) > 0 else 0.0, "resolution": self.resolutions[self.level]}


# ================================================================================================ 3-D
class PointCloud:
    def __init__(self, points: torch.Tensor, colors: torch.Tensor | None = None, normals: torch.Tensor | None = None):
        self.points, self.colors, self.normals = points.float(), colors, normals

    def __len__(self): return len(self.points)
    def bounds(self): return self.points.amin(0), self.points.amax(0)
    def centroid(self): return self.points.mean(0)

    def voxel_downsample(self, voxel: float) -> "PointCloud":
        """One point per occupied voxel: the mean of the points (and colours) inside."""
        key = torch.floor(self.points / voxel).long()
        _, inv, cnt = torch.unique(key, dim=0, return_inverse=True, return_counts=True)
        mean = lambda t: torch.zeros(len(cnt), t.shape[1]).index_add_(0, inv, t.float()) / cnt[:, None]
        return PointCloud(mean(self.points), mean(self.colors) if self.colors is not None else None)

    def filter_by_distance(self, centre, radius: float) -> "PointCloud":
        keep = (self.points - torch.as_tensor(centre, dtype=torch.float32)).norm(dim=1) <= radius
        return PointCloud(self.points[keep], self.colors[keep] if self.colors is not None else None, self.normals[keep] if self.normals is not None else None)

    def remove_statistical_outliers(self, k: int = 8, std_ratio: float = 2.0) -> "PointCloud":
        d = torch.cdist(self.points, self.points).topk(k + 1, largest=False).values[:, 1:].mean(1)
        keep = d <= d.mean() + std_ratio * d.std()
        return PointCloud(self.points[keep], self.colors[keep] if self.colors is not None else None)

    def estimate_normals(self, k: int = 8) -> torch.Tensor:
        """Smallest-eigenvalue direction of each point's neighbourhood covariance, oriented away from the centroid."""
        idx = torch.cdist(self.points, self.points).topk(k + 1, largest=False).indices
        nb = self.points[idx]
        c = nb - nb.mean(1, keepdim=True)
        _, vec = torch.linalg.eigh(c.transpose(1, 2) @ c)
        n = vec[:, :, 0]
        sign = torch.sign((n * (self.points - self.centroid())).sum(1, keepdim=True))
        n = n * torch.where(sign == 0, torch.ones_like(sign), sign)
        self.normals = n
        return n

    def transform(self, matrix: torch.Tensor) -> "PointCloud":
        p = torch.cat([self.points, torch.ones(len(self), 1)], 1) @ matrix.float().t()
        return PointCloud(p[:, :3] / p[:, 3:4], self.colors)

    def to_tensor(self):
        parts = [self.points] + ([self.colors.float()] if self.colors is not None else []) + ([self.normals] if self.normals is not None else [])
        return torch.cat(parts, 1)


@dataclass
class BoundingBox3D:
    lo: torch.Tensor
    hi: torch.Tensor

    @classmethod
    def from_points(cls, p): return cls(p.amin(0), p.amax(0))
    def volume(self): return float((self.hi - self.lo).clamp(min=0).prod())
    def contains_point(self, p): p = torch.as_tensor(p, dtype=torch.float32); return bool(((p >= self.lo) & (p <= self.hi)).all())
    def corners(self): return torch.tensor([[(self.lo, self.hi)[(i >> a) & 1][a] for a in range(3)] for i in range(8)])
    def center(self): return (self.lo + self.hi) / 2

    def iou(self, o: "BoundingBox3D") -> float:
        inter = float((torch.minimum(self.hi, o.hi) - torch.maximum(self.lo, o.lo)).clamp(min=0).prod())
        return inter / max(self.volume() + o.volume() - inter, 1e-12)


class Mesh3D:
    def __init__(self, vertices: torch.Tensor, faces: torch.Tensor):
        self.vertices, self.faces = vertices.float(), faces.long()

    @classmethod
    def create_cube(cls, size: float = 1.0):
        s = size / 2
        v = torch.tensor([[x, y, z] for x in (-s, s) for y in (-s, s) for z in (-s, s)])
        f = torch.tensor([[0, 1, 3], [0, 3, 2], [4, 6, 7], [4, 7, 5], [0, 4, 5], [0, 5, 1], [2, 3, 7], [2, 7, 6], [0, 2, 6], [0, 6, 4], [1, 5, 7], [1, 7, 3]])
        return cls(v, f)

    @classmethod
    def create_sphere(cls, radius: float = 1.0, rings: int = 16, segments: int = 32):
        v = [[0.0, 0.0, radius]]
        for i in range(1, rings):
            th = math.pi * i / rings
            v += [[radius * math.sin(th) * math.cos(2 * math.pi * j / segments), radius * math.sin(th) * math.sin(2 * math.pi * j / segments), radius * math.cos(th)] for j in range(segments)]
        v.append([0.0, 0.0, -radius])
        f, last = [], len(v) - 1
        ring = lambda i, j: 1 + (i - 1) * segments + j % segments
        for j in range(segments):
            f.append([0, ring(1, j), ring(1, j + 1)])
            f.append([last, ring(rings - 1, j + 1), ring(rings - 1, j)])
        for i in range(1, rings - 1):
            for j in range(segments):
                f += [[ring(i, j), ring(i + 1, j), ring(i + 1, j + 1)], [ring(i, j), ring(i + 1, j + 1), ring(i, j + 1)]]
        return cls(torch.tensor(v), torch.tensor(f))

    def _tri(self): return self.vertices[self.faces[:, 0]], self.vertices[self.faces[:, 1]], self.vertices[self.faces[:, 2]]
    def compute_face_normals(self): a, b, c = self._tri(); return F.normalize(torch.linalg.cross(b - a, c - a), dim=1)
    def surface_area(self): a, b, c = self._tri(); return float(torch.linalg.cross(b - a, c - a).norm(dim=1).sum() / 2)
    def volume(self): a, b, c = self._tri(); return abs(float((a * torch.linalg.cross(b, c)).sum() / 6))

    def compute_vertex_normals(self):
        a, b, c = self._tri()
        fn = torch.linalg.cross(b - a, c - a)                                  # area-weighted
        vn = torch.zeros_like(self.vertices)
        for k in range(3):
            vn.index_add_(0, self.faces[:, k], fn)
        return F.normalize(vn, dim=1)

    def sample_points(self, n: int, seed: int = 0) -> PointCloud:
        g = torch.Generator().manual_seed(seed)
        a, b, c = self._tri()
        area = torch.linalg.cross(b - a, c - a).norm(dim=1)
        f = torch.multinomial(area / area.sum(), n, replacement=True, generator=g)
        u, v = torch.rand(n, 1, generator=g), torch.rand(n, 1, generator=g)
        flip = u + v > 1
        u, v = torch.where(flip, 1 - u, u), torch.where(flip, 1 - v, v)
        return PointCloud(a[f] + u * (b[f] - a[f]) + v * (c[f] - a[f]))


class Scene3D:
    def __init__(self): self.objects: list = []
    def add_point_cloud(self, pc, name=""): self.objects.append(("point_cloud", name, pc))
    def add_mesh(self, m, name=""): self.objects.append(("mesh", name, m))
    def add_bounding_box(self, b, name=""): self.objects.append(("box", name, b))
    def clear(self): self.objects.clear()
    def num_objects(self): return len(self.objects)

    def export_summary(self) -> dict:
        pts = [o.points for k, _, o in self.objects if k == "point_cloud"] + [o.vertices for k, _, o in self.objects if k == "mesh"] + [o.corners() for k, _, o in self.objects if k == "box"]
        allp = torch.cat(pts) if pts else torch.zeros(0, 3)
        return {"objects": [{"kind": k, "name": n} for k, n, _ in self.objects], "points": int(sum(len(o.points) for k, _, o in self.objects if k == "point_cloud")),
                "faces": int(sum(len(o.faces) for k, _, o in self.objects if k == "mesh")),
                "bounds": [allp.amin(0).tolist(), allp.amax(0).tolist()] if len(allp) else None}

    def export_ply(self, path):
        """ASCII PLY of every point cloud and mesh in the scene (vertices of all objects, faces re-indexed)."""
        verts, faces, off = [], [], 0
        for k, _, o in self.objects:
            if k == "point_cloud":
                verts.append(o.points); off += len(o.points)
            elif k == "mesh":
                verts.append(o.vertices); faces.append(o.faces + off); off += len(o.vertices)
        v = torch.cat(verts) if verts else torch.zeros(0, 3)
        f = torch.cat(faces) if faces else torch.zeros(0, 3, dtype=torch.long)
        with open(path, "w") as fh:
            fh.write(f"ply\nformat ascii 1.0\nelement vertex {len(v)}\nproperty float x\nproperty float y\nproperty float z\nelement face {len(f)}\nproperty list uchar int vertex_indices\nend_header\n")
            fh.writelines(f"{p[0]:.6g} {p[1]:.6g} {p[2]:.6g}\n" for p in v.tolist())
            fh.writelines(f"3 {t[0]} {t[1]} {t[2]}\n" for t in f.tolist())
