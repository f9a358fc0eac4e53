"""Image operators on ``[..., C, H, W]`` float tensors of any device (``crates/torsh-vision/src/ops/{color,filtering,
geometric,detection,analysis}/mod.rs``): colour spaces and adjustments, histograms and equalisation, linear and rank
filters, edges (Sobel / Prewitt / Laplacian / Canny), grey-scale morphology, resampling / rotation / affine warps,
box utilities with RoI pooling and alignment, and task losses / metrics for classification, detection and segmentation.
Everything is batched tensor arithmetic (convolutions, unfold, grid_sample), so the same code runs on the GPU."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ================================================================================================ colour
def rgb_to_grayscale(x): return (0.299 * x[..., 0:1, :, :] + 0.587 * x[..., 1:2, :, :] + 0.114 * x[..., 2:3, :, :])


def rgb_to_hsv(x):
    r, g, b = x.unbind(-3)
    mx, mn = x.amax(-3), x.amin(-3)
    d = mx - mn
    safe = torch.where(d == 0, torch.ones_like(d), d)
    h = torch.where(mx == r, ((g - b) / safe) % 6, torch.where(mx == g, (b - r) / safe + 2, (r - g) / safe + 4))
    h = torch.where(d == 0, torch.zeros_like(h), h) / 6
    s = torch.where(mx == 0, torch.zeros_like(mx), d / torch.where(mx == 0, torch.ones_like(mx), mx))
    return torch.stack([h, s, mx], -3)


def hsv_to_rgb(x):
    h, s, v = x.unbind(-3)
    i = torch.floor(h * 6)
    f = h * 6 - i
    p, q, t = v * (1 - s), v * (1 - f * s), v * (1 - (1 - f) * s)
    i = i.long() % 6
    pick = lambda a0, a1, a2, a3, a4, a5: torch.where(i == 0, a0, torch.where(i == 1, a1, torch.where(i == 2, a2, torch.where(i == 3, a3, torch.where(i == 4, a4, a5)))))
    return torch.stack([pick(v, q, p, p, t, v), pick(t, v, v, q, p, p), pick(p, p, t, v, v, q)], -3)


def rgb_to_yuv(x):
    m = x.new_tensor([[0.299, 0.587, 0.114], [-0.14713, -0.28886, 0.436], [0.615, -0.51499, -0.10001]])
    return torch.einsum("ij,...jhw->...ihw", m, x)


def yuv_to_rgb(x):
    m = torch.linalg.inv(x.new_tensor([[0.299, 0.587, 0.114], [-0.14713, -0.28886, 0.436], [0.615, -0.51499, -0.10001]]))
    return torch.einsum("ij,...jhw->...ihw", m, x)


def rgb_to_lab(x):
    """sRGB in [0, 1] to CIE L*a*b* (D65)."""
    lin = torch.where(x > 0.04045, ((x + 0.055) / 1.055) ** 2.4, x / 12.92)
    m = x.new_tensor([[0.4124564, 0.3575761, 0.1804375], [0.2126729, 0.7151522, 0.0721750], [0.0193339, 0.1191920, 0.9503041]])
    xyz = torch.einsum("ij,...jhw->...ihw", m, lin) / x.new_tensor([0.95047, 1.0, 1.08883]).reshape(3, 1, 1)
    f = torch.where(xyz > 216 / 24389, xyz.clamp(min=1e-12) ** (1 / 3), (24389 / 27 * xyz + 16) / 116)
    fx, fy, fz = f.unbind(-3)
    return torch.stack([116 * fy - 16, 500 * (fx - fy), 200 * (fy - fz)], -3)


def adjust_brightness(x, factor): return (x * factor).clamp(0, 1)
def adjust_contrast(x, factor): m = rgb_to_grayscale(x).mean((-3, -2, -1), keepdim=True) if x.shape[-3] == 3 else x.mean((-3, -2, -1), keepdim=True); return ((x - m) * factor + m).clamp(0, 1)
def adjust_saturation(x, factor): g = rgb_to_grayscale(x); return ((x - g) * factor + g).clamp(0, 1)
def gamma_correction(x, gamma, gain=1.0): return (gain * x.clamp(min=0) ** gamma).clamp(0, 1)


def adjust_hue(x, delta):
    hsv = rgb_to_hsv(x)
    return hsv_to_rgb(torch.stack([(hsv[..., 0, :, :] + delta) % 1.0, hsv[..., 1, :, :], hsv[..., 2, :, :]], -3))


def normalize(x, mean, std): return (x - x.new_tensor(mean).reshape(-1, 1, 1)) / x.new_tensor(std).reshape(-1, 1, 1)
def normalize_imagenet(x): return normalize(x, (0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
def zscore(x, per_channel=True): d = (-2, -1) if per_channel else (-3, -2, -1); return (x - x.mean(d, keepdim=True)) / x.std(d, keepdim=True).clamp(min=1e-12)
def extract_channel(x, c): return x[..., c:c + 1, :, :]


def compute_histogram(x, bins=256, lo=0.0, hi=1.0):
    """Per-channel histogram ``[..., C, bins]``."""
    idx = ((x - lo) / (hi - lo) * bins).long().clamp(0, bins - 1).flatten(-2)
    return torch.zeros(*idx.shape[:-1], bins, device=x.device).scatter_add_(-1, idx, torch.ones_like(idx, dtype=torch.float32))


def histogram_equalization(x, bins=256):
    """Maps every channel through its own cumulative distribution."""
    hist = compute_histogram(x, bins)
    cdf = hist.cumsum(-1)
    lo = cdf.gather(-1, (hist > 0).float().argmax(-1, keepdim=True))
    lut = ((cdf - lo) / (cdf[..., -1:] - lo).clamp(min=1)).clamp(0, 1)
    idx = (x * bins).long().clamp(0, bins - 1)
    return lut.gather(-1, idx.flatten(-2)).reshape(x.shape)


def clahe(x, tiles=(4, 4), clip_limit=2.0, bins=64):
    """Contrast-limited adaptive equalisation: clipped per-tile look-up tables, bilinearly blended between tile centres."""
    *lead, c, h, w = x.shape
    th, tw = h // tiles[0], w // tiles[1]
    t = x[..., :th * tiles[0], :tw * tiles[1]].reshape(*lead, c, tiles[0], th, tiles[1], tw).transpose(-3, -2)      # [..., C, ty, tx, th, tw]
    idx = (t * bins).long().clamp(0, bins - 1).flatten(-2)
    hist = torch.zeros(*idx.shape[:-1], bins, device=x.device).scatter_add_(-1, idx, torch.ones_like(idx, dtype=torch.float32))
    limit = clip_limit * th * tw / bins
    excess = (hist - limit).clamp(min=0).sum(-1, keepdim=True)
    hist = hist.clamp(max=limit) + excess / bins
    lut = hist.cumsum(-1) / (th * tw)                                                                                # [..., C, ty, tx, bins]
    pix = (x * bins).long().clamp(0, bins - 1)
    # value of every tile's LUT at every pixel, then bilinear weights between the four nearest tile centres
    gy = ((torch.arange(h, device=x.device) + 0.5) / th - 0.5).clamp(0, tiles[0] - 1)
    gx = ((torch.arange(w, device=x.device) + 0.5) / tw - 0.5).clamp(0, tiles[1] - 1)
    y0, x0 = gy.floor().long(), gx.floor().long()
    y1, x1 = (y0 + 1).clamp(max=tiles[0] - 1), (x0 + 1).clamp(max=tiles[1] - 1)
    wy, wx = (gy - y0).reshape(-1, 1), (gx - x0).reshape(1, -1)
    def look(yi, xi):
        table = lut[..., yi, :, :][..., :, xi, :]                                                                  # [..., C, H, W, bins]
        return table.gather(-1, pix.unsqueeze(-1)).squeeze(-1)
    return ((1 - wy) * (1 - wx) * look(y0, x0) + (1 - wy) * wx * look(y0, x1) + wy * (1 - wx) * look(y1, x0) + wy * wx * look(y1, x1)).clamp(0, 1)


# ================================================================================================ filtering
def _as4(x):
    lead = x.shape[:-3]
    return x.reshape(-1, *x.shape[-3:]), lead


def conv2d_per_channel(x, kernel, padding="reflect"):
    """Same-size correlation of every channel with one 2-D kernel."""
    x4, lead = _as4(x)
    kh, kw = kernel.shape
    c = x4.shape[1]
    xp = F.pad(x4, (kw // 2, (kw - 1) // 2, kh // 2, (kh - 1) // 2), mode=padding) if padding != "zeros" else F.pad(x4, (kw // 2, (kw - 1) // 2, kh // 2, (kh - 1) // 2))
    out = F.conv2d(xp, kernel.to(x).expand(c, 1, kh, kw), groups=c)
    return out.reshape(*lead, *out.shape[1:])


def gaussian_kernel1d(sigma, size=None):
    size = size or 2 * int(math.ceil(3 * sigma)) + 1
    t = torch.arange(size, dtype=torch.float32) - (size - 1) / 2
    k = torch.exp(-t * t / (2 * sigma * sigma))
    return k / k.sum()


def gaussian_blur(x, sigma, size=None, padding="reflect"):
    k = gaussian_kernel1d(sigma, size)
    return conv2d_per_channel(conv2d_per_channel(x, k[None, :], padding), k[:, None], padding)


def box_blur(x, size=3): return conv2d_per_channel(x, torch.full((size, size), 1.0 / size ** 2))


_SOBEL_X = torch.tensor([[-1.0, 0, 1], [-2, 0, 2], [-1, 0, 1]])
_PREWITT_X = torch.tensor([[-1.0, 0, 1], [-1, 0, 1], [-1, 0, 1]])
_LAPLACE = torch.tensor([[0.0, 1, 0], [1, -4, 1], [0, 1, 0]])


def sobel(x): return conv2d_per_channel(x, _SOBEL_X), conv2d_per_channel(x, _SOBEL_X.t())
def prewitt(x): return conv2d_per_channel(x, _PREWITT_X), conv2d_per_channel(x, _PREWITT_X.t())
def laplacian(x): return conv2d_per_channel(x, _LAPLACE)
def sobel_edge_detection(x): gx, gy = sobel(x); return torch.sqrt(gx * gx + gy * gy)
def unsharp_mask(x, sigma=1.0, amount=1.0): return (x + amount * (x - gaussian_blur(x, sigma))).clamp(0, 1)


def _patches(x, size, mode="reflect"):
    x4, lead = _as4(x)
    xp = F.pad(x4, (size // 2,) * 4, mode=mode)
    p = xp.unfold(2, size, 1).unfold(3, size, 1)                              # [N, C, H, W, k, k]
    return p.reshape(*lead, *p.shape[1:4], size * size)


def median_filter(x, size=3): return _patches(x, size).median(-1).values
def erosion(x, size=3, iterations=1):
    for _ in range(iterations):
        x = _patches(x, size, "replicate").amin(-1)
    return x


def dilation(x, size=3, iterations=1):
    for _ in range(iterations):
        x = _patches(x, size, "replicate").amax(-1)
    return x


def opening(x, size=3): return dilation(erosion(x, size), size)
def closing(x, size=3): return erosion(dilation(x, size), size)
def morphological_gradient(x, size=3): return dilation(x, size) - erosion(x, size)
def top_hat(x, size=3): return x - opening(x, size)


def bilateral_filter(x, size=5, sigma_space=2.0, sigma_color=0.1):
    p = _patches(x, size)
    t = torch.arange(size, dtype=torch.float32, device=x.device) - size // 2
    ws = torch.exp(-(t[:, None] ** 2 + t[None, :] ** 2) / (2 * sigma_space ** 2)).reshape(-1)
    wc = torch.exp(-(p - x.unsqueeze(-1)) ** 2 / (2 * sigma_color ** 2))
    w = ws * wc
    return (w * p).sum(-1) / w.sum(-1)


def canny(x, low=0.1, high=0.2, sigma=1.0):
    """Binary edge map of a single-channel image: smoothing, Sobel, non-maximum suppression along the quantised gradient
    direction, double threshold, and hysteresis by repeated dilation of the strong set inside the weak set."""
    g = gaussian_blur(x, sigma)
    gx, gy = sobel(g)
    mag = torch.sqrt(gx * gx + gy * gy)
    ang = (torch.atan2(gy, gx) * 180 / math.pi) % 180
    sector = (((ang + 22.5) // 45).long() % 4)
    m4, lead = _as4(mag)
    mp = F.pad(m4, (1, 1, 1, 1))
    h, w = m4.shape[-2:]
    sh = lambda dy, dx: mp[..., 1 + dy:1 + dy + h, 1 + dx:1 + dx + w].reshape(mag.shape)
    n1 = torch.where(sector == 0, sh(0, 1), torch.where(sector == 1, sh(1, 1), torch.where(sector == 2, sh(1, 0), sh(1, -1))))
    n2 = torch.where(sector == 0, sh(0, -1), torch.where(sector == 1, sh(-1, -1), torch.where(sector == 2, sh(-1, 0), sh(-1, 1))))
    thin = torch.where((mag >= n1) & (mag >= n2), mag, torch.zeros_like(mag))
    strong, weak = thin >= high, thin >= low
    cur = strong
    while True:
        nxt = (dilation(cur.float(), 3) > 0) & weak
        if torch.equal(nxt, cur):
            return cur
        cur = nxt


# ================================================================================================ geometry
def horizontal_flip(x): return x.flip(-1)
def vertical_flip(x): return x.flip(-2)
def center_crop(x, size): h, w = x.shape[-2:]; t, l = (h - size[0]) // 2, (w - size[1]) // 2; return x[..., t:t + size[0], l:l + size[1]]
def crop_region(x, top, left, height, width): return x[..., top:top + height, left:left + width]
def pad(x, padding, mode="constant", value=0.0): x4, lead = _as4(x); o = F.pad(x4, padding, mode=mode, value=value) if mode == "constant" else F.pad(x4, padding, mode=mode); return o.reshape(*lead, *o.shape[1:])


def resize(x, size, mode="bilinear", antialias=True):
    x4, lead = _as4(x)
    kw = {} if mode in ("nearest", "area") else {"align_corners": False, "antialias": antialias and mode in ("bilinear", "bicubic")}
    o = F.interpolate(x4, size=size, mode=mode, **kw)
    return o.reshape(*lead, *o.shape[1:])


def affine_grid_matrix(angle=0.0, translate=(0.0, 0.0), scale=1.0, shear=(0.0, 0.0)):
    """2 x 3 matrix in normalised coordinates mapping output to input positions (rotation about the centre, degrees)."""
    a, sx, sy = -math.radians(angle), math.radians(shear[0]), math.radians(shear[1])           # y points down: counter-clockwise on screen
    rot = torch.tensor([[math.cos(a), -math.sin(a)], [math.sin(a), math.cos(a)]])
    sh = torch.tensor([[1.0, math.tan(sx)], [math.tan(sy), 1.0]])
    m = (rot @ sh) * scale
    inv = torch.linalg.inv(m)
    t = -inv @ torch.tensor(translate, dtype=torch.float32)
    return torch.cat([inv, t[:, None]], 1)


def warp_affine(x, theta, mode="bilinear", padding_mode="zeros"):
    x4, lead = _as4(x)
    theta = theta.to(x4).expand(x4.shape[0], 2, 3)
    grid = F.affine_grid(theta, list(x4.shape), align_corners=False)
    o = F.grid_sample(x4, grid, mode=mode, padding_mode=padding_mode, align_corners=False)
    return o.reshape(*lead, *o.shape[1:])


def rotate(x, angle, mode="bilinear"):
    h, w = x.shape[-2:]
    th = affine_grid_matrix(angle)
    th = th * torch.tensor([[1.0, h / w, 1.0], [w / h, 1.0, 1.0]])            # keep the rotation rigid for non-square images
    return warp_affine(x, th, mode)


def translate(x, dx, dy):
    h, w = x.shape[-2:]
    return warp_affine(x, affine_grid_matrix(translate=(2 * dx / w, 2 * dy / h)))


def warp_perspective(x, hmat, mode="bilinear"):
    """``hmat``: 3 x 3 homography mapping output pixel coordinates to input pixel coordinates."""
    x4, lead = _as4(x)
    h, w = x4.shape[-2:]
    ys, xs = torch.meshgrid(torch.arange(h, dtype=torch.float32, device=x.device), torch.arange(w, dtype=torch.float32, device=x.device), indexing="ij")
    pts = torch.stack([xs, ys, torch.ones_like(xs)], -1) @ hmat.to(x4).t()
    px, py = pts[..., 0] / pts[..., 2], pts[..., 1] / pts[..., 2]
    grid = torch.stack([(2 * px + 1) / w - 1, (2 * py + 1) / h - 1], -1).expand(x4.shape[0], h, w, 2)
    o = F.grid_sample(x4, grid, mode=mode, padding_mode="zeros", align_corners=False)
    return o.reshape(*lead, *o.shape[1:])


# ================================================================================================ boxes / RoI
def convert_bbox_format(b, src: str, dst: str):
    """Formats: ``xyxy``, ``xywh`` (top-left + size), ``cxcywh``."""
    if src == dst:
        return b
    if src == "xywh":
        b = torch.cat([b[..., :2], b[..., :2] + b[..., 2:]], -1)
    elif src == "cxcywh":
        b = torch.cat([b[..., :2] - b[..., 2:] / 2, b[..., :2] + b[..., 2:] / 2], -1)
    if dst == "xywh":
        return torch.cat([b[..., :2], b[..., 2:] - b[..., :2]], -1)
    if dst == "cxcywh":
        return torch.cat([(b[..., :2] + b[..., 2:]) / 2, b[..., 2:] - b[..., :2]], -1)
    return b


def clip_bbox(b, h, w): return torch.stack([b[..., 0].clamp(0, w), b[..., 1].clamp(0, h), b[..., 2].clamp(0, w), b[..., 3].clamp(0, h)], -1)
def scale_bbox(b, sx, sy): return b * b.new_tensor([sx, sy, sx, sy])
def filter_boxes_by_size(b, min_size): wh = b[..., 2:] - b[..., :2]; return ((wh[..., 0] >= min_size) & (wh[..., 1] >= min_size)).nonzero().flatten()


def generalized_iou(a, b):
    """IoU minus the share of the smallest enclosing box that neither box covers; ``[len(a), len(b)]``."""
    area = lambda t: (t[:, 2] - t[:, 0]) * (t[:, 3] - t[:, 1])
    inter = (torch.minimum(a[:, None, 2:], b[None, :, 2:]) - torch.maximum(a[:, None, :2], b[None, :, :2])).clamp(min=0).prod(-1)
    union = area(a)[:, None] + area(b)[None] - inter
    hull = (torch.maximum(a[:, None, 2:], b[None, :, 2:]) - torch.minimum(a[:, None, :2], b[None, :, :2])).clamp(min=0).prod(-1)
    return inter / union.clamp(min=1e-12) - (hull - union) / hull.clamp(min=1e-12)


def roi_align(feat, rois, output_size, spatial_scale=1.0, sampling_ratio=2):
    """``feat``: ``[N, C, H, W]``; ``rois``: ``[K, 5]`` rows ``(batch, x1, y1, x2, y2)``; bilinear samples averaged per bin
    (the half-pixel aligned form)."""
    oh, ow = output_size
    k = rois.shape[0]
    b = rois[:, 0].long()
    x1, y1, x2, y2 = (rois[:, i] * spatial_scale - 0.5 for i in range(1, 5))
    bw, bh = (x2 - x1) / ow, (y2 - y1) / oh
    s = sampling_ratio
    iy = (torch.arange(oh * s, device=feat.device) + 0.5) / s
    ix = (torch.arange(ow * s, device=feat.device) + 0.5) / s
    ys = y1[:, None] + iy[None] * bh[:, None]                                  # [K, oh*s]
    xs = x1[:, None] + ix[None] * bw[:, None]
    h, w = feat.shape[-2:]
    grid = torch.stack([(2 * xs[:, None, :].expand(k, oh * s, ow * s) + 1) / w - 1, (2 * ys[:, :, None].expand(k, oh * s, ow * s) + 1) / h - 1], -1)
    samp = F.grid_sample(feat[b], grid, mode="bilinear", padding_mode="border", align_corners=False)
    inside = ((ys >= -1) & (ys <= h))[:, :, None] & ((xs >= -1) & (xs <= w))[:, None, :]   # samples up to one pixel outside clamp to the edge
    return F.avg_pool2d(samp * inside[:, None].to(samp), s)


def roi_pool(feat, rois, output_size, spatial_scale=1.0):
    """Max over each quantised bin (the original RoI pooling)."""
    oh, ow = output_size
    out = feat.new_zeros(rois.shape[0], feat.shape[1], oh, ow)
    h, w = feat.shape[-2:]
    for i, r in enumerate(rois.tolist()):
        b = int(r[0])
        x1, y1, x2, y2 = (int(round(v * spatial_scale)) for v in r[1:])
        rh, rw = max(y2 - y1 + 1, 1), max(x2 - x1 + 1, 1)
        for py in range(oh):
            ys, ye = min(max(y1 + int(math.floor(py * rh / oh)), 0), h), min(max(y1 + int(math.ceil((py + 1) * rh / oh)), 0), h)
            for px in range(ow):
                xs, xe = min(max(x1 + int(math.floor(px * rw / ow)), 0), w), min(max(x1 + int(math.ceil((px + 1) * rw / ow)), 0), w)
                if ye > ys and xe > xs:
                    out[i, :, py, px] = feat[b, :, ys:ye, xs:xe].amax((-2, -1))
    return out


# ================================================================================================ losses / metrics
def dice_loss(logits, target, eps=1.0):
    """``logits``: ``[N, C, H, W]``; ``target``: ``[N, H, W]`` class ids; soft Dice averaged over classes."""
    p = logits.softmax(1)
    t = F.one_hot(target, logits.shape[1]).permute(0, 3, 1, 2).to(p)
    inter, den = (p * t).sum((0, 2, 3)), (p + t).sum((0, 2, 3))
    return 1 - ((2 * inter + eps) / (den + eps)).mean()


def focal_loss(logits, target, gamma=2.0, alpha: float | None = None, ignore_index: int | None = None):
    ce = F.cross_entropy(logits, target, reduction="none", ignore_index=ignore_index if ignore_index is not None else -100)
    pt = torch.exp(-ce)
    loss = (1 - pt) ** gamma * ce
    if alpha is not None:
        loss = loss * torch.where(target > 0, torch.full_like(ce, alpha), torch.full_like(ce, 1 - alpha))
    keep = target != ignore_index if ignore_index is not None else torch.ones_like(target, dtype=torch.bool)
    return loss[keep].mean()


def iou_loss(pred_boxes, target_boxes, kind="iou"):
    from . import box_iou
    if kind == "giou":
        return (1 - generalized_iou(pred_boxes, target_boxes).diagonal()).mean()
    return (1 - box_iou(pred_boxes, target_boxes).diagonal()).mean()


def compute_segmentation_metrics(pred, target, num_classes, ignore_index: int | None = None) -> dict:
    keep = target != ignore_index if ignore_index is not None else torch.ones_like(target, dtype=torch.bool)
    cm = torch.bincount(target[keep] * num_classes + pred[keep], minlength=num_classes ** 2).reshape(num_classes, num_classes).double()
    tp = cm.diagonal()
    iou = tp / (cm.sum(0) + cm.sum(1) - tp).clamp(min=1)
    dice = 2 * tp / (cm.sum(0) + cm.sum(1)).clamp(min=1)
    present = cm.sum(1) > 0
    freq = cm.sum(1) / cm.sum()
    return {"pixel_accuracy": float(tp.sum() / cm.sum()), "mean_iou": float(iou[present].mean()), "mean_dice": float(dice[present].mean()),
            "frequency_weighted_iou": float((freq * iou).sum()), "per_class_iou": iou.tolist(), "confusion": cm}


def compute_detection_metrics(pred_boxes, pred_scores, pred_labels, gt_boxes, gt_labels, iou_threshold=0.5) -> dict:
    """Single-image precision / recall / AP (all-point interpolation) per class and their mean."""
    from . import box_iou
    aps, tp_total, fp_total = {}, 0, 0
    for c in gt_labels.unique().tolist():
        pm, gm = pred_labels == c, gt_labels == c
        pb, ps, gb = pred_boxes[pm], pred_scores[pm], gt_boxes[gm]
        order = ps.argsort(descending=True)
        used, tp = torch.zeros(len(gb), dtype=torch.bool), []
        iou = box_iou(pb[order], gb) if len(pb) and len(gb) else torch.zeros(len(pb), len(gb))
        for i in range(len(order)):
            j = int(iou[i].argmax()) if len(gb) else -1
            hit = j >= 0 and iou[i, j] >= iou_threshold and not used[j]
            if hit:
                used[j] = True
            tp.append(float(hit))
        tp = torch.tensor(tp)
        ctp, cfp = tp.cumsum(0), (1 - tp).cumsum(0)
        rec, prec = ctp / max(len(gb), 1), ctp / (ctp + cfp).clamp(min=1)
        mrec, mpre = torch.cat([torch.zeros(1), rec, torch.ones(1)]), torch.cat([torch.zeros(1), prec, torch.zeros(1)])
        mpre = mpre.flip(0).cummax(0).values.flip(0)
        aps[c] = float(((mrec[1:] - mrec[:-1]) * mpre[1:]).sum())
        tp_total, fp_total = tp_total + int(tp.sum()), fp_total + int((1 - tp).sum())
    return {"ap_per_class": aps, "map": sum(aps.values()) / max(len(aps), 1), "precision": tp_total / max(tp_total + fp_total, 1),
            "recall": tp_total / max(len(gt_boxes), 1)}


def compute_classification_metrics(logits, target, topk=(1, 5)) -> dict:
    out = {}
    for k in topk:
        k = min(k, logits.shape[1])
        out[f"top{k}"] = float((logits.topk(k, 1).indices == target[:, None]).any(1).float().mean())
    pred = logits.argmax(1)
    c = logits.shape[1]
    cm = torch.bincount(target * c + pred, minlength=c * c).reshape(c, c).double()
    prec, rec = cm.diagonal() / cm.sum(0).clamp(min=1), cm.diagonal() / cm.sum(1).clamp(min=1)
    out.update(macro_precision=float(prec.mean()), macro_recall=float(rec.mean()), macro_f1=float((2 * prec * rec / (prec + rec).clamp(min=1e-12)).mean()))
    return out
