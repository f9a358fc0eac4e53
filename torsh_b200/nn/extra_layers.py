"""Layers of the reference's ``torsh-nn`` that ``torch.nn`` does not provide
(``crates/torsh-nn/src/layers/{normalization,attention,regularization,blocks,embedding}``)."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .module import Module


class DepthwiseSeparableConv2d(Module):
    def __init__(self, cin, cout, kernel_size=3, stride=1, padding=1, bias=False):
        super().__init__()
        self.depthwise = torch.nn.Conv2d(cin, cin, kernel_size, stride, padding, groups=cin, bias=False)
        self.pointwise = torch.nn.Conv2d(cin, cout, 1, bias=bias)

    def forward(self, x):
        return self.pointwise(self.depthwise(x))


class WeightStandardizedConv2d(torch.nn.Conv2d):
    def forward(self, x):
        w = self.weight
        w = (w - w.mean((1, 2, 3), keepdim=True)) / (w.std((1, 2, 3), keepdim=True) + 1e-5)
        return F.conv2d(x, w, self.bias, self.stride, self.padding, self.dilation, self.groups)


class BatchRenorm2d(Module):
    """Batch renormalisation: batch statistics corrected towards the running ones by clipped ``r, d``."""

    def __init__(self, c, eps=1e-5, momentum=0.1, r_max=3.0, d_max=5.0):
        super().__init__()
        self.weight, self.bias = torch.nn.Parameter(torch.ones(c)), torch.nn.Parameter(torch.zeros(c))
        self.register_buffer("running_mean", torch.zeros(c)); self.register_buffer("running_std", torch.ones(c))
        self.eps, self.momentum, self.r_max, self.d_max = eps, momentum, r_max, d_max

    def forward(self, x):
        sh = (1, -1, 1, 1)
        if self.training:
            mean, std = x.mean((0, 2, 3)), x.var((0, 2, 3), unbiased=False).add(self.eps).sqrt()
            r = (std.detach() / self.running_std).clamp(1 / self.r_max, self.r_max)
            d = ((mean.detach() - self.running_mean) / self.running_std).clamp(-self.d_max, self.d_max)
            y = (x - mean.view(sh)) / std.view(sh) * r.view(sh) + d.view(sh)
            with torch.no_grad():
                self.running_mean += self.momentum * (mean - self.running_mean)
                self.running_std += self.momentum * (std - self.running_std)
        else:
            y = (x - self.running_mean.view(sh)) / self.running_std.view(sh)
        return y * self.weight.view(sh) + self.bias.view(sh)


class VirtualBatchNorm2d(Module):
    """Normalises with the statistics of a fixed reference batch (set on the first call or via ``set_reference``)."""

    def __init__(self, c, eps=1e-5):
        super().__init__()
        self.weight, self.bias, self.eps = torch.nn.Parameter(torch.ones(c)), torch.nn.Parameter(torch.zeros(c)), eps
        self.register_buffer("ref_mean", torch.zeros(c)); self.register_buffer("ref_var", torch.ones(c))
        self.has_ref = False

    def set_reference(self, x):
        with torch.no_grad():
            self.ref_mean.copy_(x.mean((0, 2, 3))); self.ref_var.copy_(x.var((0, 2, 3), unbiased=False))
        self.has_ref = True

    def forward(self, x):
        if not self.has_ref:
            self.set_reference(x)
        sh = (1, -1, 1, 1)
        return (x - self.ref_mean.view(sh)) / (self.ref_var.view(sh) + self.eps).sqrt() * self.weight.view(sh) + self.bias.view(sh)


class SwitchableNorm2d(Module):
    """Learned softmax mixture of instance-, layer- and batch-norm statistics."""

    def __init__(self, c, eps=1e-5, momentum=0.1):
        super().__init__()
        self.weight, self.bias = torch.nn.Parameter(torch.ones(c)), torch.nn.Parameter(torch.zeros(c))
        self.mean_w, self.var_w = torch.nn.Parameter(torch.ones(3)), torch.nn.Parameter(torch.ones(3))
        self.register_buffer("running_mean", torch.zeros(c)); self.register_buffer("running_var", torch.ones(c))
        self.eps, self.momentum = eps, momentum

    def forward(self, x):
        n, c, h, w = x.shape
        xi = x.reshape(n, c, -1)
        m_in, v_in = xi.mean(-1, keepdim=True), xi.var(-1, keepdim=True, unbiased=False)
        m_ln, t = m_in.mean(1, keepdim=True), (v_in + m_in ** 2).mean(1, keepdim=True)
        v_ln = t - m_ln ** 2
        if self.training:
            m_bn, t = m_in.mean(0, keepdim=True), (v_in + m_in ** 2).mean(0, keepdim=True)
            v_bn = t - m_bn ** 2
            with torch.no_grad():
                self.running_mean += self.momentum * (m_bn.flatten() - self.running_mean)
                self.running_var += self.momentum * (v_bn.flatten() - self.running_var)
        else:
            m_bn, v_bn = self.running_mean.view(1, c, 1), self.running_var.view(1, c, 1)
        mw, vw = torch.softmax(self.mean_w, 0), torch.softmax(self.var_w, 0)
        mean = mw[0] * m_in + mw[1] * m_ln + mw[2] * m_bn
        var = vw[0] * v_in + vw[1] * v_ln + vw[2] * v_bn
        y = ((xi - mean) / (var + self.eps).sqrt()).reshape(n, c, h, w)
        return y * self.weight.view(1, c, 1, 1) + self.bias.view(1, c, 1, 1)


class StochasticDepth(Module):
    def __init__(self, p: float = 0.1, mode: str = "row"):
        super().__init__()
        self.p, self.mode = p, mode

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        shape = [x.shape[0]] + [1] * (x.dim() - 1) if self.mode == "row" else [1] * x.dim()
        keep = torch.empty(shape, dtype=x.dtype, device=x.device).bernoulli_(1 - self.p)
        return x * keep / (1 - self.p)


class DropBlock2d(Module):
    def __init__(self, p: float = 0.1, block_size: int = 7):
        super().__init__()
        self.p, self.bs = p, block_size

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        n, c, h, w = x.shape
        bs = min(self.bs, h, w)
        gamma = self.p * h * w / (bs * bs) / max((h - bs + 1) * (w - bs + 1), 1)
        seeds = (torch.rand(n, c, h, w, device=x.device) < gamma).to(x.dtype)
        mask = 1 - F.max_pool2d(seeds, bs, 1, bs // 2)[..., :h, :w]
        return x * mask * mask.numel() / mask.sum().clamp(min=1)


def mixup(x, y, alpha: float = 0.2, num_classes: int | None = None, generator=None):
    lam = float(torch.distributions.Beta(alpha, alpha).sample()) if alpha > 0 else 1.0
    perm = torch.randperm(x.shape[0], device=x.device, generator=generator)
    yo = F.one_hot(y, num_classes).float() if num_classes else y.float()
    return lam * x + (1 - lam) * x[perm], lam * yo + (1 - lam) * yo[perm]


def cutmix(x, y, alpha: float = 1.0, num_classes: int | None = None, generator=None):
    lam = float(torch.distributions.Beta(alpha, alpha).sample())
    perm = torch.randperm(x.shape[0], device=x.device, generator=generator)
    h, w = x.shape[-2:]
    rh, rw = int(h * math.sqrt(1 - lam)), int(w * math.sqrt(1 - lam))
    cy, cx = int(torch.randint(0, h, (1,))), int(torch.randint(0, w, (1,)))
    y0, y1, x0, x1 = max(cy - rh // 2, 0), min(cy + rh // 2, h), max(cx - rw // 2, 0), min(cx + rw // 2, w)
    out = x.clone()
    out[..., y0:y1, x0:x1] = x[perm][..., y0:y1, x0:x1]
    lam = 1 - (y1 - y0) * (x1 - x0) / (h * w)
    yo = F.one_hot(y, num_classes).float() if num_classes else y.float()
    return out, lam * yo + (1 - lam) * yo[perm]


class AdditiveAttention(Module):
    """Bahdanau scoring ``vᵀ tanh(W_q q + W_k k)``."""

    def __init__(self, q_dim, k_dim, hidden):
        super().__init__()
        self.wq, self.wk, self.v = torch.nn.Linear(q_dim, hidden, bias=False), torch.nn.Linear(k_dim, hidden, bias=False), torch.nn.Linear(hidden, 1, bias=False)

    def forward(self, q, k, v, mask=None):
        s = self.v(torch.tanh(self.wq(q)[:, :, None] + self.wk(k)[:, None])).squeeze(-1)
        if mask is not None:
            s = s.masked_fill(~mask, float("-inf"))
        a = torch.softmax(s, -1)
        return a @ v, a


class MultiplicativeAttention(Module):
    """Luong scoring ``qᵀ W k`` (``general``) or plain dot product."""

    def __init__(self, q_dim, k_dim, mode="general"):
        super().__init__()
        self.w = torch.nn.Linear(k_dim, q_dim, bias=False) if mode == "general" else None

    def forward(self, q, k, v, mask=None):
        s = q @ (self.w(k) if self.w is not None else k).transpose(-1, -2)
        if mask is not None:
            s = s.masked_fill(~mask, float("-inf"))
        a = torch.softmax(s, -1)
        return a @ v, a


class CrossAttention(Module):
    def __init__(self, dim, context_dim=None, heads=8):
        super().__init__()
        self.h = heads
        self.q, self.kv, self.o = torch.nn.Linear(dim, dim), torch.nn.Linear(context_dim or dim, 2 * dim), torch.nn.Linear(dim, dim)

    def forward(self, x, context):
        b, s, d = x.shape
        q = self.q(x).view(b, s, self.h, -1).transpose(1, 2)
        k, v = self.kv(context).view(b, context.shape[1], 2, self.h, -1).permute(2, 0, 3, 1, 4)
        return self.o(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, s, d))


class FlexAttention(Module):
    """Attention with a pattern chosen by name: ``causal``, ``sliding_window(w)``, ``block_diagonal(b)``, ``global_local``."""

    def __init__(self, dim, heads=8, pattern="causal", window=128, block=64, n_global=1):
        super().__init__()
        self.h, self.pattern, self.window, self.block, self.n_global = heads, pattern, window, block, n_global
        self.qkv, self.o = torch.nn.Linear(dim, 3 * dim), torch.nn.Linear(dim, dim)

    def mask(self, s, device):
        i, j = torch.arange(s, device=device)[:, None], torch.arange(s, device=device)[None]
        if self.pattern == "causal":
            return j <= i
        if self.pattern == "sliding_window":
            return (j <= i) & (i - j < self.window)
        if self.pattern == "block_diagonal":
            return i // self.block == j // self.block
        if self.pattern == "global_local":
            return ((i - j).abs() < self.window) | (j < self.n_global) | (i < self.n_global)
        return torch.ones(s, s, dtype=torch.bool, device=device)

    def forward(self, x):
        b, s, d = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.h, -1).permute(2, 0, 3, 1, 4)
        if self.pattern == "causal" and x.is_cuda and x.dtype == torch.bfloat16:
            from ..ops.attention import flash_attention
            y = flash_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=True).reshape(b, s, d)
        else:
            y = F.scaled_dot_product_attention(q, k, v, attn_mask=self.mask(s, x.device)).transpose(1, 2).reshape(b, s, d)
        return self.o(y)


class RelativePositionBias(Module):
    """T5-style bucketed relative position bias ``[heads, q, k]``."""

    def __init__(self, heads, num_buckets=32, max_distance=128, bidirectional=True):
        super().__init__()
        self.nb, self.md, self.bi = num_buckets, max_distance, bidirectional
        self.emb = torch.nn.Embedding(num_buckets, heads)

    def _bucket(self, rel):
        nb, ret = self.nb, 0
        if self.bi:
            nb //= 2
            ret = (rel > 0).long() * nb
            rel = rel.abs()
        else:
            rel = (-rel).clamp(min=0)
        exact = nb // 2
        large = exact + (torch.log(rel.float().clamp(min=1) / exact) / math.log(self.md / exact) * (nb - exact)).long()
        return ret + torch.where(rel < exact, rel, large.clamp(max=nb - 1))

    def forward(self, q_len, k_len):
        dev = self.emb.weight.device
        rel = torch.arange(k_len, device=dev)[None] - torch.arange(q_len, device=dev)[:, None]
        return self.emb(self._bucket(rel)).permute(2, 0, 1)


def interpolate_positions(pos_emb: torch.Tensor, new_len: int) -> torch.Tensor:
    """Position interpolation: stretch a learned ``[L, D]`` table to ``new_len`` rows (linear)."""
    return F.interpolate(pos_emb.t()[None], size=new_len, mode="linear", align_corners=True)[0].t()


class MBConvBlock(Module):
    """MobileNetV2 / EfficientNet inverted residual with optional squeeze-excitation."""

    def __init__(self, cin, cout, expand=4, kernel=3, stride=1, se_ratio=0.25, drop_path=0.0):
        super().__init__()
        mid = cin * expand
        layers = [] if expand == 1 else [torch.nn.Conv2d(cin, mid, 1, bias=False), torch.nn.BatchNorm2d(mid), torch.nn.SiLU()]
        layers += [torch.nn.Conv2d(mid, mid, kernel, stride, kernel // 2, groups=mid, bias=False), torch.nn.BatchNorm2d(mid), torch.nn.SiLU()]
        self.body = torch.nn.Sequential(*layers)
        sq = max(1, int(cin * se_ratio)) if se_ratio else 0
        self.se = torch.nn.Sequential(torch.nn.AdaptiveAvgPool2d(1), torch.nn.Conv2d(mid, sq, 1), torch.nn.SiLU(), torch.nn.Conv2d(sq, mid, 1), torch.nn.Sigmoid()) if sq else None
        self.project = torch.nn.Sequential(torch.nn.Conv2d(mid, cout, 1, bias=False), torch.nn.BatchNorm2d(cout))
        self.skip = stride == 1 and cin == cout
        self.drop = StochasticDepth(drop_path)

    def forward(self, x):
        y = self.body(x)
        if self.se is not None:
            y = y * self.se(y)
        y = self.project(y)
        return x + self.drop(y) if self.skip else y


class DenseBlock(Module):
    def __init__(self, cin, growth, layers):
        super().__init__()
        self.layers = torch.nn.ModuleList(torch.nn.Sequential(torch.nn.BatchNorm2d(cin + i * growth), torch.nn.ReLU(), torch.nn.Conv2d(cin + i * growth, growth, 3, padding=1, bias=False)) for i in range(layers))

    def forward(self, x):
        for layer in self.layers:
            x = torch.cat([x, layer(x)], 1)
        return x


class GlobalAvgPool2d(Module):
    def forward(self, x): return x.mean((2, 3))


class GlobalMaxPool2d(Module):
    def forward(self, x): return x.amax((2, 3))


class LocationBasedAttention(Module):
    """Location-aware scoring (``crates/torsh-nn/src/layers/attention.rs``): the previous alignment is convolved along
    time and enters the additive score, ``vᵀ tanh(W_q q + W_k k + W_f (F * a_prev))``."""

    def __init__(self, q_dim, k_dim, hidden, conv_channels: int = 32, kernel_size: int = 31):
        super().__init__()
        self.wq, self.wk = torch.nn.Linear(q_dim, hidden, bias=False), torch.nn.Linear(k_dim, hidden, bias=False)
        self.loc = torch.nn.Conv1d(1, conv_channels, kernel_size, padding=kernel_size // 2, bias=False)
        self.wf, self.v = torch.nn.Linear(conv_channels, hidden, bias=False), torch.nn.Linear(hidden, 1, bias=False)

    def forward(self, q, k, v, prev_alignment=None, mask=None):
        """``q``: ``[B, q_dim]`` (one decoder step); ``k, v``: ``[B, T, ·]``; ``prev_alignment``: ``[B, T]``."""
        b, t, _ = k.shape
        if prev_alignment is None:
            prev_alignment = torch.zeros(b, t, device=k.device, dtype=k.dtype)
        f = self.loc(prev_alignment[:, None]).transpose(1, 2)               # [B, T, conv_channels]
        s = self.v(torch.tanh(self.wq(q)[:, None] + self.wk(k) + self.wf(f))).squeeze(-1)
        if mask is not None:
            s = s.masked_fill(~mask, float("-inf"))
        a = torch.softmax(s, -1)
        return (a[:, None] @ v).squeeze(1), a


class Mixup(Module):
    """Batch-level mixup as a module (``crates/torsh-nn/src/layers/regularization``); identity in eval mode."""

    def __init__(self, alpha: float = 0.2, num_classes: int | None = None):
        super().__init__()
        self.alpha, self.num_classes = alpha, num_classes

    def forward(self, x, y):
        if not self.training:
            return x, (F.one_hot(y, self.num_classes).float() if self.num_classes else y)
        return mixup(x, y, self.alpha, self.num_classes)


class CutMix(Module):
    def __init__(self, alpha: float = 1.0, num_classes: int | None = None):
        super().__init__()
        self.alpha, self.num_classes = alpha, num_classes

    def forward(self, x, y):
        if not self.training:
            return x, (F.one_hot(y, self.num_classes).float() if self.num_classes else y)
        return cutmix(x, y, self.alpha, self.num_classes)


class PositionInterpolation(Module):
    """Rotary embedding whose positions are scaled by ``train_len / target_len`` so a model trained on ``train_len``
    tokens addresses ``target_len`` (``crates/torsh-nn/src/layers/embedding.rs``: position interpolation)."""

    def __init__(self, head_dim: int, train_len: int, target_len: int, base: float = 10000.0):
        super().__init__()
        self.scale = min(1.0, train_len / float(target_len))
        inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
        self.register_buffer("inv_freq", inv, persistent=False)

    def forward(self, x, offset: int = 0):
        """``x``: ``[B, S, H, D]``; rotates pairs ``(x[2i], x[2i+1])`` by the scaled position angle."""
        s = x.shape[1]
        pos = (torch.arange(s, device=x.device, dtype=torch.float32) + offset) * self.scale
        ang = pos[:, None] * self.inv_freq.to(x.device)[None]
        cos, sin = ang.cos()[None, :, None], ang.sin()[None, :, None]
        xf = x.float()
        a, b = xf[..., 0::2], xf[..., 1::2]
        return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).flatten(-2).to(x.dtype)


class WeightStandardization(Module):
    """Wraps a convolution / linear layer and standardises its weight per output unit on every forward."""

    def __init__(self, module: torch.nn.Module, eps: float = 1e-5):
        super().__init__()
        self.module, self.eps = module, eps

    def forward(self, x):
        w = self.module.weight
        dims = tuple(range(1, w.dim()))
        ws = (w - w.mean(dims, keepdim=True)) / (w.var(dims, keepdim=True, unbiased=False) + self.eps).sqrt()
        return torch.func.functional_call(self.module, {"weight": ws}, (x,), strict=False)


def WeightNorm(module: torch.nn.Module, name: str = "weight", dim: int = 0):
    """``w = g · v / ‖v‖`` re-parametrisation (``crates/torsh-nn/src/layers/normalization``: weight norm)."""
    return torch.nn.utils.parametrizations.weight_norm(module, name, dim)


def SpectralNorm(module: torch.nn.Module, name: str = "weight", n_power_iterations: int = 1, eps: float = 1e-12):
    """Divides the weight by its largest singular value, tracked by power iteration."""
    return torch.nn.utils.parametrizations.spectral_norm(module, name, n_power_iterations, eps)


LazyLinear = torch.nn.LazyLinear
LazyConv2d = torch.nn.LazyConv2d
