"""Named building blocks of the reference's layer library (``crates/torsh-nn/src/layers/``): activation and normalisation
factories with presets and statistics (``activation/``, ``normalization/``), positional encodings and attention bias
(``attention.rs``, ``embedding.rs``), multi-head attention with the reference's constructor (``attention.rs``), gated linear
units (``activation/gated.rs``), residual, dense and mobile blocks with the small backbones built from them (``blocks.rs``,
``mobilenet.rs``, ``efficientnet.rs``), pooling variants (``pooling/``) and a cell-level recurrent layer (``recurrent.rs``)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Callable, Sequence

import torch
import torch.nn.functional as F
from torch import nn

__all__ = ["ActivationFactory", "ActivationBuilder", "AdvancedLayerNorm", "NormalizationConfig", "NormalizationFactory", "NormalizationPresets", "NormalizationStats", "PositionalEncoding", "SinusoidalPositionEmbedding",
           "RelativePositionalEncoding", "AlibiPositionalBias", "MultiHeadAttention", "GEGLU", "BasicBlock", "BottleneckBlock", "DenseLayer", "TransitionLayer", "DepthwiseSeparableConv", "InvertedResidual", "MobileNetV1Block",
           "MobileNetV2Block", "MobileNetConfig", "MobileNetV1", "MBConvWithStochasticDepth", "EfficientNetConfig", "EfficientNetBackbone", "GlobalPool", "FractionalMaxPool1d", "CustomRNNCell", "BlockConfig"]


# ================================================================================================ factories
class ActivationFactory:
    """Activations by name (case-insensitive), with keyword arguments passed through."""
    TABLE = {"relu": nn.ReLU, "relu6": nn.ReLU6, "leaky_relu": nn.LeakyReLU, "prelu": nn.PReLU, "elu": nn.ELU, "selu": nn.SELU, "celu": nn.CELU, "gelu": nn.GELU, "silu": nn.SiLU, "swish": nn.SiLU, "mish": nn.Mish, "tanh": nn.Tanh,
             "sigmoid": nn.Sigmoid, "hardswish": nn.Hardswish, "hardsigmoid": nn.Hardsigmoid, "hardtanh": nn.Hardtanh, "softplus": nn.Softplus, "softsign": nn.Softsign, "softmax": nn.Softmax, "log_softmax": nn.LogSoftmax, "identity": nn.Identity,
             "tanhshrink": nn.Tanhshrink, "softshrink": nn.Softshrink, "hardshrink": nn.Hardshrink, "threshold": nn.Threshold, "glu": nn.GLU}

    @classmethod
    def create(cls, name: str, **kw) -> nn.Module:
        key = name.lower().replace("-", "_")
        if key == "geglu":
            return GEGLU(**kw)
        if key not in cls.TABLE:
            raise ValueError(f"unknown activation {name!r}; known: {', '.join(sorted(cls.TABLE))}, geglu")
        return cls.TABLE[key](**kw)

    @classmethod
    def available(cls) -> list[str]: return sorted(list(cls.TABLE) + ["geglu"])


class ActivationBuilder:
    """``ActivationBuilder("leaky_relu").negative_slope(0.2).inplace().build()``: keyword arguments collected fluently."""

    def __init__(self, name: str): self.name, self.kw = name, {}
    def inplace(self, flag: bool = True): self.kw["inplace"] = flag; return self
    def __getattr__(self, key):
        if key.startswith("_"):
            raise AttributeError(key)
        def setter(value): self.kw[key] = value; return self
        return setter
    def build(self) -> nn.Module: return ActivationFactory.create(self.name, **self.kw)


class AdvancedLayerNorm(nn.Module):
    """Layer normalisation with switches: RMS mode (no centring), no bias, and a residual input added before normalising
    (the pre-norm ``x + r`` fusion); statistics are accumulated in float32 for half-precision inputs."""

    def __init__(self, dim: int, eps: float = 1e-5, rms: bool = False, bias: bool = True, elementwise_affine: bool = True):
        super().__init__()
        self.dim, self.eps, self.rms = dim, eps, rms
        self.weight = nn.Parameter(torch.ones(dim)) if elementwise_affine else None
        self.bias = nn.Parameter(torch.zeros(dim)) if elementwise_affine and bias and not rms else None

    def forward(self, x, residual: torch.Tensor | None = None):
        h = (x + residual if residual is not None else x).float()
        if self.rms:
            y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)
        else:
            mu = h.mean(-1, keepdim=True)
            y = (h - mu) * torch.rsqrt((h - mu).pow(2).mean(-1, keepdim=True) + self.eps)
        if self.weight is not None:
            y = y * self.weight.float()
        if self.bias is not None:
            y = y + self.bias.float()
        return y.to(x.dtype)


@dataclass
class NormalizationConfig:
    kind: str = "layer"                                                              # batch | layer | group | instance | rms | none
    eps: float = 1e-5
    momentum: float = 0.1
    affine: bool = True
    groups: int = 32
    dims: int = 2                                                                    # spatial dimensions for batch / instance norm


class NormalizationFactory:
    @staticmethod
    def create(cfg: NormalizationConfig | str, features: int, **kw) -> nn.Module:
        cfg = NormalizationConfig(kind=cfg, **kw) if isinstance(cfg, str) else cfg
        k = cfg.kind.lower()
        if k == "batch":
            return {1: nn.BatchNorm1d, 2: nn.BatchNorm2d, 3: nn.BatchNorm3d}[cfg.dims](features, cfg.eps, cfg.momentum, cfg.affine)
        if k == "instance":
            return {1: nn.InstanceNorm1d, 2: nn.InstanceNorm2d, 3: nn.InstanceNorm3d}[cfg.dims](features, cfg.eps, cfg.momentum, cfg.affine)
        if k == "layer":
            return nn.LayerNorm(features, cfg.eps, cfg.affine)
        if k == "rms":
            return AdvancedLayerNorm(features, cfg.eps, rms=True, elementwise_affine=cfg.affine)
        if k == "group":
            g = math.gcd(cfg.groups, features)
            return nn.GroupNorm(g, features, cfg.eps, cfg.affine)
        if k == "none":
            return nn.Identity()
        raise ValueError(f"unknown normalisation {cfg.kind!r}")


class NormalizationPresets:
    """Configurations that families of models use."""
    @staticmethod
    def resnet() -> NormalizationConfig: return NormalizationConfig("batch", 1e-5, 0.1, True, dims=2)
    @staticmethod
    def transformer() -> NormalizationConfig: return NormalizationConfig("layer", 1e-5)
    @staticmethod
    def llama() -> NormalizationConfig: return NormalizationConfig("rms", 1e-6)
    @staticmethod
    def diffusion_unet() -> NormalizationConfig: return NormalizationConfig("group", 1e-5, groups=32)
    @staticmethod
    def style_transfer() -> NormalizationConfig: return NormalizationConfig("instance", 1e-5, affine=True, dims=2)


class NormalizationStats:
    """Per-layer mean, variance and range of what a normalisation layer receives and emits (a forward hook)."""

    def __init__(self, layer: nn.Module):
        self.records = []
        self._h = layer.register_forward_hook(self._hook)
    def _hook(self, mod, inp, out):
        i, o = inp[0].detach().float(), out.detach().float()
        self.records.append({"in_mean": float(i.mean()), "in_var": float(i.var()), "out_mean": float(o.mean()), "out_var": float(o.var()), "out_abs_max": float(o.abs().max())})
    def summary(self) -> dict:
        n = max(len(self.records), 1)
        return {k: sum(r[k] for r in self.records) / n for k in (self.records[0] if self.records else {})}
    def remove(self): self._h.remove()


# ================================================================================================ positions and attention
class PositionalEncoding(nn.Module):
    """Adds fixed sinusoids to ``[batch, seq, dim]`` inputs, with dropout."""

    def __init__(self, d_model: int, dropout: float = 0.0, max_len: int = 5000):
        super().__init__()
        pos = torch.arange(max_len)[:, None]
        div = torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div); pe[:, 1::2] = torch.cos(pos * div[: d_model // 2])
        self.register_buffer("pe", pe); self.drop = nn.Dropout(dropout)
    def forward(self, x): return self.drop(x + self.pe[: x.shape[1]].to(x.dtype))


class SinusoidalPositionEmbedding(nn.Module):
    """Embedding of scalar positions or diffusion time steps ``[batch] -> [batch, dim]`` (sine half, cosine half)."""

    def __init__(self, dim: int, max_period: float = 10000.0): super().__init__(); self.dim, self.max_period = dim, max_period
    def forward(self, t):
        half = self.dim // 2
        freqs = torch.exp(-math.log(self.max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
        a = t.float()[..., None] * freqs
        return torch.cat([a.sin(), a.cos()], -1)


class RelativePositionalEncoding(nn.Module):
    """Learned bias per head and clipped relative distance, added to attention scores (``[heads, q, k]``)."""

    def __init__(self, num_heads: int, max_distance: int = 128):
        super().__init__()
        self.max_distance, self.table = max_distance, nn.Embedding(2 * max_distance + 1, num_heads)
    def forward(self, q_len: int, k_len: int) -> torch.Tensor:
        rel = torch.arange(k_len, device=self.table.weight.device)[None] - torch.arange(q_len, device=self.table.weight.device)[:, None]
        return self.table(rel.clamp(-self.max_distance, self.max_distance) + self.max_distance).permute(2, 0, 1)


class AlibiPositionalBias(nn.Module):
    """Attention with linear biases: head ``h`` subtracts ``slope_h |i - j|`` from the scores; slopes form the geometric sequence
    of the original method (also for head counts that are not powers of two)."""

    def __init__(self, num_heads: int, causal: bool = True):
        super().__init__()
        def pow2(n): s = 2.0 ** (-8.0 / n); return [s ** (i + 1) for i in range(n)]
        if math.log2(num_heads).is_integer():
            slopes = pow2(num_heads)
        else:
            p = 2 ** math.floor(math.log2(num_heads))
            slopes = pow2(p) + pow2(2 * p)[0::2][: num_heads - p]
        self.register_buffer("slopes", torch.tensor(slopes)); self.causal = causal
    def forward(self, q_len: int, k_len: int) -> torch.Tensor:
        rel = torch.arange(k_len, device=self.slopes.device)[None] - torch.arange(q_len, device=self.slopes.device)[:, None] - (k_len - q_len)
        bias = -self.slopes[:, None, None] * rel.abs()
        return bias.masked_fill(rel[None] > 0, float("-inf")) if self.causal else bias


class MultiHeadAttention(nn.Module):
    """``MultiHeadAttention(embed_dim, num_heads, dropout, bias)`` on batch-first inputs; optional additive bias (relative or
    ALiBi), key-padding mask and causal flag; returns the output and, when asked, the head-averaged weights."""

    def __init__(self, embed_dim: int, num_heads: int, dropout: float = 0.0, bias: bool = True):
        super().__init__()
        if embed_dim % num_heads:
            raise ValueError("embed_dim must be divisible by num_heads")
        self.h, self.d, self.p = num_heads, embed_dim // num_heads, dropout
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(embed_dim, embed_dim, bias=bias) for _ in range(4))

    def forward(self, query, key=None, value=None, attn_bias: torch.Tensor | None = None, key_padding_mask: torch.Tensor | None = None, causal: bool = False, need_weights: bool = False):
        key = query if key is None else key
        value = key if value is None else value
        B, Lq, _ = query.shape
        split = lambda t: t.view(B, -1, self.h, self.d).transpose(1, 2)
        q, k, v = split(self.q_proj(query)), split(self.k_proj(key)), split(self.v_proj(value))
        mask = None
        if attn_bias is not None:
            mask = attn_bias.to(q.dtype).expand(B, self.h, Lq, k.shape[2]) if attn_bias.dim() == 3 else attn_bias.to(q.dtype)
        if key_padding_mask is not None:
            pad = torch.zeros(B, 1, 1, k.shape[2], dtype=q.dtype, device=q.device).masked_fill(key_padding_mask[:, None, None, :], float("-inf"))
            mask = pad if mask is None else mask + pad
        if causal:
            cm = torch.full((Lq, k.shape[2]), float("-inf"), dtype=q.dtype, device=q.device).triu(1 + k.shape[2] - Lq)
            mask = cm if mask is None else mask + cm
        if need_weights:
            w = (q @ k.transpose(-1, -2) / math.sqrt(self.d) + (mask if mask is not None else 0)).softmax(-1)
            out = F.dropout(w, self.p, self.training) @ v
        else:
            w, out = None, F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=self.p if self.training else 0.0)
        out = self.out_proj(out.transpose(1, 2).reshape(B, Lq, self.h * self.d))
        return (out, w.mean(1)) if need_weights else out


class GEGLU(nn.Module):
    """``GELU(x W_g) * (x W_v)`` with both projections in one matrix; without dimensions it gates the two halves of its input."""

    def __init__(self, in_features: int | None = None, out_features: int | None = None, bias: bool = True):
        super().__init__()
        self.proj = nn.Linear(in_features, 2 * out_features, bias=bias) if in_features else None
    def forward(self, x):
        a, b = (self.proj(x) if self.proj is not None else x).chunk(2, -1)
        return F.gelu(a) * b


# ================================================================================================ convolutional blocks
@dataclass
class BlockConfig:
    norm: str = "batch"
    activation: str = "relu"
    dropout: float = 0.0


def _cna(cin, cout, k, stride=1, groups=1, cfg: BlockConfig | None = None, act: bool = True):
    cfg = cfg or BlockConfig()
    layers = [nn.Conv2d(cin, cout, k, stride, k // 2, groups=groups, bias=cfg.norm == "none"), NormalizationFactory.create(cfg.norm, cout, dims=2)]
    return nn.Sequential(*layers, ActivationFactory.create(cfg.activation)) if act else nn.Sequential(*layers)


class BasicBlock(nn.Module):
    expansion = 1
    def __init__(self, in_channels: int, out_channels: int, stride: int = 1, cfg: BlockConfig | None = None):
        super().__init__()
        self.body = nn.Sequential(_cna(in_channels, out_channels, 3, stride, cfg=cfg), _cna(out_channels, out_channels, 3, cfg=cfg, act=False))
        self.short = None if stride == 1 and in_channels == out_channels else _cna(in_channels, out_channels, 1, stride, cfg=cfg, act=False)
        self.act = ActivationFactory.create((cfg or BlockConfig()).activation)
    def forward(self, x): return self.act(self.body(x) + (x if self.short is None else self.short(x)))


class BottleneckBlock(nn.Module):
    expansion = 4
    def __init__(self, in_channels: int, width: int, stride: int = 1, cfg: BlockConfig | None = None):
        super().__init__()
        out = width * self.expansion
        self.body = nn.Sequential(_cna(in_channels, width, 1, cfg=cfg), _cna(width, width, 3, stride, cfg=cfg), _cna(width, out, 1, cfg=cfg, act=False))
        self.short = None if stride == 1 and in_channels == out else _cna(in_channels, out, 1, stride, cfg=cfg, act=False)
        self.act = ActivationFactory.create((cfg or BlockConfig()).activation)
    def forward(self, x): return self.act(self.body(x) + (x if self.short is None else self.short(x)))


class DenseLayer(nn.Module):
    """DenseNet layer: BN-ReLU-1x1 (bottleneck of ``bn_size * growth``), BN-ReLU-3x3 producing ``growth`` channels, concatenated
    to the input."""

    def __init__(self, in_channels: int, growth_rate: int = 32, bn_size: int = 4, dropout: float = 0.0):
        super().__init__()
        mid = bn_size * growth_rate
        self.body = nn.Sequential(nn.BatchNorm2d(in_channels), nn.ReLU(), nn.Conv2d(in_channels, mid, 1, bias=False), nn.BatchNorm2d(mid), nn.ReLU(), nn.Conv2d(mid, growth_rate, 3, padding=1, bias=False), nn.Dropout(dropout))
    def forward(self, x): return torch.cat([x, self.body(x)], 1)


class TransitionLayer(nn.Module):
    def __init__(self, in_channels: int, out_channels: int | None = None):
        super().__init__()
        self.body = nn.Sequential(nn.BatchNorm2d(in_channels), nn.ReLU(), nn.Conv2d(in_channels, out_channels or in_channels // 2, 1, bias=False), nn.AvgPool2d(2))
    def forward(self, x): return self.body(x)


class DepthwiseSeparableConv(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1, cfg: BlockConfig | None = None):
        super().__init__()
        self.depthwise, self.pointwise = _cna(in_channels, in_channels, kernel_size, stride, groups=in_channels, cfg=cfg), _cna(in_channels, out_channels, 1, cfg=cfg)
    def forward(self, x): return self.pointwise(self.depthwise(x))
    def multiply_adds(self, h: int, w: int) -> int:
        dw, pw = self.depthwise[0], self.pointwise[0]
        oh, ow = h // dw.stride[0], w // dw.stride[1]
        return oh * ow * (dw.in_channels * dw.kernel_size[0] * dw.kernel_size[1] + pw.in_channels * pw.out_channels)


MobileNetV1Block = DepthwiseSeparableConv


class InvertedResidual(nn.Module):
    """Expand 1x1 - depthwise 3x3 - linear 1x1 projection, with the identity when stride is 1 and channels match."""

    def __init__(self, in_channels: int, out_channels: int, stride: int = 1, expand_ratio: float = 6.0, kernel_size: int = 3, activation: str = "relu6"):
        super().__init__()
        cfg, mid = BlockConfig(activation=activation), int(round(in_channels * expand_ratio))
        layers = [] if expand_ratio == 1 else [_cna(in_channels, mid, 1, cfg=cfg)]
        layers += [_cna(mid, mid, kernel_size, stride, groups=mid, cfg=cfg), _cna(mid, out_channels, 1, cfg=cfg, act=False)]
        self.body, self.use_res = nn.Sequential(*layers), stride == 1 and in_channels == out_channels
    def forward(self, x): return x + self.body(x) if self.use_res else self.body(x)


MobileNetV2Block = InvertedResidual


@dataclass
class MobileNetConfig:
    num_classes: int = 1000
    width_multiplier: float = 1.0
    in_channels: int = 3
    dropout: float = 0.0
    layers: Sequence[tuple[int, int]] = ((64, 1), (128, 2), (128, 1), (256, 2), (256, 1), (512, 2), (512, 1), (512, 1), (512, 1), (512, 1), (512, 1), (1024, 2), (1024, 1))


class MobileNetV1(nn.Module):
    def __init__(self, cfg: MobileNetConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or MobileNetConfig(**kw)
        c = lambda v: max(8, int(v * cfg.width_multiplier))
        feats, cin = [_cna(cfg.in_channels, c(32), 3, 2)], c(32)
        for ch, s in cfg.layers:
            feats.append(DepthwiseSeparableConv(cin, c(ch), 3, s)); cin = c(ch)
        self.features, self.head = nn.Sequential(*feats), nn.Sequential(GlobalPool("avg"), nn.Dropout(cfg.dropout), nn.Linear(cin, cfg.num_classes))
    def forward(self, x): return self.head(self.features(x))


class MBConvWithStochasticDepth(nn.Module):
    """EfficientNet block: expansion, depthwise convolution, squeeze-and-excitation, projection; the residual branch is dropped
    per sample with probability ``drop_rate`` during training (and rescaled)."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size: int = 3, stride: int = 1, expand_ratio: float = 6.0, se_ratio: float = 0.25, drop_rate: float = 0.0):
        super().__init__()
        cfg, mid = BlockConfig(activation="silu"), int(round(in_channels * expand_ratio))
        self.expand = _cna(in_channels, mid, 1, cfg=cfg) if expand_ratio != 1 else nn.Identity()
        self.dw = _cna(mid, mid, kernel_size, stride, groups=mid, cfg=cfg)
        sq = max(1, int(in_channels * se_ratio))
        self.se = nn.Sequential(nn.AdaptiveAvgPool2d(1), nn.Conv2d(mid, sq, 1), nn.SiLU(), nn.Conv2d(sq, mid, 1), nn.Sigmoid())
        self.project = _cna(mid, out_channels, 1, cfg=cfg, act=False)
        self.use_res, self.drop_rate = stride == 1 and in_channels == out_channels, drop_rate

    def forward(self, x):
        h = self.dw(self.expand(x))
        h = self.project(h * self.se(h))
        if not self.use_res:
            return h
        if self.training and self.drop_rate > 0:
            keep = (torch.rand(x.shape[0], 1, 1, 1, device=x.device) >= self.drop_rate).to(x.dtype)
            h = h * keep / (1 - self.drop_rate)
        return x + h


@dataclass
class EfficientNetConfig:
    width_coefficient: float = 1.0
    depth_coefficient: float = 1.0
    dropout: float = 0.2
    drop_connect_rate: float = 0.2
    num_classes: int = 1000
    in_channels: int = 3
    stages: Sequence[tuple[float, int, int, int, int]] = ((1, 16, 1, 1, 3), (6, 24, 2, 2, 3), (6, 40, 2, 2, 5), (6, 80, 3, 2, 3), (6, 112, 3, 1, 5), (6, 192, 4, 2, 5), (6, 320, 1, 1, 3))   # expand, channels, repeats, stride, kernel

    def round_channels(self, c: int, divisor: int = 8) -> int:
        c *= self.width_coefficient
        new = max(divisor, int(c + divisor / 2) // divisor * divisor)
        return new + divisor if new < 0.9 * c else new
    def round_repeats(self, r: int) -> int: return int(math.ceil(self.depth_coefficient * r))


class EfficientNetBackbone(nn.Module):
    def __init__(self, cfg: EfficientNetConfig | None = None, **kw):
        super().__init__()
        self.cfg = cfg = cfg or EfficientNetConfig(**kw)
        sc = BlockConfig(activation="silu")
        stem = cfg.round_channels(32)
        blocks, cin = [_cna(cfg.in_channels, stem, 3, 2, cfg=sc)], stem
        total = sum(cfg.round_repeats(r) for _, _, r, _, _ in cfg.stages)
        idx = 0
        for e, c, r, s, k in cfg.stages:
            cout = cfg.round_channels(c)
            for j in range(cfg.round_repeats(r)):
                blocks.append(MBConvWithStochasticDepth(cin, cout, k, s if j == 0 else 1, e, drop_rate=cfg.drop_connect_rate * idx / total)); cin, idx = cout, idx + 1
        head = cfg.round_channels(1280)
        self.features = nn.Sequential(*blocks, _cna(cin, head, 1, cfg=sc))
        self.classifier = nn.Sequential(GlobalPool("avg"), nn.Dropout(cfg.dropout), nn.Linear(head, cfg.num_classes))
        self.out_channels = head
    def forward(self, x): return self.classifier(self.features(x))
    def forward_features(self, x): return self.features(x)


# ================================================================================================ pooling and recurrence
class GlobalPool(nn.Module):
    """Global ``avg``, ``max``, ``avgmax`` (their mean) or ``catavgmax`` (concatenated) pooling over all spatial dimensions, flattened."""

    def __init__(self, kind: str = "avg"): super().__init__(); self.kind = kind
    def forward(self, x):
        dims = tuple(range(2, x.dim()))
        a, m = x.mean(dims), x.amax(dims)
        return {"avg": a, "max": m, "avgmax": 0.5 * (a + m), "catavgmax": torch.cat([a, m], 1)}[self.kind]


class FractionalMaxPool1d(nn.Module):
    """Max pooling with a non-integer reduction: window starts follow a pseudo-random increasing sequence with steps of
    ``floor`` or ``ceil`` of the ratio (a fresh sequence per call in training, a fixed one in evaluation)."""

    def __init__(self, kernel_size: int = 2, output_ratio: float = 0.7): super().__init__(); self.k, self.ratio = kernel_size, output_ratio
    def forward(self, x):
        L = x.shape[-1]
        out_len = max(1, int(L * self.ratio))
        alpha = (L - self.k) / max(out_len - 1, 1)
        u = float(torch.rand(())) if self.training else 0.5
        starts = torch.tensor([min(L - self.k, int(math.ceil(alpha * (i + u))) - 1 if i else 0) for i in range(out_len)]).clamp(min=0)
        idx = starts[:, None] + torch.arange(self.k)[None]
        return x[..., idx.to(x.device)].amax(-1)


class CustomRNNCell(nn.Module):
    """Recurrent cell with a chosen non-linearity, optional layer normalisation of the pre-activation and a learned initial
    state; ``unroll`` runs it over a ``[batch, time, features]`` sequence."""

    def __init__(self, input_size: int, hidden_size: int, activation: str = "tanh", layer_norm: bool = False, learn_initial_state: bool = False):
        super().__init__()
        self.ih, self.hh = nn.Linear(input_size, hidden_size), nn.Linear(hidden_size, hidden_size, bias=False)
        self.act, self.norm = ActivationFactory.create(activation), nn.LayerNorm(hidden_size) if layer_norm else nn.Identity()
        self.h0 = nn.Parameter(torch.zeros(hidden_size)) if learn_initial_state else None
        self.hidden_size = hidden_size
    def initial_state(self, batch: int, device=None): return (self.h0.expand(batch, -1) if self.h0 is not None else torch.zeros(batch, self.hidden_size, device=device))
    def forward(self, x, h=None): return self.act(self.norm(self.ih(x) + self.hh(self.initial_state(x.shape[0], x.device) if h is None else h)))
    def unroll(self, seq, h=None):
        outs = []
        for t in range(seq.shape[1]):
            h = self(seq[:, t], h); outs.append(h)
        return torch.stack(outs, 1), h
