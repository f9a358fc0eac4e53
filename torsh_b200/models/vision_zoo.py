"""Convolutional and hierarchical-transformer image classifiers of the reference's zoo
(``crates/torsh-vision/src/models/*.rs``, ``crates/torsh-models/src/vision/*``): AlexNet, VGG, DenseNet, MobileNetV2,
EfficientNet-B0, ConvNeXt and Swin. Standard architectures on ``torch.nn`` layers; every model maps ``[B, 3, H, W]`` to
``[B, num_classes]`` and takes ``width`` / ``depth`` style arguments so tests can build small variants."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class AlexNet(nn.Module):
    def __init__(self, num_classes: int = 1000, dropout: float = 0.5):
        super().__init__()
        self.features = nn.Sequential(
            nn.Conv2d(3, 64, 11, 4, 2), nn.ReLU(True), nn.MaxPool2d(3, 2),
            nn.Conv2d(64, 192, 5, padding=2), nn.ReLU(True), nn.MaxPool2d(3, 2),
            nn.Conv2d(192, 384, 3, padding=1), nn.ReLU(True), nn.Conv2d(384, 256, 3, padding=1), nn.ReLU(True),
            nn.Conv2d(256, 256, 3, padding=1), nn.ReLU(True), nn.MaxPool2d(3, 2))
        self.pool = nn.AdaptiveAvgPool2d(6)
        self.classifier = nn.Sequential(nn.Dropout(dropout), nn.Linear(256 * 36, 4096), nn.ReLU(True), nn.Dropout(dropout),
                                        nn.Linear(4096, 4096), nn.ReLU(True), nn.Linear(4096, num_classes))

    def forward(self, x):
        return self.classifier(self.pool(self.features(x)).flatten(1))


_VGG = {11: [64, "M", 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        13: [64, 64, "M", 128, 128, "M", 256, 256, "M", 512, 512, "M", 512, 512, "M"],
        16: [64, 64, "M", 128, 128, "M", 256, 256, 256, "M", 512, 512, 512, "M", 512, 512, 512, "M"],
        19: [64, 64, "M", 128, 128, "M", 256, 256, 256, 256, "M", 512, 512, 512, 512, "M", 512, 512, 512, 512, "M"]}


class VGG(nn.Module):
    def __init__(self, depth: int = 16, batch_norm: bool = False, num_classes: int = 1000, width: float = 1.0, hidden: int = 4096):
        super().__init__()
        layers, c = [], 3
        for v in _VGG[depth]:
            if v == "M":
                layers.append(nn.MaxPool2d(2, 2))
            else:
                o = max(8, int(v * width))
                layers += [nn.Conv2d(c, o, 3, padding=1)] + ([nn.BatchNorm2d(o)] if batch_norm else []) + [nn.ReLU(True)]
                c = o
        self.features, self.pool = nn.Sequential(*layers), nn.AdaptiveAvgPool2d(7)
        self.classifier = nn.Sequential(nn.Linear(c * 49, hidden), nn.ReLU(True), nn.Dropout(), nn.Linear(hidden, hidden),
                                        nn.ReLU(True), nn.Dropout(), nn.Linear(hidden, num_classes))

    def forward(self, x):
        return self.classifier(self.pool(self.features(x)).flatten(1))


class _DenseLayer(nn.Module):
    def __init__(self, c, growth, bn_size=4):
        super().__init__()
        self.n1, self.c1 = nn.BatchNorm2d(c), nn.Conv2d(c, bn_size * growth, 1, bias=False)
        self.n2, self.c2 = nn.BatchNorm2d(bn_size * growth), nn.Conv2d(bn_size * growth, growth, 3, padding=1, bias=False)

    def forward(self, x):
        return torch.cat([x, self.c2(F.relu(self.n2(self.c1(F.relu(self.n1(x))))))], 1)


class DenseNet(nn.Module):
    def __init__(self, block_config=(6, 12, 24, 16), growth: int = 32, init_features: int = 64, num_classes: int = 1000):
        super().__init__()
        feats = [nn.Conv2d(3, init_features, 7, 2, 3, bias=False), nn.BatchNorm2d(init_features), nn.ReLU(True), nn.MaxPool2d(3, 2, 1)]
        c = init_features
        for i, n in enumerate(block_config):
            for _ in range(n):
                feats.append(_DenseLayer(c, growth))
                c += growth
            if i + 1 < len(block_config):
                feats += [nn.BatchNorm2d(c), nn.ReLU(True), nn.Conv2d(c, c // 2, 1, bias=False), nn.AvgPool2d(2, 2)]
                c //= 2
        feats.append(nn.BatchNorm2d(c))
        self.features, self.classifier = nn.Sequential(*feats), nn.Linear(c, num_classes)

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(F.relu(self.features(x)), 1).flatten(1))


class _InvertedResidual(nn.Module):
    def __init__(self, c_in, c_out, stride, expand, kernel=3, se_ratio: float = 0.0, act=nn.ReLU6):
        super().__init__()
        hid = c_in * expand
        self.skip = stride == 1 and c_in == c_out
        layers = []
        if expand != 1:
            layers += [nn.Conv2d(c_in, hid, 1, bias=False), nn.BatchNorm2d(hid), act(inplace=True)]
        layers += [nn.Conv2d(hid, hid, kernel, stride, kernel // 2, groups=hid, bias=False), nn.BatchNorm2d(hid), act(inplace=True)]
        self.pre = nn.Sequential(*layers)
        self.se = None
        if se_ratio > 0:
            sq = max(1, int(c_in * se_ratio))
            self.se = nn.Sequential(nn.AdaptiveAvgPool2d(1), nn.Conv2d(hid, sq, 1), nn.SiLU(), nn.Conv2d(sq, hid, 1), nn.Sigmoid())
        self.post = nn.Sequential(nn.Conv2d(hid, c_out, 1, bias=False), nn.BatchNorm2d(c_out))

    def forward(self, x):
        h = self.pre(x)
        if self.se is not None:
            h = h * self.se(h)
        h = self.post(h)
        return x + h if self.skip else h


class MobileNetV2(nn.Module):
    CFG = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]

    def __init__(self, num_classes: int = 1000, width: float = 1.0):
        super().__init__()
        c = int(32 * width)
        layers = [nn.Conv2d(3, c, 3, 2, 1, bias=False), nn.BatchNorm2d(c), nn.ReLU6(True)]
        for t, ch, n, s in self.CFG:
            o = max(8, int(ch * width))
            for i in range(n):
                layers.append(_InvertedResidual(c, o, s if i == 0 else 1, t))
                c = o
        last = max(1280, int(1280 * width)) if width > 1 else int(1280 * max(width, 0.25))
        layers += [nn.Conv2d(c, last, 1, bias=False), nn.BatchNorm2d(last), nn.ReLU6(True)]
        self.features, self.classifier = nn.Sequential(*layers), nn.Sequential(nn.Dropout(0.2), nn.Linear(last, num_classes))

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(self.features(x), 1).flatten(1))


class EfficientNet(nn.Module):
    """EfficientNet-B0 layout; ``width`` / ``depth`` are the compound-scaling multipliers."""
    CFG = [(1, 16, 1, 1, 3), (6, 24, 2, 2, 3), (6, 40, 2, 2, 5), (6, 80, 3, 2, 3), (6, 112, 3, 1, 5), (6, 192, 4, 2, 5), (6, 320, 1, 1, 3)]

    def __init__(self, num_classes: int = 1000, width: float = 1.0, depth: float = 1.0, dropout: float = 0.2):
        super().__init__()
        rnd = lambda ch: max(8, int(ch * width + 4) // 8 * 8)
        c = rnd(32)
        layers = [nn.Conv2d(3, c, 3, 2, 1, bias=False), nn.BatchNorm2d(c), nn.SiLU(True)]
        for t, ch, n, s, k in self.CFG:
            o = rnd(ch)
            for i in range(max(1, math.ceil(n * depth))):
                layers.append(_InvertedResidual(c, o, s if i == 0 else 1, t, k, se_ratio=0.25, act=nn.SiLU))
                c = o
        last = rnd(1280)
        layers += [nn.Conv2d(c, last, 1, bias=False), nn.BatchNorm2d(last), nn.SiLU(True)]
        self.features, self.classifier = nn.Sequential(*layers), nn.Sequential(nn.Dropout(dropout), nn.Linear(last, num_classes))

    def forward(self, x):
        return self.classifier(F.adaptive_avg_pool2d(self.features(x), 1).flatten(1))


class _LayerNorm2d(nn.LayerNorm):
    def forward(self, x):                                    # [B, C, H, W]
        return super().forward(x.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)


class _ConvNeXtBlock(nn.Module):
    def __init__(self, dim, layer_scale=1e-6):
        super().__init__()
        self.dw, self.norm = nn.Conv2d(dim, dim, 7, padding=3, groups=dim), nn.LayerNorm(dim, eps=1e-6)
        self.fc1, self.fc2 = nn.Linear(dim, 4 * dim), nn.Linear(4 * dim, dim)
        self.gamma = nn.Parameter(layer_scale * torch.ones(dim))

    def forward(self, x):
        h = self.dw(x).permute(0, 2, 3, 1)
        h = self.fc2(F.gelu(self.fc1(self.norm(h)))) * self.gamma
        return x + h.permute(0, 3, 1, 2)


class ConvNeXt(nn.Module):
    def __init__(self, depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), num_classes: int = 1000):
        super().__init__()
        layers = [nn.Conv2d(3, dims[0], 4, 4), _LayerNorm2d(dims[0], eps=1e-6)]
        for i, (d, c) in enumerate(zip(depths, dims)):
            if i:
                layers += [_LayerNorm2d(dims[i - 1], eps=1e-6), nn.Conv2d(dims[i - 1], c, 2, 2)]
            layers += [_ConvNeXtBlock(c) for _ in range(d)]
        self.features = nn.Sequential(*layers)
        self.norm, self.head = nn.LayerNorm(dims[-1], eps=1e-6), nn.Linear(dims[-1], num_classes)

    def forward(self, x):
        return self.head(self.norm(self.features(x).mean((-2, -1))))


class _WindowAttention(nn.Module):
    """Multi-head attention inside non-overlapping ``ws x ws`` windows with a learned relative position bias."""

    def __init__(self, dim, heads, ws):
        super().__init__()
        self.h, self.ws = heads, ws
        self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.bias_table = nn.Parameter(torch.zeros((2 * ws - 1) ** 2, heads))
        nn.init.trunc_normal_(self.bias_table, std=0.02)
        co = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)
        rel = (co[:, :, None] - co[:, None, :]).permute(1, 2, 0) + ws - 1
        self.register_buffer("rel_index", rel[..., 0] * (2 * ws - 1) + rel[..., 1], persistent=False)

    def forward(self, x, mask=None):                          # x: [nW*B, ws*ws, C]
        b, n, c = x.shape
        q, k, v = self.qkv(x).view(b, n, 3, self.h, c // self.h).permute(2, 0, 3, 1, 4)
        bias = self.bias_table[self.rel_index.reshape(-1)].view(n, n, -1).permute(2, 0, 1)[None]
        if mask is not None:                                  # mask: [nW, n, n] additive
            bias = bias + mask.repeat(b // mask.shape[0], 1, 1)[:, None]
        out = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype))
        return self.proj(out.transpose(1, 2).reshape(b, n, c))


class _SwinBlock(nn.Module):
    def __init__(self, dim, heads, ws, shift):
        super().__init__()
        self.ws, self.shift = ws, shift
        self.n1, self.attn, self.n2 = nn.LayerNorm(dim), _WindowAttention(dim, heads, ws), nn.LayerNorm(dim)
        self.mlp = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))

    def _windows(self, x):                                    # [B, H, W, C] -> [B*nW, ws*ws, C]
        b, h, w, c = x.shape
        x = x.view(b, h // self.ws, self.ws, w // self.ws, self.ws, c).permute(0, 1, 3, 2, 4, 5)
        return x.reshape(-1, self.ws * self.ws, c)

    def _mask(self, h, w, device):
        img = torch.zeros(1, h, w, 1, device=device)
        cnt = 0
        for hs in (slice(0, -self.ws), slice(-self.ws, -self.shift), slice(-self.shift, None)):
            for wsl in (slice(0, -self.ws), slice(-self.ws, -self.shift), slice(-self.shift, None)):
                img[:, hs, wsl] = cnt
                cnt += 1
        win = self._windows(img).squeeze(-1)
        diff = win[:, None, :] - win[:, :, None]
        return torch.zeros_like(diff).masked_fill(diff != 0, -1e4)

    def forward(self, x):                                     # [B, H, W, C]
        b, h, w, c = x.shape
        y = self.n1(x)
        shift = self.shift if min(h, w) > self.ws else 0
        mask = None
        if shift:
            y = torch.roll(y, (-shift, -shift), (1, 2))
            mask = self._mask(h, w, x.device)
        y = self.attn(self._windows(y), mask)
        y = y.view(b, h // self.ws, w // self.ws, self.ws, self.ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, h, w, c)
        if shift:
            y = torch.roll(y, (shift, shift), (1, 2))
        x = x + y
        return x + self.mlp(self.n2(x))


class SwinTransformer(nn.Module):
    def __init__(self, embed_dim: int = 96, depths=(2, 2, 6, 2), heads=(3, 6, 12, 24), window: int = 7, patch: int = 4,
                 num_classes: int = 1000):
        super().__init__()
        self.patch, self.embed, self.norm0 = patch, nn.Conv2d(3, embed_dim, patch, patch), nn.LayerNorm(embed_dim)
        self.stages, self.merges = nn.ModuleList(), nn.ModuleList()
        dim = embed_dim
        for i, (d, h) in enumerate(zip(depths, heads)):
            self.stages.append(nn.Sequential(*[_SwinBlock(dim, h, window, 0 if j % 2 == 0 else window // 2) for j in range(d)]))
            if i + 1 < len(depths):
                self.merges.append(nn.Sequential(nn.LayerNorm(4 * dim), nn.Linear(4 * dim, 2 * dim, bias=False)))
                dim *= 2
        self.norm, self.head = nn.LayerNorm(dim), nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.norm0(self.embed(x).permute(0, 2, 3, 1))    # [B, H/4, W/4, C]
        for i, stage in enumerate(self.stages):
            x = stage(x)
            if i < len(self.merges):
                x = torch.cat([x[:, 0::2, 0::2], x[:, 1::2, 0::2], x[:, 0::2, 1::2], x[:, 1::2, 1::2]], -1)
                x = self.merges[i](x)
        return self.head(self.norm(x).mean((1, 2)))
