"""Video models: 3-D ResNet, SlowFast (two pathways with lateral connections) and a video transformer with tubelet
embedding and divided space / time attention. Input ``[N, C, T, H, W]``.
Reference: crates/torsh-models/src/video.rs (ResNet3D, SlowFast, VideoTransformer).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn


class BasicBlock3D(nn.Module):
    def __init__(self, cin: int, cout: int, stride: int = 1, temporal_kernel: int = 3):
        super().__init__()
        k, p = (temporal_kernel, 3, 3), (temporal_kernel // 2, 1, 1)
        self.conv1 = nn.Conv3d(cin, cout, k, (1, stride, stride), p, bias=False)
        self.bn1 = nn.BatchNorm3d(cout)
        self.conv2 = nn.Conv3d(cout, cout, k, 1, p, bias=False)
        self.bn2 = nn.BatchNorm3d(cout)
        self.down = None
        if stride != 1 or cin != cout:
            self.down = nn.Sequential(nn.Conv3d(cin, cout, 1, (1, stride, stride), bias=False), nn.BatchNorm3d(cout))

    def forward(self, x):
        y = torch.relu(self.bn1(self.conv1(x)))
        y = self.bn2(self.conv2(y))
        return torch.relu(y + (x if self.down is None else self.down(x)))


@dataclass
class ResNet3DConfig:
    in_channels: int = 3
    num_classes: int = 400
    widths: tuple = (64, 128, 256, 512)
    depths: tuple = (2, 2, 2, 2)
    temporal_kernel: int = 3


class ResNet3D(nn.Module):
    def __init__(self, cfg: ResNet3DConfig | None = None):
        super().__init__()
        self.cfg = cfg or ResNet3DConfig()
        c = self.cfg
        self.stem = nn.Sequential(nn.Conv3d(c.in_channels, c.widths[0], (3, 7, 7), (1, 2, 2), (1, 3, 3), bias=False),
                                  nn.BatchNorm3d(c.widths[0]), nn.ReLU(inplace=True), nn.MaxPool3d((1, 3, 3), (1, 2, 2), (0, 1, 1)))
        blocks, cin = [], c.widths[0]
        for i, (w, d) in enumerate(zip(c.widths, c.depths)):
            for j in range(d):
                blocks.append(BasicBlock3D(cin, w, 2 if (j == 0 and i > 0) else 1, c.temporal_kernel))
                cin = w
        self.layers = nn.Sequential(*blocks)
        self.fc = nn.Linear(cin, c.num_classes)

    def features(self, x):
        return self.layers(self.stem(x))

    def forward(self, x):
        return self.fc(self.features(x).mean((2, 3, 4)))


@dataclass
class SlowFastConfig:
    num_classes: int = 400
    alpha: int = 4            # the fast pathway sees alpha times more frames
    beta: float = 0.125       # ... with beta times the channels
    widths: tuple = (64, 128, 256)


class SlowFast(nn.Module):
    def __init__(self, cfg: SlowFastConfig | None = None):
        super().__init__()
        self.cfg = cfg or SlowFastConfig()
        c = self.cfg
        fw = [max(int(w * c.beta), 4) for w in c.widths]
        self.slow_stem = nn.Sequential(nn.Conv3d(3, c.widths[0], (1, 7, 7), (1, 2, 2), (0, 3, 3), bias=False), nn.BatchNorm3d(c.widths[0]), nn.ReLU(inplace=True))
        self.fast_stem = nn.Sequential(nn.Conv3d(3, fw[0], (5, 7, 7), (1, 2, 2), (2, 3, 3), bias=False), nn.BatchNorm3d(fw[0]), nn.ReLU(inplace=True))
        self.slow, self.fast, self.lateral = nn.ModuleList(), nn.ModuleList(), nn.ModuleList()
        s_in, f_in = c.widths[0], fw[0]
        for i, (sw, fwid) in enumerate(zip(c.widths, fw)):
            # the lateral connection squeezes the fast pathway's alpha-fold frame rate into channels of the slow one
            self.lateral.append(nn.Conv3d(f_in, 2 * f_in, (5, 1, 1), (c.alpha, 1, 1), (2, 0, 0), bias=False))
            self.slow.append(BasicBlock3D(s_in + 2 * f_in, sw, 2 if i else 1, temporal_kernel=1 if i < 2 else 3))
            self.fast.append(BasicBlock3D(f_in, fwid, 2 if i else 1, temporal_kernel=3))
            s_in, f_in = sw, fwid
        self.fc = nn.Linear(s_in + f_in, c.num_classes)

    def forward(self, x):
        """``x`` [N, 3, T, H, W] with T a multiple of alpha: the slow pathway takes every alpha-th frame."""
        slow, fast = self.slow_stem(x[:, :, ::self.cfg.alpha]), self.fast_stem(x)
        for lat, sb, fb in zip(self.lateral, self.slow, self.fast):
            slow = sb(torch.cat([slow, lat(fast)], 1))
            fast = fb(fast)
        return self.fc(torch.cat([slow.mean((2, 3, 4)), fast.mean((2, 3, 4))], 1))


@dataclass
class VideoTransformerConfig:
    num_classes: int = 400
    frames: int = 8
    image_size: int = 64
    tubelet: tuple = (2, 16, 16)
    dim: int = 128
    depth: int = 2
    heads: int = 4
    mlp_ratio: float = 4.0


class VideoTransformerBlock(nn.Module):
    """Divided attention: over time for every spatial position, then over space for every frame, then the MLP."""

    def __init__(self, dim: int, heads: int, mlp_ratio: float):
        super().__init__()
        self.n1, self.n2, self.n3 = nn.LayerNorm(dim), nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.time_attn = nn.MultiheadAttention(dim, heads, batch_first=True)
        self.space_attn = nn.MultiheadAttention(dim, heads, batch_first=True)
        self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), nn.GELU(), nn.Linear(int(dim * mlp_ratio), dim))

    def forward(self, x):                       # x [N, T, S, D]
        n, t, s, d = x.shape
        y = self.n1(x).permute(0, 2, 1, 3).reshape(n * s, t, d)
        x = x + self.time_attn(y, y, y, need_weights=False)[0].reshape(n, s, t, d).permute(0, 2, 1, 3)
        y = self.n2(x).reshape(n * t, s, d)
        x = x + self.space_attn(y, y, y, need_weights=False)[0].reshape(n, t, s, d)
        return x + self.mlp(self.n3(x))


class VideoTransformer(nn.Module):
    def __init__(self, cfg: VideoTransformerConfig | None = None):
        super().__init__()
        self.cfg = cfg or VideoTransformerConfig()
        c = self.cfg
        self.embed = nn.Conv3d(3, c.dim, c.tubelet, c.tubelet)
        self.t, self.s = c.frames // c.tubelet[0], (c.image_size // c.tubelet[1]) * (c.image_size // c.tubelet[2])
        self.pos_t = nn.Parameter(torch.zeros(1, self.t, 1, c.dim))
        self.pos_s = nn.Parameter(torch.zeros(1, 1, self.s, c.dim))
        self.blocks = nn.ModuleList(VideoTransformerBlock(c.dim, c.heads, c.mlp_ratio) for _ in range(c.depth))
        self.norm, self.head = nn.LayerNorm(c.dim), nn.Linear(c.dim, c.num_classes)
        nn.init.trunc_normal_(self.pos_t, std=0.02)
        nn.init.trunc_normal_(self.pos_s, std=0.02)

    def forward(self, x):
        y = self.embed(x)                                           # [N, D, T', H', W']
        n, d, t, h, w = y.shape
        y = y.reshape(n, d, t, h * w).permute(0, 2, 3, 1) + self.pos_t + self.pos_s
        for b in self.blocks:
            y = b(y)
        return self.head(self.norm(y).mean((1, 2)))
