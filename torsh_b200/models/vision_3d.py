"""3-D vision: a volumetric CNN, PointNet (input / feature transform nets with the orthogonality regulariser) and
PointNet++ (farthest-point sampling, ball query grouping, set abstraction). Point clouds are ``[N, P, 3]``.
Reference: crates/torsh-models/src/vision_3d.rs (CNN3D, TransformNet, PointNet, SetAbstractionLayer, PointNetPlusPlus).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn


@dataclass
class CNN3DConfig:
    in_channels: int = 1
    num_classes: int = 10
    widths: tuple = (16, 32, 64)


class CNN3D(nn.Module):
    def __init__(self, cfg: CNN3DConfig | None = None):
        super().__init__()
        self.cfg = cfg or CNN3DConfig()
        layers, cin = [], self.cfg.in_channels
        for w in self.cfg.widths:
            layers += [nn.Conv3d(cin, w, 3, padding=1, bias=False), nn.BatchNorm3d(w), nn.ReLU(inplace=True), nn.MaxPool3d(2)]
            cin = w
        self.features = nn.Sequential(*layers)
        self.fc = nn.Linear(cin, self.cfg.num_classes)

    def forward(self, x):
        return self.fc(self.features(x).mean((2, 3, 4)))


def _shared_mlp(sizes, dims=1):
    conv, bn = (nn.Conv1d, nn.BatchNorm1d) if dims == 1 else (nn.Conv2d, nn.BatchNorm2d)
    layers = []
    for i in range(len(sizes) - 1):
        layers += [conv(sizes[i], sizes[i + 1], 1, bias=False), bn(sizes[i + 1]), nn.ReLU(inplace=True)]
    return nn.Sequential(*layers)


class TransformNet(nn.Module):
    """Predicts a k x k alignment matrix (initialised to the identity) from a point set ``[N, k, P]``."""

    def __init__(self, k: int = 3):
        super().__init__()
        self.k = k
        self.mlp = _shared_mlp([k, 64, 128, 256])
        self.fc = nn.Sequential(nn.Linear(256, 128), nn.ReLU(inplace=True), nn.Linear(128, k * k))
        nn.init.zeros_(self.fc[-1].weight)
        nn.init.zeros_(self.fc[-1].bias)

    def forward(self, x):
        m = self.fc(self.mlp(x).max(-1).values).reshape(-1, self.k, self.k)
        return m + torch.eye(self.k, device=x.device)


def orthogonality_regularizer(m: torch.Tensor) -> torch.Tensor:
    """|| I - M M^T ||_F^2, averaged over the batch."""
    eye = torch.eye(m.shape[-1], device=m.device)
    return ((m @ m.transpose(1, 2) - eye) ** 2).sum((1, 2)).mean()


@dataclass
class PointNetConfig:
    num_classes: int = 10
    feature_transform: bool = True


class PointNet(nn.Module):
    def __init__(self, cfg: PointNetConfig | None = None):
        super().__init__()
        self.cfg = cfg or PointNetConfig()
        self.t_in = TransformNet(3)
        self.mlp1 = _shared_mlp([3, 64])
        self.t_feat = TransformNet(64) if self.cfg.feature_transform else None
        self.mlp2 = _shared_mlp([64, 128, 256])
        self.head = nn.Sequential(nn.Linear(256, 128), nn.ReLU(inplace=True), nn.Dropout(0.3), nn.Linear(128, self.cfg.num_classes))

    def forward(self, pts):
        """``pts`` [N, P, 3] -> (logits, feature transform or None). Invariant to the order of the points."""
        x = pts.transpose(1, 2)
        x = torch.bmm(self.t_in(x), x)
        x = self.mlp1(x)
        tf = None
        if self.t_feat is not None:
            tf = self.t_feat(x)
            x = torch.bmm(tf, x)
        return self.head(self.mlp2(x).max(-1).values), tf

    def loss(self, pts, labels, reg_weight: float = 1e-3):
        logits, tf = self(pts)
        l = nn.functional.cross_entropy(logits, labels)
        return l + (reg_weight * orthogonality_regularizer(tf) if tf is not None else 0.0)


def farthest_point_sampling(pts: torch.Tensor, m: int) -> torch.Tensor:
    """Indices ``[N, m]`` of points chosen greedily to be far apart (the first one is point 0)."""
    n, p, _ = pts.shape
    idx = torch.zeros(n, m, dtype=torch.long, device=pts.device)
    dist = torch.full((n, p), float("inf"), device=pts.device)
    cur = torch.zeros(n, dtype=torch.long, device=pts.device)
    ar = torch.arange(n, device=pts.device)
    for i in range(m):
        idx[:, i] = cur
        d = ((pts - pts[ar, cur][:, None]) ** 2).sum(-1)
        dist = torch.minimum(dist, d)
        cur = dist.argmax(-1)
    return idx


def ball_query(pts: torch.Tensor, centers: torch.Tensor, radius: float, k: int) -> torch.Tensor:
    """For each centre the indices ``[N, M, k]`` of up to k points within ``radius`` (padded with the nearest one)."""
    d = torch.cdist(centers, pts)
    order = d.argsort(-1)[..., :k]
    dk = d.gather(-1, order)
    first = order[..., :1].expand_as(order)
    return torch.where(dk <= radius, order, first)


class SetAbstractionLayer(nn.Module):
    def __init__(self, n_centers: int, radius: float, k: int, in_features: int, mlp: tuple):
        super().__init__()
        self.m, self.radius, self.k = n_centers, radius, k
        self.mlp = _shared_mlp([in_features + 3, *mlp], dims=2)

    def forward(self, xyz, feats):
        """``xyz`` [N, P, 3], ``feats`` [N, P, F] or None -> (centres [N, M, 3], features [N, M, F'])."""
        n = xyz.shape[0]
        ar = torch.arange(n, device=xyz.device)[:, None]
        ci = farthest_point_sampling(xyz, self.m)
        centers = xyz[ar, ci]
        gi = ball_query(xyz, centers, self.radius, self.k)                       # [N, M, k]
        grouped = xyz[ar[:, :, None], gi] - centers[:, :, None]                  # local coordinates
        if feats is not None:
            grouped = torch.cat([grouped, feats[ar[:, :, None], gi]], -1)
        out = self.mlp(grouped.permute(0, 3, 1, 2)).max(-1).values              # [N, F', M]
        return centers, out.transpose(1, 2)


@dataclass
class PointNetPlusPlusConfig:
    num_classes: int = 10
    centers: tuple = (64, 16)
    radii: tuple = (0.3, 0.6)
    k: int = 16


class PointNetPlusPlus(nn.Module):
    def __init__(self, cfg: PointNetPlusPlusConfig | None = None):
        super().__init__()
        self.cfg = cfg or PointNetPlusPlusConfig()
        c = self.cfg
        self.sa1 = SetAbstractionLayer(c.centers[0], c.radii[0], c.k, 0, (32, 64))
        self.sa2 = SetAbstractionLayer(c.centers[1], c.radii[1], c.k, 64, (64, 128))
        self.head = nn.Sequential(nn.Linear(128, 64), nn.ReLU(inplace=True), nn.Dropout(0.3), nn.Linear(64, c.num_classes))

    def forward(self, pts):
        xyz, f = self.sa1(pts, None)
        xyz, f = self.sa2(xyz, f)
        return self.head(f.max(1).values)
