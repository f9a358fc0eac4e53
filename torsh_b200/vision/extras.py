"""Explainability, video, super-resolution and style transfer (``crates/torsh-vision/src``: explainability, video,
models/super_resolution, models/style_transfer)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


# --------------------------------------------------------------------------------------------------- explainability
def saliency(model: nn.Module, x: torch.Tensor, target: torch.Tensor | None = None) -> torch.Tensor:
    """|∂ score / ∂ input| maximised over channels: ``[B, H, W]``. ``target`` defaults to the predicted class."""
    x = x.clone().requires_grad_(True)
    logits = model(x)
    idx = logits.argmax(1) if target is None else target
    logits.gather(1, idx[:, None]).sum().backward()
    return x.grad.abs().amax(1)


class GradCAM:
    """Class-activation map of one convolutional layer: channel weights are the spatial mean of the gradients."""

    def __init__(self, model: nn.Module, layer: nn.Module):
        self.model, self.act, self.grad = model, None, None
        self._h = [layer.register_forward_hook(lambda m, i, o: setattr(self, "act", o)),
                   layer.register_full_backward_hook(lambda m, gi, go: setattr(self, "grad", go[0]))]

    def __call__(self, x: torch.Tensor, target: torch.Tensor | None = None) -> torch.Tensor:
        self.model.zero_grad(set_to_none=True)
        logits = self.model(x)
        idx = logits.argmax(1) if target is None else target
        logits.gather(1, idx[:, None]).sum().backward()
        w = self.grad.mean((2, 3), keepdim=True)
        cam = F.relu((w * self.act).sum(1, keepdim=True))
        cam = F.interpolate(cam, size=x.shape[-2:], mode="bilinear", align_corners=False)[:, 0]
        return cam / cam.flatten(1).amax(1).clamp(min=1e-12)[:, None, None]

    def close(self):
        for h in self._h:
            h.remove()


def integrated_gradients(model: nn.Module, x: torch.Tensor, target: torch.Tensor, baseline: torch.Tensor | None = None,
                         steps: int = 32) -> torch.Tensor:
    """Path integral of the gradients from ``baseline`` (zeros) to ``x``; the attributions sum to the score difference."""
    baseline = torch.zeros_like(x) if baseline is None else baseline
    total = torch.zeros_like(x)
    for a in (torch.arange(steps, dtype=x.dtype) + 0.5) / steps:
        p = (baseline + a * (x - baseline)).requires_grad_(True)
        model(p).gather(1, target[:, None]).sum().backward()
        total += p.grad
    return (x - baseline) * total / steps


# ------------------------------------------------------------------------------------------------------------ video
def sample_frames(video: torch.Tensor, num: int, mode: str = "uniform", generator=None) -> torch.Tensor:
    """``video``: ``[T, C, H, W]`` → ``[num, C, H, W]`` (uniformly spaced, or one random frame per segment)."""
    t = video.shape[0]
    edges = torch.linspace(0, t, num + 1)
    if mode == "uniform":
        idx = ((edges[:-1] + edges[1:]) / 2).long().clamp(max=t - 1)
    else:
        idx = (edges[:-1] + torch.rand(num, generator=generator) * (edges[1:] - edges[:-1])).long().clamp(max=t - 1)
    return video[idx]


def frame_difference(video: torch.Tensor) -> torch.Tensor:
    """Temporal gradient ``[T-1, C, H, W]``: a cheap motion cue."""
    return video[1:] - video[:-1]


class Conv3dClassifier(nn.Module):
    """Small 3-D convolutional clip classifier: ``[B, C, T, H, W]`` → ``[B, num_classes]``."""

    def __init__(self, num_classes: int = 10, width: int = 16):
        super().__init__()
        self.net = nn.Sequential(nn.Conv3d(3, width, 3, padding=1), nn.BatchNorm3d(width), nn.ReLU(True), nn.MaxPool3d((1, 2, 2)),
                                 nn.Conv3d(width, 2 * width, 3, padding=1), nn.BatchNorm3d(2 * width), nn.ReLU(True),
                                 nn.AdaptiveAvgPool3d(1), nn.Flatten(), nn.Linear(2 * width, num_classes))

    def forward(self, x):
        return self.net(x)


# -------------------------------------------------------------------------------------------------- super-resolution
class SRCNN(nn.Module):
    """Three-layer super-resolution network on a bicubically up-sampled input."""

    def __init__(self, scale: int = 2, channels: int = 3):
        super().__init__()
        self.scale = scale
        self.net = nn.Sequential(nn.Conv2d(channels, 64, 9, padding=4), nn.ReLU(True), nn.Conv2d(64, 32, 5, padding=2), nn.ReLU(True),
                                 nn.Conv2d(32, channels, 5, padding=2))

    def forward(self, x):
        up = F.interpolate(x, scale_factor=self.scale, mode="bicubic", align_corners=False)
        return up + self.net(up)


class ESPCN(nn.Module):
    """Sub-pixel network: convolutions at low resolution, then one ``PixelShuffle``."""

    def __init__(self, scale: int = 2, channels: int = 3):
        super().__init__()
        self.net = nn.Sequential(nn.Conv2d(channels, 64, 5, padding=2), nn.Tanh(), nn.Conv2d(64, 32, 3, padding=1), nn.Tanh(),
                                 nn.Conv2d(32, channels * scale * scale, 3, padding=1), nn.PixelShuffle(scale))

    def forward(self, x):
        return self.net(x)


def psnr(pred: torch.Tensor, target: torch.Tensor, max_value: float = 1.0) -> float:
    mse = F.mse_loss(pred.float(), target.float()).item()
    return float("inf") if mse == 0 else 10.0 * torch.log10(torch.tensor(max_value ** 2 / mse)).item()


# ----------------------------------------------------------------------------------------------------- style transfer
def gram_matrix(feat: torch.Tensor) -> torch.Tensor:
    b, c, h, w = feat.shape
    f = feat.reshape(b, c, h * w)
    return f @ f.transpose(1, 2) / (c * h * w)


class StyleTransferLoss(nn.Module):
    """Gatys-style objective over the activations of chosen layers of a feature network: content = MSE of features,
    style = MSE of Gram matrices."""

    def __init__(self, features: nn.Sequential, content_layers=(3,), style_layers=(0, 1, 2, 3), style_weight: float = 1e3):
        super().__init__()
        self.features, self.content_layers, self.style_layers, self.style_weight = features, set(content_layers), set(style_layers), style_weight
        for p in self.features.parameters():
            p.requires_grad_(False)

    def _acts(self, x):
        out = {}
        for i, layer in enumerate(self.features):
            x = layer(x)
            if i in self.content_layers or i in self.style_layers:
                out[i] = x
        return out

    def forward(self, image, content, style):
        a, c, s = self._acts(image), self._acts(content), self._acts(style)
        content_loss = sum(F.mse_loss(a[i], c[i]) for i in self.content_layers)
        style_loss = sum(F.mse_loss(gram_matrix(a[i]), gram_matrix(s[i])) for i in self.style_layers)
        return content_loss + self.style_weight * style_loss, content_loss, style_loss
