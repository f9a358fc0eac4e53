"""Quantization (``crates/torsh-quantization``): affine / symmetric INT8 and INT4 schemes (per-tensor, per-channel,
group-wise), binary / ternary, observers (min-max, moving average, histogram percentile), fake-quant with a
straight-through estimator for QAT, post-training quantization of ``nn.Linear`` models, and error metrics."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn


@dataclass
class QParams:
    scale: torch.Tensor
    zero_point: torch.Tensor
    qmin: int
    qmax: int
    axis: int | None = None


def _range(bits: int, symmetric: bool):
    return (-(1 << (bits - 1)) + (1 if symmetric else 0), (1 << (bits - 1)) - 1) if symmetric else (0, (1 << bits) - 1)


def calc_qparams(lo: torch.Tensor, hi: torch.Tensor, bits=8, symmetric=True, axis=None) -> QParams:
    qmin, qmax = _range(bits, symmetric)
    if symmetric:
        scale = torch.maximum(lo.abs(), hi.abs()).clamp(min=1e-12) / qmax
        zp = torch.zeros_like(scale)
    else:
        lo, hi = torch.minimum(lo, torch.zeros_like(lo)), torch.maximum(hi, torch.zeros_like(hi))
        scale = ((hi - lo) / (qmax - qmin)).clamp(min=1e-12)
        zp = (qmin - lo / scale).round().clamp(qmin, qmax)
    return QParams(scale, zp, qmin, qmax, axis)


def _bshape(t, qp):
    if qp.axis is None:
        return qp.scale, qp.zero_point
    shp = [1] * t.dim(); shp[qp.axis] = -1
    return qp.scale.reshape(shp), qp.zero_point.reshape(shp)


def quantize(t: torch.Tensor, qp: QParams) -> torch.Tensor:
    s, z = _bshape(t, qp)
    return (t / s + z).round().clamp(qp.qmin, qp.qmax).to(torch.int8 if qp.qmin < 0 else torch.uint8)


def dequantize(q: torch.Tensor, qp: QParams) -> torch.Tensor:
    s, z = _bshape(q, qp)
    return (q.float() - z) * s


def quantize_per_tensor(t, bits=8, symmetric=True):
    qp = calc_qparams(t.min(), t.max(), bits, symmetric)
    return quantize(t, qp), qp


def quantize_per_channel(t, axis=0, bits=8, symmetric=True):
    red = [d for d in range(t.dim()) if d != axis]
    qp = calc_qparams(t.amin(red), t.amax(red), bits, symmetric, axis)
    return quantize(t, qp), qp


def quantize_groupwise(w: torch.Tensor, group: int = 128, bits: int = 4):
    """Symmetric group-wise quantization along the last dim; returns int8 codes (INT4 values packed two per byte when
    ``bits == 4``) and per-group scales."""
    g = w.reshape(*w.shape[:-1], -1, group)
    qmax = (1 << (bits - 1)) - 1
    scale = g.abs().amax(-1, keepdim=True).clamp(min=1e-12) / qmax
    q = (g / scale).round().clamp(-qmax, qmax).to(torch.int8).reshape(w.shape)
    if bits == 4:
        q = ((q[..., 0::2] & 0xF) | (q[..., 1::2] << 4)).to(torch.int8)
    return q, scale.squeeze(-1)


def dequantize_groupwise(q, scale, group=128, bits=4):
    if bits == 4:
        lo = ((q << 4).to(torch.int8) >> 4)
        hi = q >> 4
        q = torch.stack([lo, hi], -1).reshape(*q.shape[:-1], -1)
    return (q.float().reshape(*q.shape[:-1], -1, group) * scale[..., None]).reshape(q.shape)


def binarize(w): return w.sign() * w.abs().mean()
def ternarize(w, t=0.7):
    thr = t * w.abs().mean()
    m = w.abs() > thr
    return torch.where(m, w.sign() * w[m].abs().mean(), torch.zeros_like(w))


class MinMaxObserver(nn.Module):
    def __init__(self, bits=8, symmetric=True):
        super().__init__()
        self.bits, self.symmetric = bits, symmetric
        self.register_buffer("lo", torch.tensor(float("inf"))); self.register_buffer("hi", torch.tensor(float("-inf")))

    def forward(self, x):
        self.lo, self.hi = torch.minimum(self.lo, x.detach().min()), torch.maximum(self.hi, x.detach().max())
        return x

    def qparams(self): return calc_qparams(self.lo, self.hi, self.bits, self.symmetric)


class MovingAverageObserver(MinMaxObserver):
    def __init__(self, momentum=0.01, **kw):
        super().__init__(**kw); self.momentum = momentum

    def forward(self, x):
        lo, hi = x.detach().min(), x.detach().max()
        if torch.isinf(self.lo):
            self.lo, self.hi = lo, hi
        else:
            self.lo = self.lo + self.momentum * (lo - self.lo); self.hi = self.hi + self.momentum * (hi - self.hi)
        return x


class PercentileObserver(MinMaxObserver):
    def __init__(self, pct=99.99, **kw):
        super().__init__(**kw); self.pct = pct

    def forward(self, x):
        f = x.detach().float().flatten()
        if f.numel() > 1 << 20:
            f = f[torch.randint(0, f.numel(), (1 << 20,), device=f.device)]
        lo, hi = torch.quantile(f, 1 - self.pct / 100), torch.quantile(f, self.pct / 100)
        self.lo, self.hi = torch.minimum(self.lo, lo), torch.maximum(self.hi, hi)
        return x


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zp, qmin, qmax):
        q = (x / scale + zp).round()
        ctx.save_for_backward((q >= qmin) & (q <= qmax))
        return (q.clamp(qmin, qmax) - zp) * scale

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return g * mask, None, None, None, None


class FakeQuantize(nn.Module):
    def __init__(self, observer: MinMaxObserver | None = None):
        super().__init__()
        self.observer = observer or MovingAverageObserver()
        self.enabled, self.observing = True, True

    def forward(self, x):
        if self.observing:
            self.observer(x)
        if not self.enabled:
            return x
        qp = self.observer.qparams()
        return _FakeQuantSTE.apply(x, qp.scale, qp.zero_point, qp.qmin, qp.qmax)


class QuantizedLinear(nn.Module):
    """Weight-only INT8 (per-output-channel) linear; the matmul runs on dequantized bf16/fp32 weights."""

    def __init__(self, lin: nn.Linear, bits=8):
        super().__init__()
        q, qp = quantize_per_channel(lin.weight.detach().float(), 0, bits)
        self.register_buffer("qweight", q); self.register_buffer("scale", qp.scale)
        self.bias = lin.bias

    def forward(self, x):
        return nn.functional.linear(x, (self.qweight.to(x.dtype) * self.scale[:, None].to(x.dtype)), self.bias)


def quantize_model(model: nn.Module, bits=8) -> nn.Module:
    """Post-training weight quantization: every ``nn.Linear`` becomes a :class:`QuantizedLinear` (in place)."""
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear):
            setattr(model, name, QuantizedLinear(child, bits))
        else:
            quantize_model(child, bits)
    return model


def prepare_qat(model: nn.Module) -> nn.Module:
    """Insert activation fake-quant after every Linear / Conv2d (in place)."""
    for name, child in list(model.named_children()):
        if isinstance(child, (nn.Linear, nn.Conv2d)):
            setattr(model, name, nn.Sequential(child, FakeQuantize()))
        else:
            prepare_qat(child)
    return model


def sqnr_db(ref: torch.Tensor, q: torch.Tensor) -> float:
    return (10 * torch.log10(ref.pow(2).mean() / (ref - q).pow(2).mean().clamp(min=1e-30))).item()
