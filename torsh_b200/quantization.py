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


def _int4_kernel_ok(t: torch.Tensor, group: int) -> bool:
    return (t.is_cuda and t.dtype in (torch.bfloat16, torch.float32) and group in (32, 64, 128, 256)
            and t.shape[-1] % group == 0)


def quantize_groupwise(w: torch.Tensor, group: int = 128, bits: int = 4):
    """Symmetric group-wise quantization along the last dim; returns int8 codes (INT4 values packed two per byte when
    ``bits == 4``) and per-group scales. On a GPU the INT4 case is one kernel (`tb_quantize_int4_group`)."""
    if bits == 4 and _int4_kernel_ok(w, group):
        from . import _native as nv
        from .ops import _dispatch as dp
        wc = w.contiguous()
        rows = wc.numel() // wc.shape[-1]
        q = torch.empty(*wc.shape[:-1], wc.shape[-1] // 2, dtype=torch.int8, device=w.device)
        scale = torch.empty(*wc.shape[:-1], wc.shape[-1] // group, dtype=torch.float32, device=w.device)
        dp.call("tb_quantize_int4_group", [dp.P, dp.I, dp.P, dp.P, dp.L, dp.I, dp.I, dp.P], wc.data_ptr(),
                0 if wc.dtype == torch.bfloat16 else 1, q.data_ptr(), scale.data_ptr(), rows, wc.shape[-1], group, nv.stream_ptr())
        return q, scale
    g = w.reshape(*w.shape[:-1], -1, group)
    qmax = (1 << (bits - 1)) - 1
    scale = g.abs().amax(-1, keepdim=True).clamp(min=1e-12) / qmax
    q = (g / scale).round().clamp(-qmax, qmax).to(torch.int8).reshape(w.shape)
    if bits == 4:
        q = ((q[..., 0::2] & 0xF) | (q[..., 1::2] << 4)).to(torch.int8)
    return q, scale.squeeze(-1)


def dequantize_groupwise(q, scale, group=128, bits=4, dtype: torch.dtype = torch.float32):
    if bits == 4 and q.is_cuda and group in (32, 64, 128, 256) and dtype in (torch.bfloat16, torch.float32):
        from . import _native as nv
        from .ops import _dispatch as dp
        qc, sc = q.contiguous(), scale.contiguous().float()
        cols = qc.shape[-1] * 2
        rows = qc.numel() // qc.shape[-1]
        out = torch.empty(*qc.shape[:-1], cols, dtype=dtype, device=q.device)
        dp.call("tb_dequantize_int4_group", [dp.P, dp.P, dp.P, dp.I, dp.L, dp.I, dp.I, dp.P], qc.data_ptr(), sc.data_ptr(),
                out.data_ptr(), 0 if dtype == torch.bfloat16 else 1, rows, cols, group, nv.stream_ptr())
        return out
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


class Int4Linear(nn.Module):
    """Weight-only INT4 linear layer: group-wise symmetric codes, two per byte, with fp32 scales (4.25 bits per weight
    at group 128). Up to 8 activation rows go through the fused kernel that reads the packed weights once and never
    materialises them (`tb_int4_linear`, the decoding case); larger batches dequantise to bf16 and use the GEMM."""

    def __init__(self, lin: nn.Linear, group: int = 128):
        super().__init__()
        self.in_features, self.out_features, self.group = lin.in_features, lin.out_features, group
        q, s = quantize_groupwise(lin.weight.detach(), group, 4)
        self.register_buffer("qweight", q.contiguous())
        self.register_buffer("scales", s.contiguous().float())
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def dequantized_weight(self, dtype=torch.float32) -> torch.Tensor:
        return dequantize_groupwise(self.qweight, self.scales, self.group, 4, dtype=dtype) if self.qweight.is_cuda \
            else dequantize_groupwise(self.qweight, self.scales, self.group, 4).to(dtype)

    def forward(self, x):
        x2 = x.reshape(-1, self.in_features)
        if x2.is_cuda and x2.shape[0] <= 8 and self.in_features % 8 == 0:
            from . import _native as nv
            from .ops import _dispatch as dp
            xb = x2.to(torch.bfloat16).contiguous()
            y = torch.empty(x2.shape[0], self.out_features, dtype=torch.bfloat16, device=x.device)
            b = None if self.bias is None else self.bias.to(torch.bfloat16).contiguous()
            dp.call("tb_int4_linear", [dp.P, dp.P, dp.P, dp.P, dp.P, dp.I, dp.I, dp.I, dp.I, dp.P], xb.data_ptr(),
                    self.qweight.data_ptr(), self.scales.data_ptr(), 0 if b is None else b.data_ptr(), y.data_ptr(),
                    x2.shape[0], self.out_features, self.in_features, self.group, nv.stream_ptr())
            return y.to(x.dtype).reshape(*x.shape[:-1], self.out_features)
        w = self.dequantized_weight(x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.float32)
        return torch.nn.functional.linear(x, w.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


def quantize_int8_rowwise(x: torch.Tensor):
    """Per-row symmetric INT8: (codes int8 [rows, cols], scale fp32 [rows]); one kernel on a GPU."""
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    if x2.is_cuda and x2.dtype in (torch.bfloat16, torch.float32):
        from . import _native as nv
        from .ops import _dispatch as dp
        q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
        s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        dp.call("tb_quantize_int8_row", [dp.P, dp.I, dp.P, dp.P, dp.I, dp.I, dp.P], x2.data_ptr(),
                0 if x2.dtype == torch.bfloat16 else 1, q.data_ptr(), s.data_ptr(), x2.shape[0], x2.shape[1], nv.stream_ptr())
        return q.reshape(x.shape), s.reshape(x.shape[:-1])
    s = x2.float().abs().amax(-1).clamp(min=1e-12) / 127
    q = (x2.float() / s[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q.reshape(x.shape), s.reshape(x.shape[:-1])


def dequantize_int8_rowwise(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    q2 = q.reshape(-1, q.shape[-1]).contiguous()
    if q2.is_cuda and dtype in (torch.bfloat16, torch.float32):
        from . import _native as nv
        from .ops import _dispatch as dp
        out = torch.empty(q2.shape, dtype=dtype, device=q.device)
        sc = scale.reshape(-1).contiguous().float()
        dp.call("tb_dequantize_int8_row", [dp.P, dp.P, dp.P, dp.I, dp.I, dp.I, dp.P], q2.data_ptr(), sc.data_ptr(), out.data_ptr(),
                0 if dtype == torch.bfloat16 else 1, q2.shape[0], q2.shape[1], nv.stream_ptr())
        return out.reshape(q.shape)
    return (q2.float() * scale.reshape(-1, 1).float()).to(dtype).reshape(q.shape)


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
