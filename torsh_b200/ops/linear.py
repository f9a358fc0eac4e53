"""Linear layers on the tcgen05 GEMM: forward, dgrad and wgrad without transposes.

Weight layouts: ``"nk"`` = ``[out, in]`` (PyTorch) and ``"kn"`` = ``[in, out]`` (the reference's
``Linear`` stores ``[in, out]`` and computes ``x @ W + b``: ``crates/torsh-nn/src/layers/linear.rs:16-62``).
If a weight carries a ``main_grad`` attribute (an fp32 tensor of the same shape, e.g. a view into a
flat gradient buffer), wgrad accumulates into it with split-K atomics inside the GEMM epilogue and
autograd receives ``None`` for that weight; bias gradients behave the same way.
"""
from __future__ import annotations

import os

import torch

from . import elementwise as ew
from ._dispatch import kernel_ok
from .gemm import gemm


# TORSH_WGRAD_STREAM_K=0 goes back to uniform K-splits for the weight-gradient GEMMs
_STREAM_K = os.environ.get("TORSH_WGRAD_STREAM_K", "1") != "0"


def _wgrad_plan(m_out: int, n_out: int, k: int) -> tuple[int, int]:
    """(tile width, split-K factor) for a weight-gradient GEMM: wide tiles when the output is wide
    enough, and enough K-splits that the work units fill the 148 SMs about twice."""
    bn = 256 if n_out >= 256 else 128
    tiles = ((m_out + 127) // 128) * ((n_out + bn - 1) // bn)
    kb = (k + 63) // 64
    # measured on B200: the best split keeps tiles x splits within two waves of the 148 SMs and leaves every split
    # at least 32 K-blocks (K = 8192: 32 tiles -> 4, 96 -> 3, 128 -> 2); deeper splits only add fp32 atomic traffic
    sk = max(1, min(296 // max(tiles, 1), kb // 32))
    # stream-K (every CTA gets the same number of K-blocks) where uniform splits leave the last wave of the 148 SMs
    # more than a tenth empty and the tiles fit in one wave. Measured at K = 8192: 128 tiles 75.7 -> 71.7 us,
    # 32 tiles 34.8 -> 32.9 us; 96 tiles x 3 splits already fill 288 of 296 slots (57.4 vs 58.4 us), and with many tiles
    # per CTA (LM head, 1572 tiles) contiguous ranges lose the L2 reuse between neighbouring CTAs (635 -> 818 us).
    units = tiles * sk
    fill = units / (((units + 147) // 148) * 148)
    if _STREAM_K and kb >= 16 and tiles <= 148 and fill < 0.9:
        return bn, -1
    return bn, sk


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor, layout: str):
    """dW for y = x Wᵀ (nk) or y = x W (kn). Returns a grad tensor, or None after accumulating into main_grad."""
    a, b = (dy2, x2) if layout == "nk" else (x2, dy2)
    m_out, n_out, k = a.shape[1], b.shape[1], a.shape[0]
    bn, sk = _wgrad_plan(m_out, n_out, k)
    mg = getattr(weight, "main_grad", None)
    if mg is not None:
        gemm(a, b, a_major=1, b_major=1, out=mg, atomic=True, split_k=sk, bn=bn)
        return None
    if sk != 1:
        g = torch.zeros(m_out, n_out, dtype=torch.float32, device=a.device)
        gemm(a, b, a_major=1, b_major=1, out=g, atomic=True, split_k=sk, bn=bn)
        return g.to(weight.dtype)
    return gemm(a, b, a_major=1, b_major=1, bn=bn)


def _bgrad(dy2: torch.Tensor, bias: torch.Tensor):
    mg = getattr(bias, "main_grad", None)
    if mg is not None:
        ew.colsum_into(dy2, mg)
        return None
    g = torch.zeros(bias.shape, dtype=torch.float32, device=dy2.device)
    ew.colsum_into(dy2, g)
    return g.to(bias.dtype)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layout, gelu, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        N = weight.shape[0] if layout == "nk" else weight.shape[1]
        res2 = residual.reshape(-1, N) if residual is not None else None
        pre = torch.empty(x2.shape[0], N, dtype=x.dtype, device=x.device) if gelu else None
        y = gemm(x2, weight, b_major=0 if layout == "nk" else 1, bias=bias, gelu=gelu, residual=res2, preact_out=pre)
        ctx.save_for_backward(x2, weight, pre)
        ctx.bias, ctx.layout, ctx.has_res, ctx.xshape = bias, layout, residual is not None, x.shape
        return y.view(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, pre = ctx.saved_tensors
        layout, bias = ctx.layout, ctx.bias
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        if pre is not None:
            dy2 = ew.binary_raw("gelu_bwd", dy2, pre)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_major=1 if layout == "nk" else 0).view(ctx.xshape)
        dw = _wgrad(dy2, x2, weight, layout) if ctx.needs_input_grad[1] else None
        db = _bgrad(dy2, bias) if bias is not None and ctx.needs_input_grad[2] else None
        return dx, dw, db, None, None, dres


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, *, layout: str = "nk",
           gelu: bool = False, residual: torch.Tensor | None = None) -> torch.Tensor:
    """``y = act(x Wᵀ + b) + residual`` in one GEMM launch (bias / tanh-GELU / residual in the epilogue)."""
    K = x.shape[-1]
    N = weight.shape[0] if layout == "nk" else weight.shape[1]
    if (kernel_ok(x, weight, bias, residual) and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and K % 8 == 0 and N % 8 == 0 and weight.is_contiguous()):
        return _LinearFn.apply(x, weight, bias, layout, gelu, residual)
    w = weight if layout == "nk" else weight.t()
    y = torch.nn.functional.linear(x, w.to(x.dtype), None if bias is None else bias.to(x.dtype))
    if gelu:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if residual is not None:
        y = y + residual
    return y


class _MlpFn(torch.autograd.Function):
    """``y = gelu(x W1ᵀ + b1) W2ᵀ + b2 + residual`` with the GELU derivative fused into the fc2 dgrad epilogue."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M, Fh = x2.shape[0], w1.shape[0]
        u = torch.empty(M, Fh, dtype=x.dtype, device=x.device)
        h = gemm(x2, w1, bias=b1, gelu=True, preact_out=u)
        res2 = residual.reshape(M, -1) if residual is not None else None
        y = gemm(h, w2, bias=b2, residual=res2)
        ctx.save_for_backward(x2, w1, w2, u, h)
        ctx.b1, ctx.b2, ctx.has_res, ctx.xshape = b1, b2, residual is not None, x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, u, h = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        du = gemm(dy2, w2, b_major=1, dgelu_aux=u)          # (dy W2) * gelu'(u)
        dw2 = _wgrad(dy2, h, w2, "nk")
        db2 = _bgrad(dy2, ctx.b2) if ctx.b2 is not None else None
        dx = gemm(du, w1, b_major=1).view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw1 = _wgrad(du, x2, w1, "nk")
        db1 = _bgrad(du, ctx.b1) if ctx.b1 is not None else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    """Transformer MLP block (weights in ``[out, in]`` layout) with optional fused residual add."""
    if kernel_ok(x, w1, b1, w2, b2, residual) and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16:
        return _MlpFn.apply(x, w1, b1, w2, b2, residual)
    h = torch.nn.functional.gelu(torch.nn.functional.linear(x, w1.to(x.dtype), b1), approximate="tanh")
    y = torch.nn.functional.linear(h, w2.to(x.dtype), b2)
    return y if residual is None else y + residual
