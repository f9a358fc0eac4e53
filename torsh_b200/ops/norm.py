"""LayerNorm / RMSNorm with fused backward (kernels in ``csrc/kernels/norm.cu``).

Reference semantics: LayerNorm eps 1e-5, RMSNorm ``x / sqrt(mean(x²) + eps) * w`` with eps 1e-6
(``crates/torsh-nn/src/layers/normalization/layer_group/mod.rs:491-514``).
"""
from __future__ import annotations

import torch

from .. import _native as nv
from ._dispatch import F, I, P, aligned, call, dtype_code, kernel_ok

_FWD = [P, P, P, P, P, P, I, I, F, I, I, P]
_BWD = [P, P, P, P, P, P, P, P, P, I, I, I, I, P]


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        H = x.shape[-1]
        x2 = aligned(x.reshape(-1, H))
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        w = aligned(weight.to(x.dtype))
        b = aligned(bias.to(x.dtype)) if bias is not None else None
        call("tb_norm_fwd", _FWD, x2.data_ptr(), w.data_ptr(), nv.ptr(b), y.data_ptr(), mean.data_ptr(),
             rstd.data_ptr(), rows, H, float(eps), int(rms), dtype_code(x2), nv.stream_ptr())
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.rms, ctx.has_bias, ctx.shape = rms, bias is not None, x.shape
        ctx.wdtype, ctx.bdtype = weight.dtype, (bias.dtype if bias is not None else None)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = aligned(dy.reshape(rows, H).to(x2.dtype))
        dx = torch.empty_like(x2)
        dgamma = torch.zeros(H, dtype=torch.float32, device=x2.device)
        dbeta = torch.zeros(H, dtype=torch.float32, device=x2.device) if ctx.has_bias else None
        call("tb_norm_bwd", _BWD, dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
             None, dx.data_ptr(), dgamma.data_ptr(), nv.ptr(dbeta), rows, H, int(ctx.rms), dtype_code(x2),
             nv.stream_ptr())
        return (dx.view(ctx.shape), dgamma.to(ctx.wdtype), dbeta.to(ctx.bdtype) if ctx.has_bias else None, None, None)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, eps: float = 1e-5):
    """LayerNorm over the last dimension."""
    if kernel_ok(x, weight, bias) and x.shape[-1] % 8 == 0:
        return _NormFn.apply(x, weight, bias, eps, False)
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """RMSNorm over the last dimension."""
    if kernel_ok(x, weight) and x.shape[-1] % 8 == 0:
        return _NormFn.apply(x, weight, None, eps, True)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * weight.float()).to(x.dtype)
