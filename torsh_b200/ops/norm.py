"""LayerNorm / RMSNorm with fused backward (kernels in ``csrc/kernels/norm.cu``).

Reference semantics: LayerNorm eps 1e-5, RMSNorm ``x / sqrt(mean(x²) + eps) * w`` with eps 1e-6
(``crates/torsh-nn/src/layers/normalization/layer_group/mod.rs:491-514``).
"""
from __future__ import annotations

import torch

from .. import _native as nv
from ._dispatch import F, I, P, aligned, call, dtype_code, kernel_ok

_FWD = [P, P, P, P, P, P, I, I, F, I, I, P]
_BWD = [P, P, P, P, P, P, P, P, P, P, I, I, I, I, P]


_ws_cache: dict = {}


def _workspace_elems(rows: int, H: int) -> int:
    key = (rows, H, torch.cuda.current_device())
    n = _ws_cache.get(key)
    if n is None:
        import ctypes
        f = nv.require_cuda().tb_norm_bwd_workspace
        f.restype, f.argtypes = ctypes.c_long, [ctypes.c_int, ctypes.c_int]
        nv.stream_ptr()  # makes the library's device current
        n = _ws_cache[key] = int(f(rows, H))
    return n


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
        ctx.main_grads = (getattr(weight, "main_grad", None), getattr(bias, "main_grad", None) if bias is not None else None)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = aligned(dy.reshape(rows, H).to(x2.dtype))
        dx = torch.empty_like(x2)
        # gradients of weight / bias accumulate straight into fp32 `main_grad` buffers when the
        # parameters carry them (flat mixed-precision storage); autograd then receives None
        wmg, bmg = ctx.main_grads
        dgamma = wmg.view(-1) if wmg is not None else torch.zeros(H, dtype=torch.float32, device=x2.device)
        dbeta = None
        if ctx.has_bias:
            dbeta = bmg.view(-1) if bmg is not None else torch.zeros(H, dtype=torch.float32, device=x2.device)
        ws = torch.empty(_workspace_elems(rows, H), dtype=torch.float32, device=x2.device)
        call("tb_norm_bwd", _BWD, dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
             None, dx.data_ptr(), dgamma.data_ptr(), nv.ptr(dbeta), ws.data_ptr(), rows, H, int(ctx.rms),
             dtype_code(x2), nv.stream_ptr())
        nv.launch_count += 1
        gw = None if wmg is not None else dgamma.to(ctx.wdtype)
        gb = None if (not ctx.has_bias or bmg is not None) else dbeta.to(ctx.bdtype)
        return dx.view(ctx.shape), gw, gb, None, None


class _NormForkFn(torch.autograd.Function):
    """``(norm(x), x)``: the normalised branch plus the untouched residual stream as two outputs of one
    node, so that the backward adds the residual-stream gradient inside the norm-backward kernel
    instead of in a separate elementwise add."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        y = _NormFn.forward(ctx, x, weight, bias, eps, rms)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = aligned(dy.reshape(rows, H).to(x2.dtype))
        dr2 = aligned(dres.reshape(rows, H).to(x2.dtype)) if dres is not None else None
        dx = torch.empty_like(x2)
        wmg, bmg = ctx.main_grads
        dgamma = wmg.view(-1) if wmg is not None else torch.zeros(H, dtype=torch.float32, device=x2.device)
        dbeta = None
        if ctx.has_bias:
            dbeta = bmg.view(-1) if bmg is not None else torch.zeros(H, dtype=torch.float32, device=x2.device)
        ws = torch.empty(_workspace_elems(rows, H), dtype=torch.float32, device=x2.device)
        call("tb_norm_bwd", _BWD, dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
             nv.ptr(dr2), dx.data_ptr(), dgamma.data_ptr(), nv.ptr(dbeta), ws.data_ptr(), rows, H, int(ctx.rms),
             dtype_code(x2), nv.stream_ptr())
        nv.launch_count += 1
        gw = None if wmg is not None else dgamma.to(ctx.wdtype)
        gb = None if (not ctx.has_bias or bmg is not None) else dbeta.to(ctx.bdtype)
        return dx.view(ctx.shape), gw, gb, None, None


def layer_norm_fork(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, eps: float = 1e-5):
    """Returns ``(layer_norm(x), x)`` for pre-norm residual blocks (see :class:`_NormForkFn`)."""
    if kernel_ok(x, weight, bias) and x.shape[-1] % 8 == 0 and x.requires_grad and torch.is_grad_enabled():
        return _NormForkFn.apply(x, weight, bias, eps, False)
    return layer_norm(x, weight, bias, eps), x


def rms_norm_fork(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Returns ``(rms_norm(x), x)`` for pre-norm residual blocks."""
    if kernel_ok(x, weight) and x.shape[-1] % 8 == 0 and x.requires_grad and torch.is_grad_enabled():
        return _NormForkFn.apply(x, weight, None, eps, True)
    return rms_norm(x, weight, eps), x


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
