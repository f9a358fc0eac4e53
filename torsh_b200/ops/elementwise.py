"""Elementwise, activation, reduction, embedding and rotary ops.

CUDA tensors (bf16 / fp32) run the kernels in ``csrc/kernels/elementwise.cu`` and
``csrc/kernels/reduce_embed_rope.cu``; anything else uses the same maths in PyTorch. The op list
covers the reference's GPU kernels (unary relu/sigmoid/tanh/exp/log/sqrt/abs/neg, binary
add/sub/mul/div/max/min, axis sum/max/min/mean: ``crates/torsh-tensor/src/cuda_backend/ptx_ops.rs``).
"""
from __future__ import annotations

import math

import torch

from .. import _native as nv
from ._dispatch import F, I, L, P, aligned, call, dtype_code, kernel_ok

UNARY = {"relu": 0, "sigmoid": 1, "tanh": 2, "exp": 3, "log": 4, "sqrt": 5, "abs": 6, "neg": 7, "gelu_tanh": 8,
         "silu": 9, "gelu_erf": 10, "rsqrt": 11, "square": 12, "scale": 13}
BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "relu_bwd": 6, "gelu_bwd": 7, "silu_bwd": 8,
          "sigmoid_bwd": 9, "tanh_bwd": 10}
REDUCE = {"sum": 0, "max": 1, "min": 2, "mean": 3}

_TORCH_UNARY = {
    "relu": torch.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "exp": torch.exp, "log": torch.log,
    "sqrt": torch.sqrt, "abs": torch.abs, "neg": torch.neg, "silu": torch.nn.functional.silu,
    "gelu_tanh": lambda x: torch.nn.functional.gelu(x, approximate="tanh"),
    "gelu_erf": torch.nn.functional.gelu, "rsqrt": torch.rsqrt, "square": torch.square,
}
_TORCH_BINARY = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "max": torch.maximum,
                 "min": torch.minimum}


def unary_raw(op: str, x: torch.Tensor, alpha: float = 1.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Kernel call without autograd bookkeeping."""
    x = aligned(x)
    y = torch.empty_like(x) if out is None else out
    call("tb_unary", [P, P, L, I, F, I, P], x.data_ptr(), y.data_ptr(), x.numel(), UNARY[op], float(alpha),
         dtype_code(x), nv.stream_ptr())
    return y


def binary_raw(op: str, a: torch.Tensor, b, out: torch.Tensor | None = None) -> torch.Tensor:
    a = aligned(a)
    scalar = not isinstance(b, torch.Tensor)
    if not scalar:
        b = aligned(b.to(a.dtype))
        assert b.shape == a.shape
    y = torch.empty_like(a) if out is None else out
    call("tb_binary", [P, P, P, L, I, I, F, I, P], a.data_ptr(), None if scalar else b.data_ptr(), y.data_ptr(),
         a.numel(), BINARY[op], int(scalar), float(b) if scalar else 0.0, dtype_code(a), nv.stream_ptr())
    return y


_BWD_OF = {"relu": ("relu_bwd", "x"), "gelu_tanh": ("gelu_bwd", "x"), "silu": ("silu_bwd", "x"),
           "sigmoid": ("sigmoid_bwd", "y"), "tanh": ("tanh_bwd", "y")}


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op):
        y = unary_raw(op, x)
        ctx.op = op
        ctx.save_for_backward(x if _BWD_OF[op][1] == "x" else y)
        return y

    @staticmethod
    def backward(ctx, dy):
        (saved,) = ctx.saved_tensors
        return binary_raw(_BWD_OF[ctx.op][0], dy.to(saved.dtype), saved), None


def _act(op: str, x: torch.Tensor) -> torch.Tensor:
    if kernel_ok(x):
        if x.requires_grad and torch.is_grad_enabled():
            return _ActFn.apply(x, op)
        return unary_raw(op, x)
    return _TORCH_UNARY[op](x)


def relu(x): return _act("relu", x)
def sigmoid(x): return _act("sigmoid", x)
def tanh(x): return _act("tanh", x)
def silu(x): return _act("silu", x)


def gelu(x: torch.Tensor, approximate: str = "tanh") -> torch.Tensor:
    """GELU. ``tanh`` is the GPT-2 form; ``none`` is the exact erf form.

    The reference's ``approximate=false`` branch substitutes ``tanh(x/√2)`` for erf
    (``crates/torsh-nn/src/layers/activation/modern.rs:124-152``); the true erf is used here.
    """
    if approximate == "tanh":
        return _act("gelu_tanh", x)
    return torch.nn.functional.gelu(x)


def unary(op: str, x: torch.Tensor) -> torch.Tensor:
    """Non-differentiable device-resident unary op (exp, log, sqrt, abs, neg, ...)."""
    if kernel_ok(x) and not (x.requires_grad and torch.is_grad_enabled()):
        return unary_raw(op, x)
    return _TORCH_UNARY[op](x)


def binary(op: str, a: torch.Tensor, b) -> torch.Tensor:
    same = isinstance(b, torch.Tensor) and b.shape == a.shape and b.dtype == a.dtype
    needs_grad = torch.is_grad_enabled() and (a.requires_grad or (isinstance(b, torch.Tensor) and b.requires_grad))
    if kernel_ok(a) and not needs_grad and (same or not isinstance(b, torch.Tensor)):
        return binary_raw(op, a, b)
    return _TORCH_BINARY[op](a, b if isinstance(b, torch.Tensor) else torch.tensor(b, dtype=a.dtype, device=a.device))


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        half = x.shape[-1] // 2
        x2 = aligned(x.reshape(-1, 2 * half))
        y = torch.empty(x2.shape[0], half, dtype=x.dtype, device=x.device)
        call("tb_swiglu_fwd", [P, P, L, I, I, P], x2.data_ptr(), y.data_ptr(), x2.shape[0], half, dtype_code(x2),
             nv.stream_ptr())
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return y.view(*x.shape[:-1], half)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        half = x2.shape[1] // 2
        dy2 = aligned(dy.reshape(-1, half).to(x2.dtype))
        dx = torch.empty_like(x2)
        call("tb_swiglu_bwd", [P, P, P, L, I, I, P], dy2.data_ptr(), x2.data_ptr(), dx.data_ptr(), x2.shape[0], half,
             dtype_code(x2), nv.stream_ptr())
        return dx.view(ctx.shape)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    """``a * silu(b)`` with ``(a, b)`` the two halves of the last dim — the gate is the SECOND half
    (``crates/torsh-nn/src/layers/activation/gated.rs:536-608``)."""
    half = x.shape[-1] // 2
    if kernel_ok(x) and half % 8 == 0:
        return _SwiGLUFn.apply(x)
    a, b = x[..., :half], x[..., half:]
    return a * torch.nn.functional.silu(b)


def reduce(op: str, x: torch.Tensor, dim: int, keepdim: bool = False) -> torch.Tensor:
    """sum / max / min / mean along one axis, viewing the tensor as [outer, axis, inner]."""
    dim = dim % x.dim()
    if kernel_ok(x) and not (x.requires_grad and torch.is_grad_enabled()) and x.numel() > 0:
        xc = aligned(x)
        outer = math.prod(x.shape[:dim])
        axis = x.shape[dim]
        inner = math.prod(x.shape[dim + 1:])
        if inner == 1 or outer <= 65535:
            shape = list(x.shape)
            shape[dim] = 1
            y = torch.empty(shape, dtype=x.dtype, device=x.device)
            call("tb_reduce_axis", [P, P, L, L, L, I, I, P], xc.data_ptr(), y.data_ptr(), outer, axis, inner,
                 REDUCE[op], dtype_code(xc), nv.stream_ptr())
            return y if keepdim else y.squeeze(dim)
    if op == "sum":
        return x.sum(dim, keepdim)
    if op == "mean":
        return x.mean(dim, keepdim)
    return (x.max(dim, keepdim) if op == "max" else x.min(dim, keepdim)).values


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, wte, wpe, seq):
        tokens = ids.numel()
        H = wte.shape[1]
        out = torch.empty(tokens, H, dtype=wte.dtype, device=wte.device)
        idc = ids.reshape(-1).contiguous()
        call("tb_embedding_fwd", [P, P, P, P, L, I, I, L, I, P], idc.data_ptr(), wte.data_ptr(), nv.ptr(wpe),
             out.data_ptr(), tokens, H, seq, wte.shape[0], dtype_code(wte), nv.stream_ptr())
        ctx.save_for_backward(idc)
        ctx.meta = (wte, wpe, seq, H)
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dout):
        (idc,) = ctx.saved_tensors
        wte, wpe, seq, H = ctx.meta
        d2 = aligned(dout.reshape(-1, H))
        tokens = d2.shape[0]
        g_wte = getattr(wte, "main_grad", None)
        g_wpe = getattr(wpe, "main_grad", None) if wpe is not None else None
        own_wte = g_wte is None
        own_wpe = wpe is not None and g_wpe is None
        if own_wte:
            g_wte = torch.zeros(wte.shape, dtype=torch.float32, device=wte.device)
        if own_wpe:
            g_wpe = torch.zeros(wpe.shape, dtype=torch.float32, device=wpe.device)
        call("tb_embedding_bwd", [P, P, P, P, L, I, I, L, I, P], idc.data_ptr(), d2.data_ptr(), g_wte.data_ptr(),
             nv.ptr(g_wpe), tokens, H, seq, wte.shape[0], dtype_code(d2), nv.stream_ptr())
        return (None, g_wte.to(wte.dtype) if own_wte else None,
                (g_wpe.to(wpe.dtype) if own_wpe else None) if wpe is not None else None, None)


def embedding(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor | None = None) -> torch.Tensor:
    """Token (+ learned position) embedding: ``wte[ids] + wpe[arange(seq)]`` with ``seq = ids.shape[-1]``."""
    seq = ids.shape[-1]
    if kernel_ok(wte, wpe) and ids.is_cuda and wte.shape[1] % 8 == 0 and wte.is_contiguous() and (
            wpe is None or wpe.is_contiguous()):
        return _EmbeddingFn.apply(ids, wte, wpe, seq)
    out = torch.nn.functional.embedding(ids, wte)
    if wpe is not None:
        out = out + wpe[:seq]
    return out


def _rope_torch(x, base, pos_offset, inverse):
    B, S, Hh, D = x.shape
    i = torch.arange(0, D, 2, device=x.device, dtype=torch.float32)
    freq = base ** (-i / D)
    pos = torch.arange(S, device=x.device, dtype=torch.float32) + pos_offset
    ang = pos[:, None] * freq[None, :]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    if inverse:
        sn = -sn
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    out = torch.stack((a * cs - b * sn, a * sn + b * cs), dim=-1).flatten(-2)
    return out.to(x.dtype)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, base, pos_offset):
        ctx.args = (base, pos_offset)
        return _rope_raw(x, base, pos_offset, False)

    @staticmethod
    def backward(ctx, dy):
        base, pos_offset = ctx.args
        return _rope_raw(dy, base, pos_offset, True), None, None


def _rope_raw(x, base, pos_offset, inverse):
    xc = aligned(x)
    B, S, Hh, D = xc.shape
    y = torch.empty_like(xc)
    call("tb_rope", [P, P, L, I, I, I, F, I, I, I, P], xc.data_ptr(), y.data_ptr(), B, S, Hh, D, float(base),
         int(pos_offset), int(inverse), dtype_code(xc), nv.stream_ptr())
    return y


def rope(x: torch.Tensor, base: float = 10000.0, pos_offset: int = 0) -> torch.Tensor:
    """Rotary embedding on ``[B, S, heads, D]``: adjacent pairs ``(2i, 2i+1)`` rotate by
    ``pos * base^(-2i/D)`` (pairing/frequency rule of ``crates/torsh-nn/src/layers/embedding.rs:372-430``)."""
    if kernel_ok(x):
        return _RopeFn.apply(x, base, pos_offset)
    return _rope_torch(x, base, pos_offset, False)


def colsum_into(x2d: torch.Tensor, out_f32: torch.Tensor) -> None:
    """``out_f32[c] += Σ_r x2d[r, c]`` (bias gradients; fp32 accumulation)."""
    if kernel_ok(x2d) and x2d.stride(1) == 1:
        call("tb_colsum", [P, P, L, I, L, I, P], x2d.data_ptr(), out_f32.data_ptr(), x2d.shape[0], x2d.shape[1],
             x2d.stride(0), dtype_code(x2d), nv.stream_ptr())
    else:
        out_f32.add_(x2d.float().sum(0))


def _gnn_scatter_raw(x, src, dst, w, n_dst):
    out = torch.zeros(n_dst, x.shape[1], dtype=torch.float32, device=x.device)
    E = dst.numel()
    call("tb_gnn_scatter", [P, P, P, P, P, L, I, L, L, I, P], x.data_ptr(), nv.ptr(src), dst.data_ptr(), nv.ptr(w),
         out.data_ptr(), E, x.shape[1], x.shape[0], n_dst, dtype_code(x), nv.stream_ptr())
    return out


class _GnnScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, src, dst, w, n_dst):
        ctx.save_for_backward(src, dst, w, x if (w is not None and w.requires_grad) else None)
        ctx.n_src, ctx.xdtype = x.shape[0], x.dtype
        return _gnn_scatter_raw(x, src, dst, w, n_dst).to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        src, dst, w, x = ctx.saved_tensors
        dout = aligned(dout.contiguous())
        E = dst.numel()
        if src is None:  # out[dst[e]] += w[e] x[e]  →  dx[e] = w[e] dout[dst[e]]
            dx = dout[dst]
            if w is not None:
                dx = dx * w[:, None].to(dx.dtype)
        else:            # dx[src[e]] += w[e] dout[dst[e]]: the same kernel with the roles of the index lists swapped
            dx = _gnn_scatter_raw(dout, dst, src, w, ctx.n_src).to(ctx.xdtype)
        dw = None
        if x is not None:
            xs = x if src is None else x[src]
            dw = (xs.float() * dout[dst].float()).sum(1)
        return dx, None, None, dw, None


def gnn_scatter(x: torch.Tensor, dst: torch.Tensor, n_dst: int, src: torch.Tensor | None = None,
                weight: torch.Tensor | None = None) -> torch.Tensor:
    """``out[dst[e]] += weight[e] * x[src[e]]`` (``src=None``: row ``e`` of ``x``; ``weight=None``: 1), fp32 accumulation.

    The gather, the edge weight and the scatter-add are one kernel, so the ``[E, F]`` message tensor of a
    message-passing layer is never written."""
    if kernel_ok(x) and x.dim() == 2 and x.shape[1] % 4 == 0 and dst.is_cuda:
        x = aligned(x.contiguous())
        w = None if weight is None else weight.float().contiguous()
        return _GnnScatterFn.apply(x, None if src is None else src.contiguous(), dst.contiguous(), w, n_dst)
    m = x if src is None else x[src]
    if weight is not None:
        m = m * weight[:, None].to(m.dtype)
    return torch.zeros(n_dst, *x.shape[1:], dtype=x.dtype, device=x.device).index_add_(0, dst, m)
