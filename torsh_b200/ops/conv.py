"""Channels-last bf16 convolution, BatchNorm2d and pooling on the sm_100a kernels (``csrc/kernels/conv_pool.cu`` +
the tcgen05 GEMM).

Activations are ``[N, H, W, C]`` bf16 tensors.  A convolution is one GEMM: 1x1 / stride 1 passes the activation
matrix straight to the GEMM; every other geometry runs ``im2col`` first.  The input gradient is a GEMM against the
untransposed weight matrix (MN-major B operand) followed by a gather-form ``col2im``; the weight gradient is a
split-K GEMM over the pixel dimension with both operands MN-major, accumulated in fp32.  Parameters stay fp32
(``[Co, Ci, KH, KW]`` like ``torch.nn.Conv2d``); the bf16 ``[Co, KH*KW*Ci]`` operand is made inside the op, which is
the bf16-autocast recipe of the reference's ResNet benchmark.

BatchNorm2d (training) = column statistics + one fused apply pass ``relu((x - mean) * rstd * gamma + beta + residual)``;
the reference's ``fused_batch_norm`` / ``fused_conv_bn_relu`` helpers (``crates/torsh-functional/src/fusion``) are
host loops.
"""
from __future__ import annotations

import os

import torch

from .. import _native as nv
from ._dispatch import F, I, L, P, call, kernel_ok
from .gemm import gemm


def _out_hw(h, w, k, stride, pad):
    return (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1


def _weight_matrix(weight: torch.Tensor, kpad: int) -> torch.Tensor:
    co, ci, kh, kw = weight.shape
    k = kh * kw * ci
    w = weight.detach().permute(0, 2, 3, 1).reshape(co, k)
    if kpad == k:
        return w.to(torch.bfloat16).contiguous()
    out = torch.zeros(co, kpad, dtype=torch.bfloat16, device=weight.device)
    out[:, :k] = w
    return out


def _im2col(x, kh, kw, stride, pad, kpad):
    n, h, w, c = x.shape
    ho, wo = _out_hw(h, w, kh, stride, pad)
    cols = torch.empty(n * ho * wo, kpad, dtype=torch.bfloat16, device=x.device)
    call("tb_im2col_nhwc", [P, P, I, I, I, I, I, I, I, I, L, P], x.data_ptr(), cols.data_ptr(), n, h, w, c, kh, kw,
         stride, pad, kpad, nv.stream_ptr())
    return cols


def _conv3x3_gemm(x, wm, cout, mode):
    """Implicit-GEMM 3x3/1/1 convolution (mode 1) or its input gradient (mode 2): no column matrix is written."""
    n, h, w, c = x.shape
    y = torch.empty(n * h * w, cout, dtype=torch.bfloat16, device=x.device)
    st = nv.status_word(x.device)
    call("tb_conv3x3_gemm", [P, P, P, I, I, I, I, I, I, I, I, I, P, P], x.data_ptr(), wm.data_ptr(), y.data_ptr(), n, h, w, c,
         cout, mode, wm.stride(0), cout, 0, st.data_ptr(), nv.stream_ptr())
    return y


def _implicit_ok(c, co, kh, kw, stride, pad, w):
    return kh == 3 and kw == 3 and stride == 1 and pad == 1 and c % 64 == 0 and co % 64 == 0 and w <= 128


def _wgrad_split(m_out, n_out, k):
    bn = 256 if n_out >= 256 else 128
    tiles = ((m_out + 127) // 128) * ((n_out + bn - 1) // bn)
    kb = (k + 63) // 64
    # measured on B200: the best split keeps tiles x splits within two waves of the 148 SMs and leaves every split
    # at least 32 K-blocks (K = 8192: 32 tiles -> 4, 96 -> 3, 128 -> 2); deeper splits only add fp32 atomic traffic
    return bn, max(1, min(296 // max(tiles, 1), kb // 32))


class _Conv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, stride, pad):
        n, h, w, c = x.shape
        co, ci, kh, kw = weight.shape
        assert ci == c, f"conv2d: input has {c} channels, weight expects {ci}"
        k = kh * kw * ci
        kpad = (k + 7) // 8 * 8
        ho, wo = _out_hw(h, w, kh, stride, pad)
        direct = kh == 1 and kw == 1 and stride == 1 and pad == 0
        implicit = _implicit_ok(c, co, kh, kw, stride, pad, w)
        wm = _weight_matrix(weight, kpad)
        if implicit:
            a = x                                    # the column matrix is rebuilt in backward for the weight gradient only
            y = _conv3x3_gemm(x, wm, co, 1)
        else:
            a = x.reshape(n * h * w, c) if direct else _im2col(x, kh, kw, stride, pad, kpad)
            y = gemm(a, wm)
        ctx.save_for_backward(a, wm)
        ctx.geom = (n, h, w, c, co, kh, kw, stride, pad, ho, wo, k, kpad, direct, implicit)
        ctx.wshape, ctx.wdtype = weight.shape, weight.dtype
        return y.view(n, ho, wo, co)

    @staticmethod
    def backward(ctx, dy):
        a, wm = ctx.saved_tensors
        n, h, w, c, co, kh, kw, stride, pad, ho, wo, k, kpad, direct, implicit = ctx.geom
        dy2 = dy.reshape(n * ho * wo, co)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        if implicit:
            if ctx.needs_input_grad[0]:
                dx = _conv3x3_gemm(dy2.view(n, ho, wo, co), wm, c, 2).view(n, h, w, c)
            if ctx.needs_input_grad[1]:
                if w <= 64:
                    # dW = dy^T * shifted x, accumulated over pixel blocks straight from the two activations
                    kb = n * ((h + max(64 // w, 1) - 1) // max(64 // w, 1)) if h * w > 64 else (n + 64 // (h * w) - 1) // (64 // (h * w))
                    tiles = ((co + 127) // 128) * ((kpad + 255) // 256)
                    sk = max(1, min(296 // max(tiles, 1), kb // 16))
                    g = torch.zeros(co, kpad, dtype=torch.float32, device=dy.device)
                    st = nv.status_word(dy.device)
                    call("tb_conv3x3_wgrad", [P, P, P, I, I, I, I, I, I, I, I, P, P], dy2.data_ptr(), a.data_ptr(), g.data_ptr(),
                         n, h, w, c, co, kpad, sk, 0, st.data_ptr(), nv.stream_ptr())
                    dw = g[:, :k].reshape(co, kh, kw, c).permute(0, 3, 1, 2).to(ctx.wdtype)
                    return dx, dw, None, None
                a = _im2col(a, kh, kw, stride, pad, kpad)
        elif ctx.needs_input_grad[0]:
            dcols = gemm(dy2, wm, b_major=1)                       # [M, Kpad] = dy · W
            if direct:
                dx = dcols.view(n, h, w, c)
            else:
                dx = torch.empty(n, h, w, c, dtype=torch.bfloat16, device=dy.device)
                call("tb_col2im_nhwc", [P, P, I, I, I, I, I, I, I, I, L, P], dcols.data_ptr(), dx.data_ptr(), n, h, w, c,
                     kh, kw, stride, pad, kpad, nv.stream_ptr())
        if ctx.needs_input_grad[1]:
            bn, sk = _wgrad_split(co, kpad, dy2.shape[0])
            g = torch.zeros(co, kpad, dtype=torch.float32, device=dy.device)
            gemm(dy2, a, a_major=1, b_major=1, out=g, atomic=True, split_k=sk, bn=bn)   # dyᵀ · cols
            dw = g[:, :k].reshape(co, kh, kw, c).permute(0, 3, 1, 2).to(ctx.wdtype)
        return dx, dw, None, None


def conv2d_nhwc(x: torch.Tensor, weight: torch.Tensor, stride: int = 1, padding: int = 0) -> torch.Tensor:
    """``x``: ``[N, H, W, Ci]`` bf16; ``weight``: ``[Co, Ci, KH, KW]`` (any float dtype / memory format); no bias,
    no groups, no dilation.  Returns ``[N, Ho, Wo, Co]`` bf16."""
    if kernel_ok(x) and x.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0:
        if x.shape[-1] % 4:
            # odd channel counts (the 3-channel stem): pad to a multiple of 4 so im2col moves 8-byte vectors
            extra = 4 - x.shape[-1] % 4
            x = torch.nn.functional.pad(x, (0, extra))
            weight = torch.nn.functional.pad(weight, (0, 0, 0, 0, 0, extra))
        return _Conv2dFn.apply(x.contiguous(), weight, stride, padding)
    y = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2).to(weight.dtype), weight, None, stride, padding)
    return y.permute(0, 2, 3, 1).to(x.dtype)


# TORSH_BN_RECOMPUTE_MASK=0 keeps the output for the backward's ReLU mask instead of recomputing it from x
_BN_RECOMPUTE_MASK = os.environ.get("TORSH_BN_RECOMPUTE_MASK", "1") != "0"


class _BatchNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, residual, run_mean, run_var, eps, momentum, relu):
        c = x.shape[-1]
        rows = x.numel() // c
        dev = x.device
        y = torch.empty_like(x)
        sums = torch.empty(2 * c, dtype=torch.float32, device=dev)
        mean = torch.empty(c, dtype=torch.float32, device=dev)
        rstd = torch.empty(c, dtype=torch.float32, device=dev)
        g32, b32 = gamma.detach().float(), beta.detach().float()
        call("tb_bn_fwd", [P, P, P, P, P, P, P, P, P, P, L, I, F, F, I, P], x.data_ptr(), nv.ptr(residual), y.data_ptr(),
             sums.data_ptr(), mean.data_ptr(), rstd.data_ptr(), g32.data_ptr(), b32.data_ptr(), nv.ptr(run_mean),
             nv.ptr(run_var), rows, c, eps, momentum, int(relu), nv.stream_ptr())
        # without a residual the backward recomputes the ReLU mask from x, so the output need not be kept for it
        c8 = c // 8
        recompute = relu and residual is None and c8 <= 256 and (c8 & (c8 - 1)) == 0 and _BN_RECOMPUTE_MASK
        ctx.save_for_backward(x, y if (relu and not recompute) else None, mean, rstd, g32, b32)
        ctx.relu, ctx.has_res, ctx.pdtype = relu, residual is not None, gamma.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, mean, rstd, g32, b32 = ctx.saved_tensors
        c = x.shape[-1]
        rows = x.numel() // c
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dres = torch.empty_like(x) if ctx.has_res else None
        sums = torch.empty(2 * c, dtype=torch.float32, device=x.device)
        dgb = torch.zeros(2, c, dtype=torch.float32, device=x.device)
        call("tb_bn_bwd", [P, P, P, P, P, P, P, P, P, P, P, P, L, I, I, P], dy.data_ptr(), nv.ptr(y), x.data_ptr(),
             mean.data_ptr(), rstd.data_ptr(), g32.data_ptr(), b32.data_ptr(), sums.data_ptr(), dx.data_ptr(), nv.ptr(dres),
             dgb[0].data_ptr(), dgb[1].data_ptr(), rows, c, int(ctx.relu), nv.stream_ptr())
        return dx, dgb[0].to(ctx.pdtype), dgb[1].to(ctx.pdtype), dres, None, None, None, None, None


def batch_norm_nhwc(x: torch.Tensor, bn: torch.nn.BatchNorm2d, residual: torch.Tensor | None = None,
                    relu: bool = False) -> torch.Tensor:
    """``relu(BN(x) + residual)`` over the last (channel) dim of a bf16 channels-last tensor, with ``bn``'s parameters
    and running statistics (updated in training mode)."""
    c = x.shape[-1]
    if kernel_ok(x) and x.dtype == torch.bfloat16 and c % 8 == 0 and bn.affine:
        x = x.contiguous()
        residual = None if residual is None else residual.contiguous()
        if bn.training or not bn.track_running_stats:
            if bn.track_running_stats and bn.num_batches_tracked is not None:
                bn.num_batches_tracked.add_(1)
            mom = bn.momentum if bn.momentum is not None else 0.1
            return _BatchNormFn.apply(x, bn.weight, bn.bias, residual, bn.running_mean if bn.track_running_stats else None,
                                      bn.running_var if bn.track_running_stats else None, bn.eps, mom, relu)
        y = torch.empty_like(x)
        rstd = torch.rsqrt(bn.running_var.float() + bn.eps)
        call("tb_bn_apply", [P, P, P, P, P, P, P, L, I, I, P], x.data_ptr(), nv.ptr(residual), y.data_ptr(),
             bn.running_mean.float().data_ptr(), rstd.data_ptr(), bn.weight.detach().float().data_ptr(),
             bn.bias.detach().float().data_ptr(), x.numel() // c, c, int(relu), nv.stream_ptr())
        return y
    xc = x.movedim(-1, 1).float()
    y = torch.nn.functional.batch_norm(xc, bn.running_mean, bn.running_var, bn.weight, bn.bias, bn.training,
                                       bn.momentum if bn.momentum is not None else 0.1, bn.eps).movedim(1, -1)
    if residual is not None:
        y = y + residual.float()
    return (torch.relu(y) if relu else y).to(x.dtype)


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, stride, pad):
        n, h, w, c = x.shape
        ho, wo = _out_hw(h, w, k, stride, pad)
        y = torch.empty(n, ho, wo, c, dtype=x.dtype, device=x.device)
        idx = torch.empty(n, ho, wo, c, dtype=torch.uint8, device=x.device)
        call("tb_maxpool_fwd", [P, P, P, I, I, I, I, I, I, I, P], x.data_ptr(), y.data_ptr(), idx.data_ptr(), n, h, w, c, k,
             stride, pad, nv.stream_ptr())
        ctx.save_for_backward(idx)
        ctx.geom = (n, h, w, c, k, stride, pad)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        n, h, w, c, k, stride, pad = ctx.geom
        dx = torch.empty(n, h, w, c, dtype=dy.dtype, device=dy.device)
        call("tb_maxpool_bwd", [P, P, P, I, I, I, I, I, I, I, P], dy.contiguous().data_ptr(), idx.data_ptr(), dx.data_ptr(),
             n, h, w, c, k, stride, pad, nv.stream_ptr())
        return dx, None, None, None


def max_pool_nhwc(x: torch.Tensor, kernel: int = 3, stride: int = 2, padding: int = 1) -> torch.Tensor:
    if kernel_ok(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _MaxPoolFn.apply(x.contiguous(), kernel, stride, padding)
    return torch.nn.functional.max_pool2d(x.permute(0, 3, 1, 2), kernel, stride, padding).permute(0, 2, 3, 1)


class _AvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        n, h, w, c = x.shape
        y = torch.empty(n, c, dtype=x.dtype, device=x.device)
        call("tb_avgpool_fwd", [P, P, I, I, I, P], x.data_ptr(), y.data_ptr(), n, h * w, c, nv.stream_ptr())
        ctx.geom = (n, h, w, c)
        return y

    @staticmethod
    def backward(ctx, dy):
        n, h, w, c = ctx.geom
        dx = torch.empty(n, h, w, c, dtype=dy.dtype, device=dy.device)
        call("tb_avgpool_bwd", [P, P, I, I, I, P], dy.contiguous().data_ptr(), dx.data_ptr(), n, h * w, c, nv.stream_ptr())
        return dx


def global_avg_pool_nhwc(x: torch.Tensor) -> torch.Tensor:
    """``[N, H, W, C] → [N, C]`` mean over the spatial dims."""
    if kernel_ok(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _AvgPoolFn.apply(x.contiguous())
    return x.float().mean((1, 2)).to(x.dtype)


# ---- depthwise and grouped convolution ---------------------------------------------------------------------------
class _DepthwiseFn(torch.autograd.Function):
    """x [N, H, W, C] bf16, w [K, K, C] bf16 (taps major, channels contiguous), bias [C] bf16 or None."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, padding):
        n, h, wd, c = x.shape
        k = w.shape[0]
        ho, wo = _out_hw(h, wd, k, stride, padding)
        y = torch.empty(n, ho, wo, c, dtype=torch.bfloat16, device=x.device)
        call("tb_dwconv_fwd", [P, P, P, P] + [I] * 9 + [P], x.data_ptr(), w.data_ptr(), nv.ptr(bias), y.data_ptr(), n, h, wd, c,
             ho, wo, k, stride, padding, nv.stream_ptr())
        ctx.save_for_backward(x, w)
        ctx.cfg = (stride, padding, bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        stride, padding, has_bias = ctx.cfg
        n, h, wd, c = x.shape
        k = w.shape[0]
        dy = dy.contiguous()
        ho, wo = dy.shape[1], dy.shape[2]
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            call("tb_dwconv_dgrad", [P, P, P] + [I] * 9 + [P], dy.data_ptr(), w.data_ptr(), dx.data_ptr(), n, h, wd, c, ho, wo, k,
                 stride, padding, nv.stream_ptr())
        if ctx.needs_input_grad[1] or (has_bias and ctx.needs_input_grad[2]):
            gw = torch.zeros(k, k, c, dtype=torch.float32, device=x.device)
            gb = torch.zeros(c, dtype=torch.float32, device=x.device) if has_bias else None
            call("tb_dwconv_wgrad", [P, P, P, P] + [I] * 9 + [P], x.data_ptr(), dy.data_ptr(), gw.data_ptr(), nv.ptr(gb), n, h, wd, c,
                 ho, wo, k, stride, padding, nv.stream_ptr())
            dw = gw.to(w.dtype)
            db = None if gb is None else gb.to(torch.bfloat16)
        return dx, dw, db, None, None


def depthwise_conv2d_nhwc(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride: int = 1,
                          padding: int = 0) -> torch.Tensor:
    """Depthwise convolution (groups == channels), channels-last. ``x`` is ``[N, H, W, C]``, ``weight`` has PyTorch's
    ``[C, 1, K, K]`` layout. bf16 with C a multiple of 8 runs on the kernels (`tb_dwconv_*`); anything else goes through
    ``torch.nn.functional.conv2d``."""
    c = x.shape[-1]
    k = weight.shape[-1]
    if kernel_ok(x) and x.dtype == torch.bfloat16 and c % 8 == 0 and weight.shape[0] == c and weight.shape[1] == 1 \
            and weight.shape[2] == weight.shape[3]:
        w = weight.reshape(c, k, k).permute(1, 2, 0).to(torch.bfloat16).contiguous()       # [K, K, C]; autograd tracks the permute
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        return _DepthwiseFn.apply(x.contiguous(), w, b, stride, padding)
    y = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2).to(weight.dtype), weight, bias, stride, padding, groups=c)
    return y.permute(0, 2, 3, 1).to(x.dtype)


def grouped_conv2d_nhwc(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride: int = 1,
                        padding: int = 0, groups: int = 1) -> torch.Tensor:
    """Convolution with channel groups, channels-last: groups == 1 is :func:`conv2d_nhwc`, groups == C the depthwise kernel,
    anything between runs one tensor-core convolution per group on its channel slice and concatenates the results (the
    cuDNN `group_count` path of the reference, crates/torsh-backend/src/cuda/cudnn/operations.rs:364)."""
    c = x.shape[-1]
    if groups == 1:
        y = conv2d_nhwc(x, weight, stride, padding)
        return y if bias is None else y + bias.to(y.dtype)
    if groups == c and weight.shape[1] == 1:
        return depthwise_conv2d_nhwc(x, weight, bias, stride, padding)
    if c % groups or weight.shape[0] % groups:
        raise ValueError(f"channels ({c}) and filters ({weight.shape[0]}) must be multiples of groups ({groups})")
    cg, og = c // groups, weight.shape[0] // groups
    outs = []
    for g in range(groups):
        xg = x[..., g * cg:(g + 1) * cg].contiguous()
        outs.append(conv2d_nhwc(xg, weight[g * og:(g + 1) * og], stride, padding))
    y = torch.cat(outs, -1)
    return y if bias is None else y + bias.to(y.dtype)
