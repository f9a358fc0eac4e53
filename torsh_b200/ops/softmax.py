"""softmax / log_softmax / fused cross-entropy (kernels in ``csrc/kernels/softmax_xent.cu``).

``cross_entropy`` matches the reference definition log_softmax + NLL with mean reduction
(``crates/torsh-nn/src/functional/loss.rs:15-60``) but computes loss and gradient in one pass.
"""
from __future__ import annotations

import torch

from .. import _native as nv
from ._dispatch import F, I, L, P, aligned, call, dtype_code, kernel_ok


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, log):
        C = x.shape[-1]
        x2 = aligned(x.reshape(-1, C))
        y = torch.empty_like(x2)
        call("tb_softmax_fwd", [P, P, I, I, L, L, I, I, P], x2.data_ptr(), y.data_ptr(), x2.shape[0], C, C, C,
             int(log), dtype_code(x2), nv.stream_ptr())
        ctx.save_for_backward(y)
        ctx.log, ctx.shape = log, x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        dy2 = aligned(dy.reshape(y.shape).to(y.dtype))
        dx = torch.empty_like(y)
        call("tb_softmax_bwd", [P, P, P, I, I, I, I, P], dy2.data_ptr(), y.data_ptr(), dx.data_ptr(), y.shape[0],
             y.shape[1], int(ctx.log), dtype_code(y), nv.stream_ptr())
        return dx.view(ctx.shape), None


def softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if kernel_ok(x) and dim in (-1, x.dim() - 1):
        return _SoftmaxFn.apply(x, False)
    return torch.softmax(x, dim)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    if kernel_ok(x) and dim in (-1, x.dim() - 1):
        return _SoftmaxFn.apply(x, True)
    return torch.log_softmax(x, dim)


_XENT = [P, P, P, P, P, I, I, L, F, L, I, P]


class _CrossEntropyFn(torch.autograd.Function):
    """Loss and d(logits) in one kernel; the gradient is stored (in place when allowed)."""

    @staticmethod
    def forward(ctx, logits, targets, num_classes, ignore_index, inplace_grad, root_scale):
        ld = logits.shape[-1]
        lg = logits.reshape(-1, ld)
        assert lg.stride(1) == 1 and lg.data_ptr() % 16 == 0 and (lg.stride(0) * lg.element_size()) % 16 == 0
        rows = lg.shape[0]
        tg = targets.reshape(-1).contiguous().to(torch.int64)
        valid = (tg != ignore_index).sum().clamp(min=1).to(torch.float32)
        loss_rows = torch.empty(rows, dtype=torch.float32, device=logits.device)
        need_grad = logits.requires_grad
        dl = (lg if inplace_grad else torch.empty_like(lg)) if need_grad else None
        # Generic path: the kernel writes the unscaled gradient and backward multiplies by
        # dloss / valid (both device scalars). With root_scale the caller promises that this loss
        # is the root of backward (upstream gradient 1) and that no target is ignored, so the
        # final scale root_scale / rows is applied inside the kernel and backward is free.
        kscale = 1.0 if root_scale is None else float(root_scale) / rows
        call("tb_cross_entropy", _XENT, lg.data_ptr(), tg.data_ptr(), loss_rows.data_ptr(), None, nv.ptr(dl), rows,
             num_classes, lg.stride(0), kscale, ignore_index, dtype_code(lg), nv.stream_ptr())
        if root_scale is None:
            loss = loss_rows.sum() / valid
        else:
            loss = loss_rows.sum() * (float(root_scale) / rows)
        if need_grad:
            ctx.save_for_backward(dl, valid)
        ctx.shape, ctx.root = logits.shape, root_scale is not None
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dl, valid = ctx.saved_tensors
        g = dl if ctx.root else dl.mul_((dloss / valid).to(dl.dtype))
        return g.view(ctx.shape), None, None, None, None, None


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, *, num_classes: int | None = None,
                  ignore_index: int = -100, inplace_grad: bool = False,
                  root_scale: float | None = None) -> torch.Tensor:
    """Mean next-token / class cross-entropy.

    ``logits`` may carry padding columns beyond ``num_classes`` (a vocabulary padded for TMA
    alignment); those columns get probability and gradient zero. ``root_scale`` (a Python float,
    e.g. 1 / number of micro-batches) selects the fused-backward contract described in
    :class:`_CrossEntropyFn`: the returned loss is ``root_scale * mean`` and must be the tensor on
    which ``backward()`` is called.
    """
    C = logits.shape[-1] if num_classes is None else num_classes
    if kernel_ok(logits) and logits.stride(-1) == 1:
        return _CrossEntropyFn.apply(logits, targets, C, ignore_index, inplace_grad, root_scale)
    lg = logits[..., :C].reshape(-1, C).float()
    loss = torch.nn.functional.cross_entropy(lg, targets.reshape(-1), ignore_index=ignore_index)
    return loss if root_scale is None else loss * root_scale
