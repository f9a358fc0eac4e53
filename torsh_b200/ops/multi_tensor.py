"""Multi-tensor launch tables for the fused optimizer kernels (``csrc/kernels/optim.cu``).

A table row holds up to six device pointers plus a length; a block map assigns each CTA one
16 384-element chunk of one tensor. Tables live on the device and are rebuilt only when a pointer
changes, so an optimizer step over hundreds of parameters is one launch.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import _native as nv
from ._dispatch import F, I, P, call

CHUNK = 16384


class TensorTable:
    """Device-resident (pointer table, block map) for a list of tensor groups.

    ``groups[i]`` is a tuple of up to six tensors (or None) of equal numel: the slots a kernel
    expects (e.g. low-precision copy, master, grad, exp_avg, exp_avg_sq, extra).
    """

    def __init__(self, groups, device):
        self.key = tuple(tuple(0 if t is None else t.data_ptr() for t in g) for g in groups)
        n = len(groups)
        tab = np.zeros((n, 7), dtype=np.int64)
        blk_t, blk_c = [], []
        for i, g in enumerate(groups):
            numel = next(t for t in g if t is not None).numel()
            for s, t in enumerate(g):
                if t is not None:
                    assert t.is_contiguous() and t.numel() == numel
                    tab[i, s] = t.data_ptr()
            tab[i, 6] = numel
            nchunks = (numel + CHUNK - 1) // CHUNK
            blk_t.extend([i] * nchunks)
            blk_c.extend(range(nchunks))
        self.ntensors = n
        self.nblocks = len(blk_t)
        self.table = torch.from_numpy(tab).to(device)
        self.blk_tensor = torch.tensor(blk_t, dtype=torch.int32, device=device)
        self.blk_chunk = torch.tensor(blk_c, dtype=torch.int32, device=device)
        self._keep = groups  # keep the tensors alive while their pointers are in the table

    @staticmethod
    def cached(cache: dict, name: str, groups, device) -> "TensorTable":
        key = tuple(tuple(0 if t is None else t.data_ptr() for t in g) for g in groups)
        tt = cache.get(name)
        if tt is None or tt.key != key:
            tt = TensorTable(groups, device)
            cache[name] = tt
        return tt


def adam_step(tt: TensorTable, *, lr, beta1, beta2, eps, weight_decay, step, decoupled=True, amsgrad=False,
              grad_dtype=torch.float32, grad_scale=1.0, zero_grad=False, found_inf: torch.Tensor | None = None,
              dyn: torch.Tensor | None = None):
    """Slots: (lowp copy | None, master fp32, grad, exp_avg, exp_avg_sq, max_exp_avg_sq | None).

    ``dyn`` (3 fp32 on the device: lr, 1-β1ᵗ, 1-β2ᵗ) overrides the by-value scalars; a captured CUDA
    graph then keeps stepping correctly when the host refreshes ``dyn`` before each replay."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    call("tb_adam_multi", [P, P, P, I] + [F] * 8 + [I] * 4 + [P, P, P], tt.table.data_ptr(), tt.blk_tensor.data_ptr(),
         tt.blk_chunk.data_ptr(), tt.nblocks, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale, int(decoupled),
         int(amsgrad), 0 if grad_dtype == torch.bfloat16 else 1, int(zero_grad), nv.ptr(found_inf), nv.ptr(dyn),
         nv.stream_ptr())


def sgd_step(tt: TensorTable, *, lr, momentum, dampening, weight_decay, nesterov, grad_dtype=torch.float32,
             grad_scale=1.0, zero_grad=False, found_inf=None):
    """Slots: (lowp copy | None, master fp32, grad, momentum buffer | None)."""
    call("tb_sgd_multi", [P, P, P, I] + [F] * 5 + [I] * 3 + [P, P], tt.table.data_ptr(), tt.blk_tensor.data_ptr(),
         tt.blk_chunk.data_ptr(), tt.nblocks, lr, momentum, dampening, weight_decay, grad_scale, int(nesterov),
         0 if grad_dtype == torch.bfloat16 else 1, int(zero_grad), nv.ptr(found_inf), nv.stream_ptr())


def lamb_step(tt: TensorTable, norms: torch.Tensor, *, lr, beta1, beta2, eps, weight_decay, step, bias_correction=True,
              trust_clip=1.0, grad_dtype=torch.float32, grad_scale=1.0):
    """Slots: (lowp copy | None, master fp32, grad, exp_avg, exp_avg_sq, update scratch fp32)."""
    bc1 = 1.0 - beta1 ** step if bias_correction else 1.0
    bc2 = 1.0 - beta2 ** step if bias_correction else 1.0
    call("tb_lamb_multi", [P, P, P, I, I] + [F] * 9 + [I, P, P], tt.table.data_ptr(), tt.blk_tensor.data_ptr(),
         tt.blk_chunk.data_ptr(), tt.nblocks, tt.ntensors, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale,
         trust_clip, 0 if grad_dtype == torch.bfloat16 else 1, norms.data_ptr(), nv.stream_ptr())


def sq_norm(tt: TensorTable, slot: int, dtype, out: torch.Tensor, per_tensor: torch.Tensor | None = None):
    """``out[0] = Σ x²`` over slot ``slot`` of every table row (fp32)."""
    call("tb_sqnorm_multi", [P, P, P, I, I, I, P, P, P], tt.table.data_ptr(), tt.blk_tensor.data_ptr(),
         tt.blk_chunk.data_ptr(), tt.nblocks, slot, 0 if dtype == torch.bfloat16 else 1, out.data_ptr(),
         nv.ptr(per_tensor), nv.stream_ptr())


def scale_(tt: TensorTable, slot: int, dtype, scale: float = 1.0, *, clip_sqnorm: torch.Tensor | None = None,
           max_norm: float = 0.0, found_inf: torch.Tensor | None = None):
    """In-place ``x *= scale`` (or clip-by-global-norm when ``clip_sqnorm`` is given), flagging non-finite values."""
    call("tb_scale_multi", [P, P, P, I, I, I, F, P, F, I, P, P], tt.table.data_ptr(), tt.blk_tensor.data_ptr(),
         tt.blk_chunk.data_ptr(), tt.nblocks, slot, 0 if dtype == torch.bfloat16 else 1, scale, nv.ptr(clip_sqnorm),
         max_norm, 1 if clip_sqnorm is not None else 0, nv.ptr(found_inf), nv.stream_ptr())
