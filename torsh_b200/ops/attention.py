"""Flash attention (forward + backward) on tcgen05 / TMEM, plus a PyTorch fallback for CPU tensors.

Kernels: ``csrc/kernels/attention_fwd_sm100.cu`` and ``attention_bwd_sm100.cu``. The reference's
attention (``crates/torsh-functional/src/attention.rs:192-271,493-629``) uses scale ``1/sqrt(d)`` and
an additive mask; its "flash" variant still materialises ``[block, S]`` scores and has no backward.
"""
from __future__ import annotations

import math

import torch

from .. import _native as nv
from ._dispatch import F, I, L, P, call, kernel_ok

_FWD = [P, P, P, P, P, I, I, I, I, L, L, L, F, I, P, P]
_BWD = [P] * 11 + [I, I, I, I, L, L, L, L, L, F, I, P, P]


def _fwd(q, k, v, out, lse, B, S, H, D, q_stride, kv_stride, scale, causal):
    call("tb_flash_attn_fwd", _FWD, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S,
         H, D, q_stride, kv_stride, out.stride(0), float(scale), int(causal), nv.status_word(q.device).data_ptr(),
         nv.stream_ptr())


def _bwd(q, k, v, o, do, lse, dq, dk, dv, B, S, H, D, q_stride, kv_stride, dqkv_stride, scale, causal):
    delta = torch.empty(B * H * S, dtype=torch.float32, device=q.device)
    dq_acc = torch.empty(B * S * H * D, dtype=torch.float32, device=q.device)
    call("tb_flash_attn_bwd", _BWD, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(),
         lse.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), B, S, H, D,
         q_stride, kv_stride, o.stride(0), do.stride(0), dqkv_stride, float(scale), int(causal),
         nv.status_word(q.device).data_ptr(), nv.stream_ptr())


class _FlashQKVPacked(torch.autograd.Function):
    """qkv: ``[B*S, 3*H*D]`` (q | k | v column bands, head-major inside a band) -> ``[B*S, H*D]``."""

    @staticmethod
    def forward(ctx, qkv, B, S, H, D, causal, scale):
        E = H * D
        assert qkv.shape == (B * S, 3 * E) and qkv.stride(1) == 1 and qkv.dtype == torch.bfloat16
        out = torch.empty(B * S, E, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B * H * S, dtype=torch.float32, device=qkv.device)
        st = qkv.stride(0)
        _fwd(qkv[:, :E], qkv[:, E:2 * E], qkv[:, 2 * E:], out, lse, B, S, H, D, st, st, scale, causal)
        ctx.save_for_backward(qkv, out, lse)
        ctx.dims = (B, S, H, D, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        B, S, H, D, causal, scale = ctx.dims
        E = H * D
        if not dout.is_contiguous():
            dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        st = qkv.stride(0)
        _bwd(qkv[:, :E], qkv[:, E:2 * E], qkv[:, 2 * E:], out, dout, lse, dqkv[:, :E], dqkv[:, E:2 * E],
             dqkv[:, 2 * E:], B, S, H, D, st, st, dqkv.stride(0), scale, causal)
        return dqkv, None, None, None, None, None, None


class _FlashSeparate(torch.autograd.Function):
    """q, k, v: ``[B, S, H, D]`` contiguous -> ``[B, S, H, D]``."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        B, S, H, D = q.shape
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        out = torch.empty(B * S, H * D, dtype=q.dtype, device=q.device)
        lse = torch.empty(B * H * S, dtype=torch.float32, device=q.device)
        _fwd(q, k, v, out, lse, B, S, H, D, H * D, H * D, scale, causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = (causal, scale)
        return out.view(B, S, H, D)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        causal, scale = ctx.meta
        B, S, H, D = q.shape
        do = dout.reshape(B * S, H * D)
        if not do.is_contiguous():
            do = do.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _bwd(q, k, v, out, do, lse, dq, dk, dv, B, S, H, D, H * D, H * D, H * D, scale, causal)
        return dq, dk, dv, None, None


def _sdpa_reference(q, k, v, causal, scale):
    """fp32 maths on [B, S, H, D]; the CPU path and the test oracle."""
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[1]
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    o = torch.matmul(torch.softmax(s, -1), vf)
    return o.transpose(1, 2).to(q.dtype)


def flash_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                    scale: float | None = None) -> torch.Tensor:
    """Scaled dot-product attention on ``[B, S, H, D]`` tensors with O(S) memory."""
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if kernel_ok(q, k, v) and q.dtype == torch.bfloat16 and D in (64, 128) and k.shape == q.shape:
        return _FlashSeparate.apply(q, k, v, causal, scale)
    return _sdpa_reference(q, k, v, causal, scale)


def flash_attention_qkvpacked(qkv: torch.Tensor, B: int, S: int, H: int, D: int, causal: bool = True,
                              scale: float | None = None) -> torch.Tensor:
    """Attention straight from the fused QKV projection output ``[B*S, 3*H*D]``; returns ``[B*S, H*D]``."""
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    E = H * D
    if kernel_ok(qkv) and qkv.dtype == torch.bfloat16 and D in (64, 128):
        return _FlashQKVPacked.apply(qkv, B, S, H, D, causal, scale)
    q, k, v = (qkv[:, i * E:(i + 1) * E].reshape(B, S, H, D) for i in range(3))
    return _sdpa_reference(q, k, v, causal, scale).reshape(B * S, E)
