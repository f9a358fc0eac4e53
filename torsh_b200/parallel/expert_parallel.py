"""Mixture-of-experts routing and expert parallelism.

Router (``crates/torsh-distributed/src/expert_parallelism/router.rs:231-448``): gate linear → softmax → top-k →
capacity ``ceil(tokens·k/E · capacity_factor)`` with dropped tokens, load-balance loss (coefficient of variation of the
expert loads) and z-loss (mean squared probability... the reference's ``mean p²``), defaults 8 experts, top-2,
capacity factor 1.25, aux coefficients 0.01 / 0.001 (``config.rs``). Dispatch/combine (``manager.rs:101-323``) is an
all-to-all of tokens grouped by owning rank.  On GPUs (bf16, more than one rank) dispatch and combine are the
peer-memory kernels of ``csrc/kernels/moe_sm100.cu``: tokens are stored straight into the owning rank's
``[E_local][world][capacity][H]`` buffer and expert outputs are read back with peer loads weighted by the gate, with no
sort, no size exchange and no staging copy (:class:`FusedMoEDispatch`).  Otherwise it is
``torch.distributed.all_to_all_single`` (gloo: emulated), with a dense single-process path when no group is given.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..nn.module import Module, Parameter


@dataclass
class ExpertParallelismConfig:
    num_experts: int = 8
    top_k: int = 2
    capacity_factor: float = 1.25
    load_balance_coeff: float = 0.01
    z_loss_coeff: float = 0.001
    drop_tokens: bool = True


class TopKRouter(Module):
    def __init__(self, hidden: int, cfg: ExpertParallelismConfig | None = None):
        super().__init__()
        self.cfg = cfg or ExpertParallelismConfig()
        self.gate = Parameter(torch.empty(self.cfg.num_experts, hidden).normal_(0, 0.02))

    def capacity(self, tokens: int) -> int:
        c = self.cfg
        return int(math.ceil(tokens * c.top_k / c.num_experts * c.capacity_factor))

    def forward(self, x: torch.Tensor):
        """``x``: ``[T, H]`` → ``(expert_idx [T,k], weights [T,k], keep [T,k], aux_loss)``."""
        c = self.cfg
        logits = torch.nn.functional.linear(x.float(), self.gate.float())
        probs = torch.softmax(logits, -1)
        w, idx = probs.topk(c.top_k, -1)
        w = w / w.sum(-1, keepdim=True)
        T = x.shape[0]
        cap = self.capacity(T)
        onehot = torch.nn.functional.one_hot(idx, c.num_experts)                       # [T,k,E]
        pos = (onehot.reshape(T * c.top_k, c.num_experts).cumsum(0) - 1).reshape(T, c.top_k, c.num_experts)
        slot = (pos * onehot).sum(-1)                                                  # arrival order within its expert
        keep = slot < cap if c.drop_tokens else torch.ones_like(slot, dtype=torch.bool)
        load = onehot.sum((0, 1)).float()
        cv = load.std(unbiased=False) / load.mean().clamp(min=1e-9)
        aux = c.load_balance_coeff * cv * cv + c.z_loss_coeff * probs.pow(2).mean()
        return idx, w, keep, slot, aux


class FusedMoEDispatch:
    """Symmetric buffers + autograd functions of the peer-memory dispatch / combine."""

    def __init__(self, hidden: int, e_local: int, capacity: int, group=None):
        import ctypes

        from .symm import CommContext, SymmetricBuffer
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.H, self.e_local, self.C = hidden, e_local, capacity
        n = e_local * self.world * capacity * hidden
        self.ctx = CommContext(self.group)
        mk = lambda: SymmetricBuffer(n, torch.bfloat16, self.group)
        self.recv, self.out, self.d_out, self.d_recv = mk(), mk(), mk(), mk()
        self.counts = SymmetricBuffer(max(e_local * self.world, 8), torch.int32, self.group, zero=True)
        dev = self.recv.tensor.device
        self._count_ptrs = torch.tensor(self.counts.peer_ptrs, dtype=torch.int64, device=dev)
        self.shape = (e_local, self.world, capacity, hidden)
        self._ct = ctypes

    # -- raw launches ------------------------------------------------------------------------------------
    def barrier(self):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        call("tb_comm_barrier", [P, I, I, P, P, P], self.ctx.flags.ptr_array, self.rank, self.world, self.ctx.epoch.data_ptr(),
             nv.status_word().data_ptr(), nv.stream_ptr())

    def scatter(self, src, dst_buf, idx, slot, keep, scale=None, counts=None):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        T, K = idx.shape
        call("tb_moe_scatter", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P], src.data_ptr(), dst_buf.ptr_array,
             idx.data_ptr(), slot.data_ptr(), keep.data_ptr(), nv.ptr(scale), nv.ptr(counts),
             self._count_ptrs.data_ptr() if counts is not None else None, T, K, self.H, self.C, self.e_local, self.rank,
             self.world, nv.stream_ptr())

    def gather(self, src_buf, idx, slot, keep, w=None, want_y=True, dy=None):
        from .. import _native as nv
        from ..ops._dispatch import I, P, call
        T, K = idx.shape
        y = torch.empty(T, self.H, dtype=torch.bfloat16, device=idx.device) if want_y else None
        dot = torch.empty(T, K, dtype=torch.float32, device=idx.device) if dy is not None else None
        call("tb_moe_gather", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, P], src_buf.ptr_array, idx.data_ptr(),
             slot.data_ptr(), keep.data_ptr(), nv.ptr(w), nv.ptr(y), nv.ptr(dy), nv.ptr(dot), T, K, self.H, self.C,
             self.e_local, self.rank, self.world, nv.stream_ptr())
        return y, dot

    def valid_mask(self) -> torch.Tensor:
        """``[E_local, world, C, 1]`` mask of the slots the peers filled in the last dispatch."""
        c = self.counts.tensor[: self.e_local * self.world].view(self.e_local, self.world, 1)
        return (torch.arange(self.C, device=c.device).view(1, 1, -1) < c).unsqueeze(-1)

    # -- autograd -----------------------------------------------------------------------------------------
    def dispatch(self, x, idx, slot, keep, counts):
        return _MoEDispatchFn.apply(x, self, idx, slot, keep, counts)

    def combine(self, expert_out, gate, idx, slot, keep):
        return _MoECombineFn.apply(expert_out, gate, self, idx, slot, keep)


class _MoEDispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, d: FusedMoEDispatch, idx, slot, keep, counts):
        d.barrier()                                    # everybody is done reading the buffers of the previous step
        d.scatter(x.contiguous(), d.recv, idx, slot, keep, counts=counts)
        d.barrier()                                    # all rows (and counts) have landed
        ctx.d, ctx.meta = d, (idx, slot, keep)
        return d.recv.tensor.view(d.shape) * d.valid_mask()

    @staticmethod
    def backward(ctx, g):
        d = ctx.d
        idx, slot, keep = ctx.meta
        d.d_recv.tensor.view(d.shape).copy_(g)
        d.barrier()
        dx, _ = d.gather(d.d_recv, idx, slot, keep)    # dx[t] = sum over the token's kept choices of the row gradients
        d.barrier()
        return dx, None, None, None, None, None


class _MoECombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, gate, d: FusedMoEDispatch, idx, slot, keep):
        d.out.tensor.view(d.shape).copy_(expert_out)
        d.barrier()
        y, _ = d.gather(d.out, idx, slot, keep, w=gate.float().contiguous())
        ctx.d, ctx.meta = d, (idx, slot, keep)
        ctx.save_for_backward(gate)
        return y

    @staticmethod
    def backward(ctx, dy):
        d = ctx.d
        idx, slot, keep = ctx.meta
        (gate,) = ctx.saved_tensors
        dy = dy.contiguous()
        g32 = gate.float().contiguous()
        _, dgate = d.gather(d.out, idx, slot, keep, want_y=False, dy=dy)       # <dy[t], expert row>, rows still in place
        d.scatter(dy, d.d_out, idx, slot, keep, scale=g32)                      # gate * dy[t] into the owners' buffers
        d.barrier()
        d_expert = d.d_out.tensor.view(d.shape) * d.valid_mask()
        return d_expert, (dgate * keep).to(gate.dtype), None, None, None, None


class MoELayer(Module):
    """Experts are ``[E_local, H, F]`` / ``[E_local, F, H]`` weight stacks; tokens travel to the rank that owns their
    expert (all-to-all), run through the expert MLP, and travel back."""

    def __init__(self, hidden: int, ffn: int, cfg: ExpertParallelismConfig | None = None, group=None):
        super().__init__()
        self.cfg = cfg or ExpertParallelismConfig()
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        assert self.cfg.num_experts % self.world == 0
        self.e_local = self.cfg.num_experts // self.world
        self.router = TopKRouter(hidden, self.cfg)
        self.w1 = Parameter(torch.empty(self.e_local, hidden, ffn).normal_(0, 0.02))
        self.w2 = Parameter(torch.empty(self.e_local, ffn, hidden).normal_(0, 0.02))

    def _experts(self, xs: torch.Tensor, eid: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(xs)
        for e in range(self.e_local):
            m = eid == e
            if m.any():
                out[m] = torch.nn.functional.gelu(xs[m] @ self.w1[e].to(xs.dtype)) @ self.w2[e].to(xs.dtype)
        return out

    def _forward_fused(self, x, idx, w, keep, slot, aux, shape):
        T = x.shape[0]
        cap = self.router.capacity(T)
        d = getattr(self, "_fused", None)
        if d is None or d.C != cap or d.H != x.shape[1]:
            d = self._fused = FusedMoEDispatch(x.shape[1], self.e_local, cap, self.group)
        counts = torch.bincount(idx[keep].reshape(-1), minlength=self.cfg.num_experts).to(torch.int32)
        keep8 = keep.to(torch.uint8).contiguous()
        xs = d.dispatch(x, idx.contiguous(), slot.contiguous(), keep8, counts)          # [E_local, world, C, H]
        h = xs.reshape(self.e_local, -1, x.shape[1])
        out = torch.bmm(torch.nn.functional.gelu(torch.bmm(h, self.w1.to(h.dtype))), self.w2.to(h.dtype))
        y = d.combine(out.view(d.shape), w.to(torch.float32), idx, slot, keep8)
        return y.view(shape), aux

    def forward(self, x: torch.Tensor):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        idx, w, keep, _, aux = self.router(x)
        T, k = idx.shape
        tok = torch.arange(T, device=x.device).repeat_interleave(k)[keep.reshape(-1)]
        exp = idx.reshape(-1)[keep.reshape(-1)]
        wt = w.reshape(-1)[keep.reshape(-1)]
        if self.world > 1 and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and k <= 8:
            return self._forward_fused(x, idx, w, keep, _, aux, shape)
        if self.world == 1:
            y = self._experts(x[tok], exp)
        else:
            owner = exp // self.e_local
            order = torch.argsort(owner, stable=True)
            send = x[tok][order]
            send_e = (exp % self.e_local)[order]
            counts = torch.bincount(owner, minlength=self.world)
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)
            sc, rc = counts.tolist(), recv_counts.tolist()
            recv = x.new_empty(sum(rc), x.shape[1])
            recv_e = send_e.new_empty(sum(rc))
            dist.all_to_all_single(recv, send, rc, sc, group=self.group)
            dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
            out = self._experts(recv, recv_e)
            back = torch.empty_like(send)
            dist.all_to_all_single(back, out, sc, rc, group=self.group)
            y = torch.empty_like(back)
            y[order] = back
        res = torch.zeros_like(x)
        res.index_add_(0, tok, y * wt.unsqueeze(1).to(y.dtype))
        return res.view(shape), aux
