"""Mixture-of-experts routing and expert parallelism.

Router (``crates/torsh-distributed/src/expert_parallelism/router.rs:231-448``): gate linear → softmax → top-k →
capacity ``ceil(tokens·k/E · capacity_factor)`` with dropped tokens, load-balance loss (coefficient of variation of the
expert loads) and z-loss (mean squared probability... the reference's ``mean p²``), defaults 8 experts, top-2,
capacity factor 1.25, aux coefficients 0.01 / 0.001 (``config.rs``). Dispatch/combine (``manager.rs:101-323``) is an
all-to-all of tokens grouped by owning rank; here it is ``torch.distributed.all_to_all_single`` over NCCL/NVLink
(gloo: emulated), with a dense single-process path when no group is given.
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

    def forward(self, x: torch.Tensor):
        shape = x.shape
        x = x.reshape(-1, shape[-1])
        idx, w, keep, _, aux = self.router(x)
        T, k = idx.shape
        tok = torch.arange(T, device=x.device).repeat_interleave(k)[keep.reshape(-1)]
        exp = idx.reshape(-1)[keep.reshape(-1)]
        wt = w.reshape(-1)[keep.reshape(-1)]
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
