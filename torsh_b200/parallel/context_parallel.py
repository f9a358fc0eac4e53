"""Context (sequence-length) parallelism for attention: Ulysses all-to-all and ring attention.

The reference has no context parallelism (its nearest pieces are query-block tiling in
``crates/torsh-functional/src/attention.rs:493-629`` and the BigBird / Longformer sparse patterns); these two
schemes fill the slot for sequences that do not fit one GPU. Every rank holds ``S / cp`` consecutive tokens.

* :func:`ulysses_attention` swaps the sharded axis with two all-to-alls: tokens are gathered and heads scattered, each
  rank runs ordinary (flash) attention over the full sequence for ``H / cp`` heads, and the result is swapped back.
* :func:`ring_attention` keeps the queries in place and passes key / value blocks around the ring; partial results are
  merged with their log-sum-exp, so memory stays O(S / cp) per rank. Causal masks skip the blocks that lie entirely in
  the future.

Both are differentiable (the all-to-all is its own transpose; the ring's backward sends the key / value gradients on
round the ring with the blocks they belong to).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import attention as attn_ops


def _group(group):
    return group if group is not None else dist.group.WORLD


def _all_to_all_chunks(chunks: list[torch.Tensor], group) -> list[torch.Tensor]:
    out = [torch.empty(c.shape, dtype=c.dtype, device=c.device) for c in chunks]
    if chunks[0].is_cuda:
        dist.all_to_all(out, [c.contiguous() for c in chunks], group=group)
    else:  # gloo has no all-to-all: one scatter per source rank
        me = dist.get_rank(group)
        for src in range(dist.get_world_size(group)):
            dist.scatter(out[src], [c.contiguous() for c in chunks] if me == src else None,
                         dist.get_global_rank(group, src), group=group)
    return out


class _SeqToHead(torch.autograd.Function):
    """``[B, S/cp, H, D]`` (all heads, my tokens) → ``[B, S, H/cp, D]`` (my heads, all tokens)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        parts = _all_to_all_chunks(list(x.chunk(w, dim=2)), group)        # part r: rank r's tokens, my heads
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, dy):
        return _HeadToSeq.apply(dy, ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    """``[B, S, H/cp, D]`` → ``[B, S/cp, H, D]``."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        parts = _all_to_all_chunks(list(x.chunk(w, dim=1)), group)        # part r: my tokens, rank r's heads
        return torch.cat(parts, dim=2)

    @staticmethod
    def backward(ctx, dy):
        return _SeqToHead.apply(dy, ctx.group), None


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, group=None,
                      scale: float | None = None) -> torch.Tensor:
    """``q, k, v``: ``[B, S/cp, H, D]`` token shards (rank r holds tokens ``r·S/cp …``); ``H`` must divide by ``cp``."""
    g = _group(group)
    w = dist.get_world_size(g)
    if w == 1:
        return attn_ops.flash_attention(q, k, v, causal=causal, scale=scale)
    if q.shape[2] % w:
        raise ValueError(f"Ulysses attention needs heads ({q.shape[2]}) divisible by the group size ({w})")
    qh, kh, vh = (_SeqToHead.apply(t, g) for t in (q, k, v))
    out = attn_ops.flash_attention(qh.contiguous(), kh.contiguous(), vh.contiguous(), causal=causal, scale=scale)
    return _HeadToSeq.apply(out, g)


def _exchange(send: torch.Tensor, dst: int, src: int, group) -> torch.Tensor:
    recv = torch.empty(send.shape, dtype=send.dtype, device=send.device)
    ops = [dist.P2POp(dist.isend, send.contiguous(), dist.get_global_rank(group, dst), group),
           dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, src), group)]
    for wk in dist.batch_isend_irecv(ops):
        wk.wait()
    return recv


class _RingShift(torch.autograd.Function):
    """Forward: give my tensor to the next rank and take the previous rank's; backward: the gradients travel back."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w, r = dist.get_world_size(group), dist.get_rank(group)
        return _exchange(x, (r + 1) % w, (r - 1) % w, group)

    @staticmethod
    def backward(ctx, dy):
        w, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        return _exchange(dy, (r - 1) % w, (r + 1) % w, ctx.group), None


def _block_attention(q, k, v, scale, mask):
    """Attention of one query block against one key block in fp32: returns (output, log-sum-exp per query)."""
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                                      # [B, H, Sq]
    p = torch.exp(s - lse[..., None])
    return torch.einsum("bhqk,bkhd->bqhd", p, v.float()), lse


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False, group=None,
                   scale: float | None = None) -> torch.Tensor:
    """``q, k, v``: ``[B, S/cp, H, D]`` token shards in rank order. ``cp`` steps; in step ``t`` a rank holds the key /
    value block of rank ``r - t`` and merges its contribution through the running log-sum-exp."""
    g = _group(group)
    w, r = dist.get_world_size(g), dist.get_rank(g)
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    n = q.shape[1]
    tri = torch.ones(n, n, dtype=torch.bool, device=q.device).tril() if causal else None
    out, lse = None, None
    kv = torch.stack([k, v])               # one message per step, so the ranks cannot pair up different tensors
    for t in range(w):
        src = (r - t) % w
        if causal and src > r:
            # a block entirely in the future adds nothing, but it stays in the graph: every rank must take part in the
            # backward exchange of every step
            out = out + 0.0 * kv.sum().to(out.dtype)
        else:
            o_blk, lse_blk = _block_attention(q, kv[0], kv[1], scale, tri if (causal and src == r) else None)
            if out is None:
                out, lse = o_blk, lse_blk
            else:
                new = torch.logaddexp(lse, lse_blk)
                out = out * torch.exp(lse - new).transpose(1, 2)[..., None] + \
                    o_blk * torch.exp(lse_blk - new).transpose(1, 2)[..., None]
                lse = new
        if t + 1 < w:
            kv = _RingShift.apply(kv, g)
    return out.to(q.dtype)


class ContextParallelAttention(torch.nn.Module):
    """Self-attention over a sequence sharded across ``group``: ``mode`` is ``"ulysses"`` or ``"ring"``."""

    def __init__(self, embed_dim: int, num_heads: int, mode: str = "ulysses", causal: bool = True, group=None, bias: bool = True):
        super().__init__()
        if mode not in ("ulysses", "ring"):
            raise ValueError("mode must be 'ulysses' or 'ring'")
        self.h, self.mode, self.causal, self.group = num_heads, mode, causal, group
        self.qkv = torch.nn.Linear(embed_dim, 3 * embed_dim, bias=bias)
        self.proj = torch.nn.Linear(embed_dim, embed_dim, bias=bias)

    def forward(self, x):
        """``x``: ``[B, S/cp, E]``, this rank's tokens."""
        b, n, e = x.shape
        q, k, v = self.qkv(x).view(b, n, 3, self.h, e // self.h).unbind(2)
        fn = ulysses_attention if self.mode == "ulysses" else ring_attention
        return self.proj(fn(q, k, v, causal=self.causal, group=self.group).reshape(b, n, e))
