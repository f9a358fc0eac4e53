"""Tensor parallelism with Megatron-style sequence parallelism, on fused GEMM+collective kernels.

Reference (``crates/torsh-distributed/src/tensor_parallel.rs``): config ``tp_size, sequence_parallel,
communication_backend, async_communication`` (``:38-91``); strategies Row / Column / Vocab / Sequence /
AttentionHead with ``RowParallelLinear{input_is_parallel}``, ``ColumnParallelLinear{gather_output}``,
``ParallelEmbedding`` (``:95-137``); all-gather for row-parallel, reduce-scatter for column-parallel, sequence
parallel = all-gather of the input (``:356-405``); helpers ``split_tensor_for_tp`` / ``gather_tensor_from_tp``
(``:801-901``). The reference's forward returns the local output without any communication (``:685-737``).

Here activations between TP regions are sharded along the token dimension (``[M/tp, H]`` per rank):

* ``ColumnParallelLinear`` (weight ``[N/tp, K]``): ``Y = gather(X) Wᵀ`` runs as ONE kernel in which copy CTAs
  pull the peers' shards into local memory tile by tile while the tcgen05 GEMM CTAs start on the local
  shard (``tb_ag_gemm``). Backward: ``dX`` shard = GEMM → reduce-scatter (``tb_gemm_rs``), ``dW`` from the
  already-gathered input.
* ``RowParallelLinear`` (weight ``[N, K/tp]``): the GEMM epilogue adds every tile into the owning rank's
  buffer over NVLink (``tb_gemm_rs``), then a finalize kernel applies bias / residual. Backward: all-gather →
  GEMM on the output gradient.

CPU tensors (gloo) run the same algebra with ``torch.distributed`` collectives, which is also the oracle.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _native as nv
from ..nn.module import Module, Parameter
from ..ops import elementwise as ew
from ..ops._dispatch import call
from ..ops.gemm import EPI_BIAS, EPI_GELU, gemm
from ..ops.linear import _bgrad, _wgrad

P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64


@dataclass
class TensorParallelConfig:
    tp_size: int = 1
    sequence_parallel: bool = True
    communication_backend: str = "nvswitch"
    async_communication: bool = True
    copy_ctas: int = 0     # CTAs that pull peer shards in all-gather -> GEMM (0: 16 for two ranks, 32 beyond)
    rs_fp32: bool = False  # accumulate the reduce-scatter in fp32 (2x the NVLink bytes of bf16)
    fused: bool = True     # False: NCCL collectives + library GEMMs (the comparison arm of the benchmarks)


class TPContext:
    """Per-group state of the fused TP kernels: flags, epoch counter and symmetric staging buffers."""

    def __init__(self, group=None, config: TensorParallelConfig | None = None):
        from .symm import CommContext
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.cfg = config or TensorParallelConfig(tp_size=self.world)
        self.ctx = CommContext(self.group) if (self.cfg.fused and self.world > 1) else None
        # Pipeline schedules keep several micro-batches in flight; a column-parallel layer saves its gathered input
        # (a view of a staging buffer) for the weight gradient, so each in-flight micro-batch needs its own buffer.
        self.slot = 0
        # [go flag, done counter] of the wide-grid finalize kernel (CTA 0 releases the others after the cross-rank barrier)
        self.local_sync = torch.zeros(2, dtype=torch.int32, device="cuda") if self.ctx is not None else None
        self._bufs: dict = {}
        self._ready: dict = {}

    def staging(self, tag: str, numel: int, dtype):
        """Symmetric buffer reused across steps (allocated collectively on first use)."""
        from .symm import SymmetricBuffer
        key = (tag, numel, dtype)
        if key not in self._bufs:
            self._bufs[key] = SymmetricBuffer(numel, dtype, self.group)
        return self._bufs[key]

    def ready_flags(self, tag: str, n: int, device):
        key = (tag, n)
        if key not in self._ready:
            self._ready[key] = torch.zeros(n, dtype=torch.int32, device=device)
        return self._ready[key]


def _ag_gemm(tpc: TPContext, tag: str, x_shard: torch.Tensor, w: torch.Tensor, b_major: int, bias=None, gelu=False):
    """``gather_rows(x_shard) · op(W)ᵀ`` (+bias, +GELU); returns ``(y, x_full)``."""
    rows, K = x_shard.shape
    M = rows * tpc.world
    N = w.shape[0] if b_major == 0 else w.shape[1]
    buf = tpc.staging(tag, M * K, torch.bfloat16)
    a_full = buf.tensor.view(M, K)
    a_full[tpc.rank * rows:(tpc.rank + 1) * rows].copy_(x_shard)
    shards = (ctypes.c_void_p * 8)(*[p + r * rows * K * 2 for r, p in enumerate(buf.peer_ptrs)] + [0] * (8 - tpc.world))
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x_shard.device)
    ready = tpc.ready_flags(tag, 2 * (M // 128), x_shard.device)   # ready words, then arrival counters
    flags = (EPI_BIAS if bias is not None else 0) | (EPI_GELU if gelu else 0)
    st = nv.status_word(x_shard.device)
    call("tb_ag_gemm", [P, P, P, P, P, P, P, I, I, I, I, I, I, P, I, I, I, I, I, P, P], a_full.data_ptr(), shards,
         tpc.ctx.flags.ptr_array, tpc.ctx.epoch.data_ptr(), ready.data_ptr(), w.data_ptr(), y.data_ptr(), M, N, K,
         b_major, w.stride(0), y.stride(0), nv.ptr(bias), flags, tpc.rank, tpc.world,
         tpc.cfg.copy_ctas or (16 if tpc.world <= 2 else 32), 0,
         st.data_ptr(), nv.stream_ptr())
    return y, a_full


def _gemm_rs(tpc: TPContext, tag: str, x: torch.Tensor, w: torch.Tensor, b_major: int, bias=None, residual=None):
    """``reduce_scatter_rows(x · op(W)ᵀ)`` (+bias, +residual on the owner): returns this rank's ``[M/tp, N]``."""
    M, K = x.shape
    N = w.shape[0] if b_major == 0 else w.shape[1]
    rows = M // tpc.world
    acc_dtype = torch.float32 if tpc.cfg.rs_fp32 else torch.bfloat16
    buf = tpc.staging(tag, tpc.world * rows * N, acc_dtype)  # one slot per source rank
    st = nv.status_word(x.device)
    call("tb_gemm_rs", [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P], x.data_ptr(), w.data_ptr(), buf.ptr_array, M,
         N, K, b_major, x.stride(0), w.stride(0), N, int(tpc.cfg.rs_fp32), tpc.rank, tpc.world, 0, st.data_ptr(),
         nv.stream_ptr())
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    call("tb_rs_finalize", [P, I, I, P, P, I, P, P, P, L, I, P, P, P], tpc.ctx.flags.ptr_array, tpc.rank, tpc.world,
         tpc.ctx.epoch.data_ptr(), buf.tensor.data_ptr(), int(tpc.cfg.rs_fp32), nv.ptr(bias), nv.ptr(residual),
         out.data_ptr(), rows, N, tpc.local_sync.data_ptr(), st.data_ptr(), nv.stream_ptr())
    return out


def _fused_ok(tpc, *ts):
    return tpc is not None and tpc.world > 1 and tpc.cfg.fused and all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


class _ColumnParallelSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, weight, bias, tpc, tag, gelu):
        y, x_full = _ag_gemm(tpc, f"{tag}.fwd.s{tpc.slot}", x_shard.contiguous(), weight, 0, bias, gelu)
        assert not gelu, "use the un-fused activation with column-parallel layers that need a backward"
        ctx.save_for_backward(x_full, weight)
        ctx.tpc, ctx.tag, ctx.bias = tpc, tag, bias
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = _gemm_rs(ctx.tpc, ctx.tag + ".bwd", dy, weight, 1)
        dw = _wgrad(dy, x_full, weight, "nk")
        db = _bgrad(dy, ctx.bias) if ctx.bias is not None else None
        return dx, dw, db, None, None, None


class _RowParallelSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, tpc, tag):
        x = x.contiguous()
        y = _gemm_rs(tpc, tag + ".fwd", x, weight, 0, bias, residual)
        ctx.save_for_backward(x, weight)
        ctx.tpc, ctx.tag, ctx.bias, ctx.has_res = tpc, tag, bias, residual is not None
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x, weight = ctx.saved_tensors
        dy_shard = dy_shard.contiguous()
        dx, dy_full = _ag_gemm(ctx.tpc, ctx.tag + ".bwd", dy_shard, weight, 1)
        dw = _wgrad(dy_full, x, weight, "nk")
        db = _bgrad(dy_shard, ctx.bias) if ctx.bias is not None else None
        return dx, dw, db, (dy_shard if ctx.has_res else None), None, None


# ---- reference algebra with torch.distributed collectives (CPU path and oracle) --------------------------
def _all_gather_rows(x, group):
    w = dist.get_world_size(group)
    x = x.contiguous()
    if x.is_cuda:
        out = torch.empty(w * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    outs = [torch.empty_like(x) for _ in range(w)]
    dist.all_gather(outs, x, group=group)
    return torch.cat(outs, 0)


def _reduce_scatter_rows(x, group):
    w, r = dist.get_world_size(group), dist.get_rank(group)
    rows = x.shape[0] // w
    if x.is_cuda:
        out = torch.empty(rows, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x.contiguous(), group=group)
        return out
    x = x.contiguous().clone()          # gloo has no reduce-scatter
    dist.all_reduce(x, group=group)
    return x[r * rows:(r + 1) * rows].clone()


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _reduce_scatter_rows(dy, ctx.group), None


class _AllGatherRowsReplicated(torch.autograd.Function):
    """All-gather along tokens for a consumer that every rank evaluates in full on the gathered rows (a replicated
    head and loss): each rank's upstream gradient is already the complete one, so the backward keeps this rank's
    rows instead of summing ``world`` identical copies."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, dy):
        w, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        rows = dy.shape[0] // w
        return dy[r * rows:(r + 1) * rows].contiguous(), None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _all_gather_rows(dy, ctx.group), None


_layer_id = [0]


class ColumnParallelLinear(Module):
    """``Y[:, rank's N/tp columns] = gather(X) Wᵀ + b``; input sharded along tokens when ``sequence_parallel``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, gather_output: bool = False,
                 tp: TPContext | None = None, group=None, init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        self.tp, self.group = tp, (tp.group if tp is not None else group)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        assert out_features % self.world == 0
        self.in_features, self.out_features, self.gather_output = in_features, out_features, gather_output
        self.weight = Parameter(torch.empty(out_features // self.world, in_features, device=device, dtype=dtype).normal_(0, init_std))
        self.bias = Parameter(torch.zeros(out_features // self.world, device=device, dtype=dtype)) if bias else None
        _layer_id[0] += 1
        self.tag = f"col{_layer_id[0]}"

    def forward(self, x_shard):
        if _fused_ok(self.tp, x_shard, self.weight, self.bias) and x_shard.dim() == 2 and (x_shard.shape[0] % 128 == 0):
            y = _ColumnParallelSP.apply(x_shard, self.weight, self.bias, self.tp, self.tag, False)
        else:
            x = _AllGatherRows.apply(x_shard, self.group) if self.world > 1 else x_shard
            y = torch.nn.functional.linear(x, self.weight, self.bias)
        if self.gather_output and self.world > 1:
            y = torch.cat([t for t in _gather_cols(y, self.group)], -1)
        return y


class RowParallelLinear(Module):
    """``Y = reduce_scatter_rows(X[:, rank's K/tp columns] Wᵀ) + b`` (output sharded along tokens)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, input_is_parallel: bool = True,
                 tp: TPContext | None = None, group=None, init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        self.tp, self.group = tp, (tp.group if tp is not None else group)
        self.world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        assert in_features % self.world == 0
        self.in_features, self.out_features, self.input_is_parallel = in_features, out_features, input_is_parallel
        self.weight = Parameter(torch.empty(out_features, in_features // self.world, device=device, dtype=dtype).normal_(0, init_std))
        self.bias = Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        _layer_id[0] += 1
        self.tag = f"row{_layer_id[0]}"

    def forward(self, x, residual=None):
        if not self.input_is_parallel and self.world > 1:
            k = self.in_features // self.world
            x = x[..., self.rank * k:(self.rank + 1) * k]
        if _fused_ok(self.tp, x, self.weight, self.bias, residual) and x.dim() == 2 and x.shape[0] % (128 * self.world) == 0 \
                and self.out_features % 32 == 0:
            return _RowParallelSP.apply(x, self.weight, self.bias, residual, self.tp, self.tag)
        y = torch.nn.functional.linear(x, self.weight)
        if self.world > 1:
            y = _ReduceScatterRows.apply(y, self.group)
        if self.bias is not None:
            y = y + self.bias
        return y if residual is None else y + residual


def _gather_cols(y, group):
    outs = [torch.empty_like(y) for _ in range(dist.get_world_size(group))]
    dist.all_gather(outs, y.contiguous(), group=group)
    outs[dist.get_rank(group)] = y
    return outs


class ParallelEmbedding(Module):
    """Vocabulary-parallel embedding: each rank holds ``V/tp`` rows; out-of-range ids contribute zero and the
    partial results are summed (reduce-scattered along tokens under sequence parallelism)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, group=None, sequence_parallel: bool = True,
                 init_std: float = 0.02, device=None, dtype=None):
        super().__init__()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.per = (num_embeddings + self.world - 1) // self.world
        self.sequence_parallel = sequence_parallel
        self.weight = Parameter(torch.empty(self.per, embedding_dim, device=device, dtype=dtype).normal_(0, init_std))

    def forward(self, ids):
        lo = self.rank * self.per
        local = ids - lo
        mask = (local < 0) | (local >= self.per)
        out = torch.nn.functional.embedding(local.clamp(0, self.per - 1), self.weight)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0).reshape(-1, out.shape[-1])
        if self.world == 1:
            return out
        if self.sequence_parallel:
            return _ReduceScatterRows.apply(out, self.group)
        out = out.clone()
        dist.all_reduce(out, group=self.group)
        return out


class ParallelAttention(Module):
    """Self-attention with the heads split over the tensor-parallel group
    (``crates/torsh-distributed/src/tensor_parallel.rs:95-137``: ``ParallelAttention``, ``AttentionHead`` strategy):
    a column-parallel QKV projection laid out per rank as ``[q | k | v]`` of the local heads, attention over the local
    heads, and a row-parallel output projection. With sequence parallelism the input and the output are this rank's
    ``B*S/tp`` token rows; the all-gather sits in front of the QKV GEMM and the reduce-scatter behind the projection."""

    def __init__(self, embed_dim: int, num_heads: int, tp: TPContext | None = None, group=None, causal: bool = True,
                 bias: bool = False, init_std: float = 0.02):
        super().__init__()
        self.qkv = ColumnParallelLinear(embed_dim, 3 * embed_dim, bias=bias, tp=tp, group=group, init_std=init_std)
        self.out = RowParallelLinear(embed_dim, embed_dim, bias=bias, tp=tp, group=group, init_std=init_std)
        world = self.qkv.world
        if num_heads % world:
            raise ValueError(f"heads ({num_heads}) must divide by the tensor-parallel size ({world})")
        self.local_heads, self.head_dim, self.causal = num_heads // world, embed_dim // num_heads, causal

    def forward(self, x_shard, B: int, S: int, residual=None):
        from ..ops import attention as attn_ops
        H, D = self.local_heads, self.head_dim
        qkv = self.qkv(x_shard)                                            # [B*S, 3*H*D]: all tokens, local heads
        q, k, v = (qkv[:, i * H * D:(i + 1) * H * D].reshape(B, S, H, D) for i in range(3))
        ctx = attn_ops.flash_attention(q, k, v, causal=self.causal).reshape(B * S, H * D)
        return self.out(ctx, residual=residual)


def split_tensor_for_tp(t: torch.Tensor, dim: int, rank: int, world: int) -> torch.Tensor:
    """``crates/torsh-distributed/src/tensor_parallel.rs:801-901``."""
    return t.chunk(world, dim)[rank].contiguous()


def gather_tensor_from_tp(t: torch.Tensor, dim: int, group=None) -> torch.Tensor:
    outs = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(outs, t.contiguous(), group=group)
    return torch.cat(outs, dim)


def create_column_parallel_linear(in_features, out_features, tp=None, **kw):
    return ColumnParallelLinear(in_features, out_features, tp=tp, **kw)


def create_row_parallel_linear(in_features, out_features, tp=None, **kw):
    return RowParallelLinear(in_features, out_features, tp=tp, **kw)



class _VocabParallelCrossEntropy(torch.autograd.Function):
    """Mean cross-entropy over a vocabulary whose logits are split column-wise over the group: each rank holds
    ``logits[:, rank * Vp : (rank + 1) * Vp]``.  Three all-reduces of per-token scalars (max, sum of exponentials, target
    logit) replace the all-gather of the logits; the backward is local: ``(softmax - onehot) / tokens`` on this rank's
    columns.  Columns at or beyond ``num_classes`` (vocabulary padding) are ignored."""

    @staticmethod
    def forward(ctx, logits, targets, group, num_classes):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        T, Vp = logits.shape
        lo = rank * Vp
        lg = logits.float()
        valid = (torch.arange(Vp, device=logits.device) + lo) < num_classes
        lg = lg.masked_fill(~valid, float("-inf"))
        m = lg.max(1).values
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lg - m[:, None])
        ssum = e.sum(1)
        dist.all_reduce(ssum, group=group)
        tl = targets - lo
        mine = (tl >= 0) & (tl < Vp)
        tlogit = torch.where(mine, lg.gather(1, tl.clamp(0, Vp - 1)[:, None])[:, 0], torch.zeros_like(m))
        dist.all_reduce(tlogit, group=group)
        loss = (torch.log(ssum) + m - tlogit).mean()
        ctx.save_for_backward(e, ssum, tl, mine)
        ctx.dtype = logits.dtype
        return loss

    @staticmethod
    def backward(ctx, g):
        e, ssum, tl, mine = ctx.saved_tensors
        T, Vp = e.shape
        p = e / ssum[:, None]
        rows = torch.arange(T, device=e.device)[mine]
        p[rows, tl[mine]] -= 1.0
        return (p * (g / T)).to(ctx.dtype), None, None, None


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, targets: torch.Tensor, group=None, num_classes: int | None = None):
    group = group if group is not None else dist.group.WORLD
    V = logits_local.shape[1] * dist.get_world_size(group)
    return _VocabParallelCrossEntropy.apply(logits_local, targets.reshape(-1), group, num_classes or V)
