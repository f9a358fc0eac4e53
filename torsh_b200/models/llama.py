"""Llama-style decoder (RMSNorm, rotary positions, SwiGLU FFN, no biases), optionally tensor-parallel with
sequence parallelism.

Shapes of the 7B configuration named by the benchmark set: 32 layers, d_model 4096, 32 heads, FFN 11008,
vocab 32000, RoPE θ = 1e4, RMSNorm eps 1e-6. The building blocks follow the reference layers
(``RMSNorm``: ``crates/torsh-nn/src/layers/normalization/layer_group/mod.rs:491-514``; ``SwiGLU`` with the gate in
the second half: ``layers/activation/gated.rs:536-608``; ``RotaryPositionalEmbedding``: ``layers/embedding.rs:372-430``).
With a :class:`~torsh_b200.parallel.tensor_parallel.TPContext` the projections are Column/RowParallelLinear
(fused all-gather→GEMM and GEMM→reduce-scatter) and activations between blocks stay sharded along tokens.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import linear as lin_ops
from ..ops import norm as norm_ops
from ..ops import softmax as sm_ops


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_layers: int = 32
    num_heads: int = 32
    max_seq_len: int = 4096
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    initializer_range: float = 0.02

    @classmethod
    def llama_7b(cls, **kw):
        return cls(**kw)

    @classmethod
    def tiny(cls, **kw):
        base = dict(vocab_size=1024, hidden_size=256, intermediate_size=768, num_layers=2, num_heads=4, max_seq_len=256)
        base.update(kw)
        return cls(**base)

    @property
    def head_dim(self):
        return self.hidden_size // self.num_heads

    @property
    def padded_vocab(self):
        return (self.vocab_size + 63) // 64 * 64


class _W(nn.Module):
    def __init__(self, n_out, n_in, std):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in).normal_(0.0, std))

    def forward(self, x, residual=None):
        return lin_ops.linear(x, self.weight, None, residual=residual)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, tp=None):
        super().__init__()
        self.cfg, self.tp = cfg, tp
        E, F, std = cfg.hidden_size, cfg.intermediate_size, cfg.initializer_range
        self.world = tp.world if tp is not None else 1
        self.local_heads = cfg.num_heads // self.world
        self.input_norm = nn.RMSNorm(E, cfg.rms_eps)
        self.post_attn_norm = nn.RMSNorm(E, cfg.rms_eps)
        if tp is None:
            self.qkv, self.o = _W(3 * E, E, std), _W(E, E, std / math.sqrt(2 * cfg.num_layers))
            self.gate_up, self.down = _W(2 * F, E, std), _W(E, F, std / math.sqrt(2 * cfg.num_layers))
        else:
            from ..parallel.tensor_parallel import ColumnParallelLinear, RowParallelLinear
            # column-parallel outputs are laid out per rank as [q | k | v] of the local heads and [up | gate] of the
            # local FFN slice, so no re-shuffle is needed after the GEMM
            self.qkv = ColumnParallelLinear(E, 3 * E, bias=False, tp=tp, init_std=std)
            self.o = RowParallelLinear(E, E, bias=False, tp=tp, init_std=std / math.sqrt(2 * cfg.num_layers))
            self.gate_up = ColumnParallelLinear(E, 2 * F, bias=False, tp=tp, init_std=std)
            self.down = RowParallelLinear(F, E, bias=False, tp=tp, init_std=std / math.sqrt(2 * cfg.num_layers))

    def forward(self, x, B: int, S: int):
        """``x``: ``[B*S, E]`` (or this rank's ``[B*S/tp, E]`` token shard under TP+SP)."""
        cfg, H, D = self.cfg, self.local_heads, self.cfg.head_dim
        h, x = norm_ops.rms_norm_fork(x, self.input_norm.weight, cfg.rms_eps)
        qkv = self.qkv(h)                                        # [B*S, 3*H*D] (all tokens, local heads)
        E_loc = H * D
        q = ew.rope(qkv[:, :E_loc].reshape(B, S, H, D), cfg.rope_theta)
        k = ew.rope(qkv[:, E_loc:2 * E_loc].reshape(B, S, H, D), cfg.rope_theta)
        v = qkv[:, 2 * E_loc:].reshape(B, S, H, D)
        ctx = attn_ops.flash_attention(q, k, v, causal=True).reshape(B * S, E_loc)
        x = self.o(ctx, residual=x)
        h, x = norm_ops.rms_norm_fork(x, self.post_attn_norm.weight, cfg.rms_eps)
        return self.down(ew.swiglu(self.gate_up(h)), residual=x)


class LlamaModel(nn.Module):
    """Whole model, or one pipeline stage of it (``layer_range``; first stage owns the embedding, last stage the
    final norm and the LM head)."""

    def __init__(self, cfg: LlamaConfig, tp=None, layer_range: range | None = None, first_stage: bool = True,
                 last_stage: bool = True, vocab_parallel: bool = False):
        super().__init__()
        self.cfg, self.tp, self.first_stage, self.last_stage = cfg, tp, first_stage, last_stage
        # vocab_parallel: the LM head is split over the tensor-parallel ranks by vocabulary rows (column-parallel
        # linear fed by the token shards) and the loss is computed without gathering the logits; otherwise every
        # rank computes all logits from the gathered hidden states
        self.vocab_parallel = bool(vocab_parallel and tp is not None and tp.world > 1)
        layers = layer_range if layer_range is not None else range(cfg.num_layers)
        if first_stage:
            w = torch.zeros(cfg.padded_vocab, cfg.hidden_size)
            w[: cfg.vocab_size].normal_(0.0, cfg.initializer_range)
            self.embed = nn.Parameter(w)
        self.layers = nn.ModuleList([LlamaBlock(cfg, tp) for _ in layers])
        if last_stage:
            self.norm = nn.RMSNorm(cfg.hidden_size, cfg.rms_eps)
            if self.vocab_parallel:
                from ..parallel.tensor_parallel import ColumnParallelLinear
                vp = (cfg.vocab_size + 128 * tp.world - 1) // (128 * tp.world) * (128 * tp.world)
                self.lm_head_tp = ColumnParallelLinear(cfg.hidden_size, vp, bias=False, tp=tp, init_std=cfg.initializer_range)
            else:
                w = torch.zeros(cfg.padded_vocab, cfg.hidden_size)
                w[: cfg.vocab_size].normal_(0.0, cfg.initializer_range)
                self.lm_head = nn.Parameter(w)

    def replicated_parameters(self):
        """Parameters every tensor-parallel rank holds in full but feeds with its own token shard (norm weights, the
        embedding): their gradients are partial sums and must be all-reduced over the TP group."""
        out = [p for n, p in self.named_parameters() if "norm" in n]
        if self.first_stage:
            out.append(self.embed)
        return out

    def _shard_tokens(self, x):
        if self.tp is None or self.tp.world == 1:
            return x
        rows = x.shape[0] // self.tp.world
        return x[self.tp.rank * rows:(self.tp.rank + 1) * rows].contiguous()

    def forward(self, inp: torch.Tensor, B: int | None = None, S: int | None = None, targets: torch.Tensor | None = None):
        """First stage: ``inp`` = token ids ``[B, S]``. Later stages: hidden states from the previous stage."""
        if self.first_stage:
            B, S = inp.shape
            x = self._shard_tokens(ew.embedding(inp, self.embed).reshape(B * S, -1))
        else:
            x = inp
        for blk in self.layers:
            x = blk(x, B, S)
        if not self.last_stage:
            return x
        return self.head(x, B, S, targets)

    def head(self, x, B: int, S: int, targets: torch.Tensor | None = None):
        """Final norm + LM head (+ fused cross-entropy when ``targets`` is given) on the last stage's hidden states."""
        h = norm_ops.rms_norm(x, self.norm.weight, self.cfg.rms_eps)
        if self.vocab_parallel:
            from ..parallel.tensor_parallel import _gather_cols, vocab_parallel_cross_entropy
            logits_local = self.lm_head_tp(h)                       # [B*S, V/tp]: all tokens, this rank's vocabulary rows
            if targets is None:
                full = torch.cat(_gather_cols(logits_local, self.tp.group), -1)
                return full.view(B, S, -1)[..., : self.cfg.vocab_size]
            return vocab_parallel_cross_entropy(logits_local, targets, self.tp.group, self.cfg.vocab_size)
        if self.tp is not None and self.tp.world > 1:
            from ..parallel.tensor_parallel import _AllGatherRowsReplicated
            h = _AllGatherRowsReplicated.apply(h, self.tp.group)
        logits = lin_ops.linear(h, self.lm_head, None)
        if targets is None:
            return logits.view(B, S, -1)[..., : self.cfg.vocab_size]
        return sm_ops.cross_entropy(logits, targets.reshape(-1), num_classes=self.cfg.vocab_size)


LlamaForCausalLM = LlamaModel
