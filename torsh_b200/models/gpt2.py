"""GPT-2 family (causal decoder, pre-LN, learned positions, fused ``c_attn``, GELU MLP).

Presets follow ``crates/torsh-models/src/nlp/gpt2.rs:62-199`` (small 768/12/12, medium 1024/24/16,
large 1280/36/20, xl 1600/48/25; vocab 50 257, context 1024, LayerNorm eps 1e-5, init N(0, 0.02),
biases on). ``GPTForCausalLM`` is the name used by ``crates/torsh-text/src/models/gpt.rs:353``.
Parameter names are unique dotted paths (``h.3.attn.c_attn.weight``); the reference prefixes with
``_`` and collides on bare ``weight``/``bias`` keys (``gpt2.rs:447-452,796-806``) - see
:func:`reference_key` for the mapping.

The token embedding is stored with its row count padded to a multiple of 64 (50 257 → 50 304) so that
the tied LM-head GEMM and its TMA descriptors see 16-byte aligned rows; padded rows are zero, never
indexed, and the cross-entropy kernel gives their logits probability zero.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from .. import nn
from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops import linear as lin_ops
from ..ops import norm as norm_ops
from ..ops import softmax as sm_ops


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_positions: int = 1024
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_inner: int | None = None
    embd_pdrop: float = 0.1
    attn_pdrop: float = 0.1
    resid_pdrop: float = 0.1
    layer_norm_epsilon: float = 1e-5
    initializer_range: float = 0.02
    bias: bool = True
    tie_word_embeddings: bool = True

    @property
    def inner(self) -> int:
        return self.n_inner or 4 * self.n_embd

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 63) // 64 * 64

    @classmethod
    def small(cls, **kw): return cls(**{**dict(n_embd=768, n_layer=12, n_head=12), **kw})
    @classmethod
    def medium(cls, **kw): return cls(**{**dict(n_embd=1024, n_layer=24, n_head=16), **kw})
    @classmethod
    def large(cls, **kw): return cls(**{**dict(n_embd=1280, n_layer=36, n_head=20), **kw})
    @classmethod
    def xl(cls, **kw): return cls(**{**dict(n_embd=1600, n_layer=48, n_head=25), **kw})

    @classmethod
    def tiny(cls, **kw):
        """4 layers, d_model 256, 4 heads, FFN 1024, vocab 1024, context 128 (the CPU smoke configuration)."""
        base = dict(vocab_size=1024, n_positions=128, n_embd=256, n_layer=4, n_head=4, n_inner=1024, embd_pdrop=0.0,
                    attn_pdrop=0.0, resid_pdrop=0.0)
        base.update(kw)
        return cls(**base)


class _Proj(nn.Module):
    """Weight holder for a projection, ``[out, in]`` layout."""

    def __init__(self, n_in: int, n_out: int, bias: bool, std: float):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in).normal_(0.0, std))
        self.bias = nn.Parameter(torch.zeros(n_out)) if bias else None

    def forward(self, x, residual=None):
        return lin_ops.linear(x, self.weight, self.bias, residual=residual)


class GPT2Attention(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.n_head, self.head_dim = cfg.n_head, cfg.n_embd // cfg.n_head
        self.c_attn = _Proj(cfg.n_embd, 3 * cfg.n_embd, cfg.bias, cfg.initializer_range)
        self.c_proj = _Proj(cfg.n_embd, cfg.n_embd, cfg.bias, cfg.initializer_range / math.sqrt(2 * cfg.n_layer))
        self.attn_pdrop, self.resid_pdrop = cfg.attn_pdrop, cfg.resid_pdrop

    def forward(self, h, residual, B: int, S: int):
        """``h``: normalised input ``[B*S, E]``; returns ``residual + proj(attention)``."""
        qkv = self.c_attn(h)
        if self.attn_pdrop > 0 and self.training:
            E = h.shape[-1]
            q, k, v = (qkv[:, i * E:(i + 1) * E].reshape(B, S, self.n_head, self.head_dim).transpose(1, 2) for i in range(3))
            ctx = torch.nn.functional.scaled_dot_product_attention(q, k, v, dropout_p=self.attn_pdrop, is_causal=True)
            ctx = ctx.transpose(1, 2).reshape(B * S, E)
        else:
            ctx = attn_ops.flash_attention_qkvpacked(qkv, B, S, self.n_head, self.head_dim, causal=True)
        if self.resid_pdrop > 0 and self.training:
            return residual + torch.nn.functional.dropout(self.c_proj(ctx), self.resid_pdrop, True)
        return self.c_proj(ctx, residual=residual)


class GPT2MLP(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.c_fc = _Proj(cfg.n_embd, cfg.inner, cfg.bias, cfg.initializer_range)
        self.c_proj = _Proj(cfg.inner, cfg.n_embd, cfg.bias, cfg.initializer_range / math.sqrt(2 * cfg.n_layer))
        self.resid_pdrop = cfg.resid_pdrop

    def forward(self, h, residual):
        if self.resid_pdrop > 0 and self.training:
            y = lin_ops.mlp_gelu(h, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias)
            return residual + torch.nn.functional.dropout(y, self.resid_pdrop, True)
        return lin_ops.mlp_gelu(h, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias, residual)


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.ln_1 = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_epsilon)
        self.attn = GPT2Attention(cfg)
        self.ln_2 = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_epsilon)
        self.mlp = GPT2MLP(cfg)

    def forward(self, x, B: int, S: int):
        h, x = norm_ops.layer_norm_fork(x, self.ln_1.weight, self.ln_1.bias, self.ln_1.eps)
        x = self.attn(h, x, B, S)
        h, x = norm_ops.layer_norm_fork(x, self.ln_2.weight, self.ln_2.bias, self.ln_2.eps)
        return self.mlp(h, x)


class GPT2Model(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.config = cfg
        wte = torch.zeros(cfg.padded_vocab, cfg.n_embd)
        wte[: cfg.vocab_size].normal_(0.0, cfg.initializer_range)
        self.wte = nn.Parameter(wte)
        self.wpe = nn.Parameter(torch.empty(cfg.n_positions, cfg.n_embd).normal_(0.0, cfg.initializer_range))
        self.h = nn.ModuleList([GPT2Block(cfg) for _ in range(cfg.n_layer)])
        self.ln_f = nn.LayerNorm(cfg.n_embd, cfg.layer_norm_epsilon)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``[B, S]`` token ids → hidden states ``[B*S, E]`` (after the final LayerNorm)."""
        B, S = input_ids.shape
        x = ew.embedding(input_ids, self.wte, self.wpe).reshape(B * S, -1)
        if self.config.embd_pdrop > 0 and self.training:
            x = torch.nn.functional.dropout(x, self.config.embd_pdrop, True)
        for blk in self.h:
            x = blk(x, B, S)
        return self.ln_f(x)


class GPTForCausalLM(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.config = cfg
        self.transformer = GPT2Model(cfg)
        if cfg.tie_word_embeddings:
            self.lm_head_weight = None
        else:
            w = torch.zeros(cfg.padded_vocab, cfg.n_embd)
            w[: cfg.vocab_size].normal_(0.0, cfg.initializer_range)
            self.lm_head_weight = nn.Parameter(w)

    def head_weight(self) -> torch.Tensor:
        return self.transformer.wte if self.lm_head_weight is None else self.lm_head_weight

    def logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        """``[B, S, padded_vocab]``; columns ≥ ``vocab_size`` are padding."""
        B, S = input_ids.shape
        h = self.transformer(input_ids)
        return lin_ops.linear(h, self.head_weight(), None).view(B, S, -1)

    def forward(self, input_ids: torch.Tensor, targets: torch.Tensor | None = None, loss_scale: float | None = None):
        """Returns logits, or the mean next-token cross-entropy when ``targets`` (already shifted) is given.

        With ``loss_scale`` the returned loss is ``loss_scale * mean`` and must be the tensor ``backward()``
        is called on: the gradient is then produced inside the cross-entropy kernel, in place over the logits.
        """
        lg = self.logits(input_ids)
        if targets is None:
            return lg[..., : self.config.vocab_size]
        V = self.config.vocab_size
        flat = lg.view(-1, lg.shape[-1])
        if loss_scale is not None:
            return sm_ops.cross_entropy(flat, targets.reshape(-1), num_classes=V, inplace_grad=True, root_scale=loss_scale)
        return sm_ops.cross_entropy(flat, targets.reshape(-1), num_classes=V)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 1.0, top_k: int | None = None):
        for _ in range(max_new_tokens):
            ctx = input_ids[:, -self.config.n_positions:]
            lg = self.forward(ctx)[:, -1, :].float() / max(temperature, 1e-6)
            if top_k is not None:
                kth = torch.topk(lg, top_k).values[:, -1, None]
                lg = lg.masked_fill(lg < kth, float("-inf"))
            nxt = torch.multinomial(torch.softmax(lg, -1), 1) if temperature > 0 else lg.argmax(-1, keepdim=True)
            input_ids = torch.cat([input_ids, nxt], 1)
        return input_ids


GPT2LMHeadModel = GPTForCausalLM


def reference_key(name: str) -> str:
    """Dotted parameter name → the reference's underscore-prefixed key
    (``embeddings_…``, ``blocks_{i}_…``, ``ln_f_…``: ``crates/torsh-models/src/nlp/gpt2.rs:796-806``)."""
    name = name.replace("transformer.", "")
    if name in ("wte", "wpe"):
        return f"embeddings_{name}_weight"
    if name.startswith("h."):
        _, i, rest = name.split(".", 2)
        return f"blocks_{i}_{rest.replace('.', '_')}"
    return name.replace(".", "_")
