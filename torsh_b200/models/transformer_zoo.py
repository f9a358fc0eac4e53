"""Encoder-style model families: ViT, BERT / RoBERTa, T5-style encoder-decoder.

Reference inventory: ``crates/torsh-models/src/vision/mod.rs:54-87`` (ViT), ``crates/torsh-models/src/nlp`` (RoBERTa,
T5, XLNet, Longformer, BigBird compiled; BERT / BART / GPT-2 as source files), ``crates/torsh-text/src/models``
(BERT, GPT, T5, Transformer). All share one pre/post-LN encoder block built on the kernel-backed layers
(fused QKV GEMM + flash attention when no mask is given, GEMM epilogue fusions for the MLP).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import nn
from ..ops import attention as attn_ops
from ..ops import linear as lin_ops


@dataclass
class EncoderConfig:
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    intermediate_size: int = 3072
    dropout: float = 0.1
    layer_norm_eps: float = 1e-12
    pre_norm: bool = False
    activation: str = "gelu"


class EncoderBlock(nn.Module):
    def __init__(self, cfg: EncoderConfig, cross_attention: bool = False, causal: bool = False):
        super().__init__()
        E = cfg.hidden_size
        self.cfg, self.causal = cfg, causal
        self.attn = nn.MultiheadAttention(E, cfg.num_heads, dropout=cfg.dropout, batch_first=True)
        self.ln1 = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.cross = nn.MultiheadAttention(E, cfg.num_heads, dropout=cfg.dropout, batch_first=True) if cross_attention else None
        self.ln_c = nn.LayerNorm(E, cfg.layer_norm_eps) if cross_attention else None
        self.fc1 = nn.Linear(E, cfg.intermediate_size)
        self.fc2 = nn.Linear(cfg.intermediate_size, E)
        self.ln2 = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.drop = nn.Dropout(cfg.dropout)

    def _mlp(self, x):
        if self.cfg.activation == "gelu" and not (self.training and self.cfg.dropout > 0):
            return lin_ops.mlp_gelu(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias)
        act = {"gelu": torch.nn.functional.gelu, "relu": torch.relu, "silu": torch.nn.functional.silu,
               "quick_gelu": lambda t: t * torch.sigmoid(1.702 * t)}[self.cfg.activation]
        return self.fc2(self.drop(act(self.fc1(x))))

    def forward(self, x, key_padding_mask=None, memory=None, memory_mask=None):
        pre = self.cfg.pre_norm
        h = self.ln1(x) if pre else x
        a, _ = self.attn(h, key_padding_mask=key_padding_mask, is_causal=self.causal)
        x = x + self.drop(a)
        if not pre:
            x = self.ln1(x)
        if self.cross is not None and memory is not None:
            h = self.ln_c(x) if pre else x
            a, _ = self.cross(h, memory, memory, key_padding_mask=memory_mask)
            x = x + self.drop(a)
            if not pre:
                x = self.ln_c(x)
        h = self.ln2(x) if pre else x
        x = x + self.drop(self._mlp(h))
        return x if pre else self.ln2(x)


# ---------------------------------------------------------------------------------------------- ViT
@dataclass
class ViTConfig(EncoderConfig):
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    num_classes: int = 1000
    pre_norm: bool = True
    layer_norm_eps: float = 1e-6
    dropout: float = 0.0

    @classmethod
    def vit_b_16(cls, **kw): return cls(**kw)
    @classmethod
    def vit_l_16(cls, **kw): return cls(hidden_size=1024, num_layers=24, num_heads=16, intermediate_size=4096, **kw)
    @classmethod
    def vit_tiny(cls, **kw):
        d = dict(hidden_size=192, num_layers=4, num_heads=3, intermediate_size=768, image_size=32, patch_size=8, num_classes=10)
        d.update(kw)
        return cls(**d)


class VisionTransformer(nn.Module):
    def __init__(self, cfg: ViTConfig | None = None):
        super().__init__()
        cfg = cfg or ViTConfig()
        self.config = cfg
        E = cfg.hidden_size
        n = (cfg.image_size // cfg.patch_size) ** 2
        self.patch_embed = nn.Conv2d(cfg.num_channels, E, cfg.patch_size, cfg.patch_size)
        self.cls_token = nn.Parameter(torch.zeros(1, 1, E))
        self.pos_embed = nn.Parameter(torch.empty(1, n + 1, E).normal_(0, 0.02))
        self.blocks = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.norm = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.head = nn.Linear(E, cfg.num_classes)

    def forward(self, x):
        x = self.patch_embed(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], 1) + self.pos_embed.to(x.dtype)
        for b in self.blocks:
            x = b(x)
        return self.head(self.norm(x)[:, 0])


# ---------------------------------------------------------------------------------------------- BERT
@dataclass
class BertConfig(EncoderConfig):
    vocab_size: int = 30522
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    pad_token_id: int = 0

    @classmethod
    def bert_base(cls, **kw): return cls(**kw)
    @classmethod
    def bert_large(cls, **kw): return cls(hidden_size=1024, num_layers=24, num_heads=16, intermediate_size=4096, **kw)
    @classmethod
    def roberta_base(cls, **kw): return cls(vocab_size=50265, max_position_embeddings=514, type_vocab_size=1, pad_token_id=1, layer_norm_eps=1e-5, **kw)
    @classmethod
    def tiny(cls, **kw):
        d = dict(vocab_size=1000, hidden_size=128, num_layers=2, num_heads=4, intermediate_size=256, max_position_embeddings=128)
        d.update(kw)
        return cls(**d)


class BertModel(nn.Module):
    def __init__(self, cfg: BertConfig | None = None):
        super().__init__()
        cfg = cfg or BertConfig()
        self.config = cfg
        E = cfg.hidden_size
        self.word_embeddings = nn.Embedding(cfg.vocab_size, E, padding_idx=cfg.pad_token_id)
        self.position_embeddings = nn.Embedding(cfg.max_position_embeddings, E)
        self.token_type_embeddings = nn.Embedding(cfg.type_vocab_size, E)
        self.emb_norm = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.drop = nn.Dropout(cfg.dropout)
        self.layers = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.pooler = nn.Linear(E, E)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        B, S = input_ids.shape
        pos = torch.arange(S, device=input_ids.device)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = self.word_embeddings(input_ids) + self.position_embeddings(pos)[None] + self.token_type_embeddings(tt)
        x = self.drop(self.emb_norm(x))
        kpm = (attention_mask == 0) if attention_mask is not None else None
        for l in self.layers:
            x = l(x, key_padding_mask=kpm)
        return x, torch.tanh(self.pooler(x[:, 0]))


class BertForMaskedLM(nn.Module):
    def __init__(self, cfg: BertConfig | None = None):
        super().__init__()
        self.bert = BertModel(cfg)
        E = self.bert.config.hidden_size
        self.transform = nn.Linear(E, E)
        self.norm = nn.LayerNorm(E, self.bert.config.layer_norm_eps)
        self.bias = nn.Parameter(torch.zeros(self.bert.config.vocab_size))

    def forward(self, input_ids, labels=None, **kw):
        h, _ = self.bert(input_ids, **kw)
        h = self.norm(torch.nn.functional.gelu(self.transform(h)))
        logits = torch.nn.functional.linear(h, self.bert.word_embeddings.weight, self.bias)
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.view(-1), ignore_index=-100)


class BertForSequenceClassification(nn.Module):
    def __init__(self, cfg: BertConfig | None = None, num_labels: int = 2):
        super().__init__()
        self.bert = BertModel(cfg)
        self.drop = nn.Dropout(self.bert.config.dropout)
        self.classifier = nn.Linear(self.bert.config.hidden_size, num_labels)

    def forward(self, input_ids, labels=None, **kw):
        _, pooled = self.bert(input_ids, **kw)
        logits = self.classifier(self.drop(pooled))
        return logits if labels is None else torch.nn.functional.cross_entropy(logits.float(), labels)


RobertaModel = BertModel


# ---------------------------------------------------------------------------------------------- T5-style
@dataclass
class Seq2SeqConfig(EncoderConfig):
    vocab_size: int = 32128
    num_decoder_layers: int = 12
    max_position_embeddings: int = 512
    pre_norm: bool = True
    layer_norm_eps: float = 1e-6
    activation: str = "relu"

    @classmethod
    def tiny(cls, **kw):
        d = dict(vocab_size=1000, hidden_size=128, num_layers=2, num_decoder_layers=2, num_heads=4, intermediate_size=256)
        d.update(kw)
        return cls(**d)


class EncoderDecoderModel(nn.Module):
    """Pre-LN encoder-decoder with learned positions and a tied output embedding (T5 / BART family shape)."""

    def __init__(self, cfg: Seq2SeqConfig | None = None):
        super().__init__()
        cfg = cfg or Seq2SeqConfig()
        self.config = cfg
        E = cfg.hidden_size
        self.shared = nn.Embedding(cfg.vocab_size, E)
        self.pos = nn.Embedding(cfg.max_position_embeddings, E)
        self.encoder = nn.ModuleList([EncoderBlock(cfg) for _ in range(cfg.num_layers)])
        self.decoder = nn.ModuleList([EncoderBlock(cfg, cross_attention=True, causal=True) for _ in range(cfg.num_decoder_layers)])
        self.enc_norm = nn.LayerNorm(E, cfg.layer_norm_eps)
        self.dec_norm = nn.LayerNorm(E, cfg.layer_norm_eps)

    def _embed(self, ids):
        return self.shared(ids) + self.pos(torch.arange(ids.shape[1], device=ids.device))[None]

    def encode(self, input_ids, attention_mask=None):
        x = self._embed(input_ids)
        kpm = (attention_mask == 0) if attention_mask is not None else None
        for l in self.encoder:
            x = l(x, key_padding_mask=kpm)
        return self.enc_norm(x)

    def forward(self, input_ids, decoder_input_ids, attention_mask=None, labels=None):
        mem = self.encode(input_ids, attention_mask)
        mm = (attention_mask == 0) if attention_mask is not None else None
        y = self._embed(decoder_input_ids)
        for l in self.decoder:
            y = l(y, memory=mem, memory_mask=mm)
        logits = torch.nn.functional.linear(self.dec_norm(y), self.shared.weight) / math.sqrt(self.config.hidden_size)
        if labels is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]).float(), labels.view(-1), ignore_index=-100)


T5Model = EncoderDecoderModel
