"""Embedding layers for text models: word embeddings (random, Xavier or loaded from GloVe / word2vec text files),
sinusoidal and learnable positional encodings, token-type embeddings, their BERT-style combination, and similarity
utilities. Reference: crates/torsh-text/src/embeddings.rs.
"""
from __future__ import annotations

import math
from pathlib import Path

import torch
from torch import nn


class WordEmbedding(nn.Module):
    def __init__(self, vocab_size: int, dim: int, padding_idx: int | None = None, scale_by_sqrt_dim: bool = False):
        super().__init__()
        self.emb = nn.Embedding(vocab_size, dim, padding_idx=padding_idx)
        self.scale = math.sqrt(dim) if scale_by_sqrt_dim else 1.0

    @classmethod
    def from_pretrained(cls, weights: torch.Tensor, freeze: bool = True, padding_idx: int | None = None) -> "WordEmbedding":
        m = cls(weights.shape[0], weights.shape[1], padding_idx)
        m.emb.weight.data.copy_(weights)
        m.emb.weight.requires_grad_(not freeze)
        return m

    def forward(self, ids):
        from ..ops import elementwise as ew
        w = self.emb.weight
        if ids.is_cuda and w.dtype == torch.bfloat16 and self.emb.padding_idx is None:
            return ew.embedding(ids, w) * self.scale if self.scale != 1.0 else ew.embedding(ids, w)
        return self.emb(ids) * self.scale


class PositionalEncoding(nn.Module):
    """Fixed sinusoidal table added to the input (``[..., T, D]``), with dropout."""

    def __init__(self, dim: int, max_len: int = 5000, dropout: float = 0.0):
        super().__init__()
        pos = torch.arange(max_len)[:, None].float()
        div = torch.exp(torch.arange(0, dim, 2).float() * (-math.log(10000.0) / dim))
        pe = torch.zeros(max_len, dim)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div[: dim // 2])
        self.register_buffer("pe", pe)
        self.drop = nn.Dropout(dropout)

    def forward(self, x, offset: int = 0):
        return self.drop(x + self.pe[offset:offset + x.shape[-2]].to(x.dtype))


class LearnablePositionalEncoding(nn.Module):
    def __init__(self, dim: int, max_len: int = 512):
        super().__init__()
        self.emb = nn.Embedding(max_len, dim)

    def forward(self, x, offset: int = 0):
        pos = torch.arange(offset, offset + x.shape[-2], device=x.device)
        return x + self.emb(pos).to(x.dtype)


class TokenTypeEmbedding(nn.Module):
    def __init__(self, num_types: int, dim: int):
        super().__init__()
        self.emb = nn.Embedding(num_types, dim)

    def forward(self, type_ids):
        return self.emb(type_ids)


class CombinedEmbeddings(nn.Module):
    """word + position (+ token type) -> LayerNorm -> dropout, as in BERT."""

    def __init__(self, vocab_size: int, dim: int, max_len: int = 512, num_types: int = 2, dropout: float = 0.1, eps: float = 1e-12,
                 padding_idx: int | None = None, learnable_positions: bool = True):
        super().__init__()
        self.word = WordEmbedding(vocab_size, dim, padding_idx)
        self.pos = LearnablePositionalEncoding(dim, max_len) if learnable_positions else PositionalEncoding(dim, max_len)
        self.types = TokenTypeEmbedding(num_types, dim) if num_types else None
        self.norm = nn.LayerNorm(dim, eps=eps)
        self.drop = nn.Dropout(dropout)

    def forward(self, ids, token_type_ids=None, position_offset: int = 0):
        x = self.pos(self.word(ids), position_offset)
        if self.types is not None:
            tt = token_type_ids if token_type_ids is not None else torch.zeros_like(ids)
            x = x + self.types(tt).to(x.dtype)
        return self.drop(self.norm(x))

    forward_with_positions_and_types = forward


class EmbeddingUtils:
    @staticmethod
    def load_pretrained_embeddings(path, vocab=None, dim: int | None = None):
        """Reads a GloVe / word2vec *text* file (``token v1 v2 ...`` per line; an optional ``count dim`` header is
        skipped). With ``vocab`` returns a ``[len(vocab), D]`` matrix whose rows for missing tokens are N(0, 0.1); without
        it returns ``(tokens, matrix)``."""
        toks, vecs = [], []
        for k, ln in enumerate(Path(path).read_text(encoding="utf-8").splitlines()):
            parts = ln.rstrip().split(" ")
            if k == 0 and len(parts) == 2 and all(p.isdigit() for p in parts):
                continue
            if len(parts) < 2:
                continue
            if dim is not None and len(parts) - 1 != dim:
                continue
            toks.append(parts[0])
            vecs.append([float(v) for v in parts[1:]])
        mat = torch.tensor(vecs, dtype=torch.float32)
        if vocab is None:
            return toks, mat
        out = torch.randn(len(vocab), mat.shape[1]) * 0.1
        idx = {t: i for i, t in enumerate(toks)}
        found = 0
        for i, t in enumerate(vocab.itos):
            if t in idx:
                out[i] = mat[idx[t]]
                found += 1
        out.found = found
        return out

    @staticmethod
    def xavier_uniform_embeddings(vocab_size: int, dim: int) -> torch.Tensor:
        return nn.init.xavier_uniform_(torch.empty(vocab_size, dim))

    @staticmethod
    def xavier_normal_embeddings(vocab_size: int, dim: int) -> torch.Tensor:
        return nn.init.xavier_normal_(torch.empty(vocab_size, dim))

    @staticmethod
    def cosine_similarity(embeddings: torch.Tensor, idx1: int, idx2: int) -> float:
        return float(torch.nn.functional.cosine_similarity(embeddings[idx1].float(), embeddings[idx2].float(), dim=0))

    @staticmethod
    def most_similar(embeddings: torch.Tensor, idx: int, k: int = 5) -> list[tuple[int, float]]:
        e = torch.nn.functional.normalize(embeddings.float(), dim=-1)
        sim = e @ e[idx]
        sim[idx] = -2.0
        v, i = sim.topk(min(k, e.shape[0] - 1))
        return list(zip(i.tolist(), v.tolist()))
