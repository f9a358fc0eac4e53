"""Text utilities (``crates/torsh-text``): vocabulary, whitespace / character / BPE / WordPiece tokenizers, generation
helpers (greedy, top-k / top-p sampling, beam search)."""
from __future__ import annotations

import collections
import math
import re

import torch


class Vocab:
    def __init__(self, tokens=(), specials=("<pad>", "<unk>", "<bos>", "<eos>")):
        self.itos = list(specials) + [t for t in tokens if t not in specials]
        self.stoi = {t: i for i, t in enumerate(self.itos)}
        self.unk = self.stoi.get("<unk>", 0)

    @classmethod
    def build(cls, texts, min_freq: int = 1, max_size: int | None = None, tokenizer=str.split, **kw):
        c = collections.Counter(t for s in texts for t in tokenizer(s))
        toks = [t for t, n in c.most_common(max_size) if n >= min_freq]
        return cls(toks, **kw)

    def __len__(self): return len(self.itos)
    def __getitem__(self, tok): return self.stoi.get(tok, self.unk)
    def encode(self, tokens): return [self[t] for t in tokens]
    def decode(self, ids): return [self.itos[i] for i in ids]


class WhitespaceTokenizer:
    def tokenize(self, s: str): return s.split()
    __call__ = tokenize


class CharTokenizer:
    def tokenize(self, s: str): return list(s)
    __call__ = tokenize


class BPETokenizer:
    """Byte-pair encoding trained on a corpus (merges learned greedily by pair frequency)."""

    def __init__(self, merges=None):
        self.merges = list(merges or [])
        self.ranks = {m: i for i, m in enumerate(self.merges)}

    @classmethod
    def train(cls, texts, num_merges: int = 100):
        words = collections.Counter(tuple(w) + ("</w>",) for s in texts for w in s.split())
        merges = []
        for _ in range(num_merges):
            pairs = collections.Counter()
            for w, n in words.items():
                for a, b in zip(w, w[1:]):
                    pairs[(a, b)] += n
            if not pairs:
                break
            best = max(pairs, key=lambda p: (pairs[p], p))
            merges.append(best)
            new = {}
            for w, n in words.items():
                out, i = [], 0
                while i < len(w):
                    if i + 1 < len(w) and (w[i], w[i + 1]) == best:
                        out.append(w[i] + w[i + 1]); i += 2
                    else:
                        out.append(w[i]); i += 1
                new[tuple(out)] = new.get(tuple(out), 0) + n
            words = new
        return cls(merges)

    def _word(self, w: str):
        sym = list(w) + ["</w>"]
        while len(sym) > 1:
            cand = [(self.ranks.get((a, b), math.inf), i) for i, (a, b) in enumerate(zip(sym, sym[1:]))]
            r, i = min(cand)
            if r == math.inf:
                break
            sym[i:i + 2] = [sym[i] + sym[i + 1]]
        return sym

    def tokenize(self, s: str):
        return [t for w in s.split() for t in self._word(w)]
    __call__ = tokenize


class WordPieceTokenizer:
    def __init__(self, vocab: Vocab, unk="<unk>", prefix="##", max_chars=100):
        self.vocab, self.unk, self.prefix, self.max_chars = vocab, unk, prefix, max_chars

    def tokenize(self, s: str):
        out = []
        for w in re.findall(r"\w+|[^\w\s]", s.lower()):
            if len(w) > self.max_chars:
                out.append(self.unk); continue
            i, pieces = 0, []
            while i < len(w):
                j, cur = len(w), None
                while i < j:
                    sub = (self.prefix if i else "") + w[i:j]
                    if sub in self.vocab.stoi:
                        cur = sub; break
                    j -= 1
                if cur is None:
                    pieces = [self.unk]; break
                pieces.append(cur); i = j
            out += pieces
        return out
    __call__ = tokenize


def top_k_top_p_filter(logits: torch.Tensor, top_k: int = 0, top_p: float = 1.0) -> torch.Tensor:
    logits = logits.clone()
    if top_k > 0:
        kth = logits.topk(min(top_k, logits.shape[-1])).values[..., -1, None]
        logits[logits < kth] = float("-inf")
    if top_p < 1.0:
        s, idx = logits.sort(descending=True)
        cum = torch.softmax(s, -1).cumsum(-1)
        drop = cum - torch.softmax(s, -1) > top_p
        s[drop] = float("-inf")
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, s)
    return logits


@torch.no_grad()
def beam_search(step_fn, start_ids: torch.Tensor, beam: int = 4, max_new: int = 20, eos: int | None = None, length_penalty: float = 1.0):
    """``step_fn(ids [N, T]) -> logits [N, V]`` for the last position. Returns the best sequence (1-D tensor)."""
    beams = [(start_ids.reshape(1, -1), 0.0, False)]
    for _ in range(max_new):
        cand = []
        for ids, score, done in beams:
            if done:
                cand.append((ids, score, True)); continue
            lp = torch.log_softmax(step_fn(ids).float(), -1)[0]
            v, i = lp.topk(beam)
            for vv, ii in zip(v.tolist(), i.tolist()):
                cand.append((torch.cat([ids, torch.tensor([[ii]], device=ids.device)], 1), score + vv, eos is not None and ii == eos))
        cand.sort(key=lambda c: -c[1] / (c[0].shape[1] ** length_penalty))
        beams = cand[:beam]
        if all(d for _, _, d in beams):
            break
    return beams[0][0][0]


class SentencePieceTokenizer:
    """Unigram / BPE sub-word tokenizer backed by the ``sentencepiece`` package
    (``crates/torsh-text/src/tokenization``: SentencePiece): ``train`` writes a model from raw text, ``encode`` /
    ``decode`` use it. Raises ``ImportError`` with the package name when it is missing."""

    def __init__(self, model_file: str | None = None, model_proto: bytes | None = None):
        import sentencepiece as spm
        self.sp = spm.SentencePieceProcessor(model_file=model_file, model_proto=model_proto)

    @classmethod
    def train(cls, texts, vocab_size: int = 256, model_type: str = "unigram", model_prefix: str | None = None, **kw):
        import io
        import sentencepiece as spm
        buf = io.BytesIO()
        spm.SentencePieceTrainer.train(sentence_iterator=iter(texts), model_writer=buf, vocab_size=vocab_size,
                                       model_type=model_type, hard_vocab_limit=False, minloglevel=2, **kw)
        if model_prefix:
            with open(model_prefix + ".model", "wb") as f:
                f.write(buf.getvalue())
        return cls(model_proto=buf.getvalue())

    @property
    def vocab_size(self) -> int:
        return self.sp.get_piece_size()

    def encode(self, text: str, add_bos: bool = False, add_eos: bool = False) -> list[int]:
        ids = self.sp.encode(text)
        return ([self.sp.bos_id()] if add_bos and self.sp.bos_id() >= 0 else []) + ids + \
            ([self.sp.eos_id()] if add_eos and self.sp.eos_id() >= 0 else [])

    def decode(self, ids) -> str:
        return self.sp.decode([int(i) for i in ids])

    def tokenize(self, text: str) -> list[str]:
        return self.sp.encode(text, out_type=str)
