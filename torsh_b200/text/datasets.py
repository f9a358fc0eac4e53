"""Text datasets: line / CSV / TSV / JSONL classification sets, language-modelling token blocks, parallel translation
corpora, CoNLL-style sequence labelling, a preprocessing pipeline, padded / bucketed batch iteration and an in-memory
cache; loaders for the standard on-disk layouts of AG News, IMDB, WikiText and Multi30k (read from a local directory: the
library never downloads). Reference: crates/torsh-text/src/datasets/*.rs.
"""
from __future__ import annotations

import csv
import json
import os
import random
from dataclasses import dataclass, field
from pathlib import Path

import torch


@dataclass
class PreprocessingConfig:
    lowercase: bool = True
    strip: bool = True
    collapse_whitespace: bool = True
    max_length: int | None = None           # in tokens, applied after tokenisation
    remove_empty: bool = True


class PreprocessingPipeline:
    """Text normalisation steps followed by an optional tokenizer and vocabulary lookup."""

    def __init__(self, config: PreprocessingConfig | None = None, tokenizer=None, vocab=None, extra_steps=()):
        self.cfg, self.tokenizer, self.vocab, self.extra = config or PreprocessingConfig(), tokenizer, vocab, list(extra_steps)

    def normalize(self, text: str) -> str:
        c = self.cfg
        if c.strip:
            text = text.strip()
        if c.lowercase:
            text = text.lower()
        if c.collapse_whitespace:
            text = " ".join(text.split())
        for f in self.extra:
            text = f(text)
        return text

    def __call__(self, text: str):
        text = self.normalize(text)
        if self.tokenizer is None:
            return text
        toks = self.tokenizer(text)
        if self.cfg.max_length is not None:
            toks = toks[:self.cfg.max_length]
        if self.vocab is None:
            return toks
        return [self.vocab[t] if hasattr(self.vocab, "__getitem__") else self.vocab.lookup(t) for t in toks]


class TextDataset(torch.utils.data.Dataset):
    """One example per line of a text file (or from a list of strings)."""

    def __init__(self, source, pipeline: PreprocessingPipeline | None = None):
        lines = Path(source).read_text(encoding="utf-8").splitlines() if isinstance(source, (str, os.PathLike)) else list(source)
        self.pipeline = pipeline
        keep_empty = pipeline is not None and not pipeline.cfg.remove_empty
        self.items = [ln for ln in lines if ln.strip() or keep_empty]

    def __len__(self): return len(self.items)
    def __getitem__(self, i): return self.pipeline(self.items[i]) if self.pipeline else self.items[i]


@dataclass
class ColumnMapping:
    text: str | int = "text"
    label: str | int = "label"
    text_pair: str | int | None = None


class ClassificationDataset(torch.utils.data.Dataset):
    """(text, label) pairs from CSV / TSV (with or without a header) or JSON lines; labels are mapped to 0..C-1."""

    def __init__(self, path, columns: ColumnMapping | None = None, fmt: str | None = None, pipeline=None, has_header: bool = True,
                 label_names: list | None = None):
        path = Path(path)
        fmt = fmt or {".csv": "csv", ".tsv": "tsv", ".jsonl": "jsonl", ".json": "jsonl"}.get(path.suffix, "csv")
        cols = columns or ColumnMapping()
        rows = []
        if fmt == "jsonl":
            for ln in path.read_text(encoding="utf-8").splitlines():
                if ln.strip():
                    rows.append(json.loads(ln))
        else:
            with open(path, newline="", encoding="utf-8") as f:
                rd = csv.reader(f, delimiter="\t" if fmt == "tsv" else ",")
                data = list(rd)
            if has_header and isinstance(cols.text, str):
                head, data = data[0], data[1:]
                rows = [dict(zip(head, r)) for r in data]
            else:
                rows = [dict(enumerate(r)) for r in (data[1:] if has_header else data)]
        self.texts = [r[cols.text] for r in rows]
        self.pairs = [r[cols.text_pair] for r in rows] if cols.text_pair is not None else None
        raw = [r[cols.label] for r in rows]
        self.label_names = label_names or sorted(set(raw), key=str)
        idx = {n: i for i, n in enumerate(self.label_names)}
        self.labels = [idx[x] for x in raw]
        self.pipeline = pipeline

    @property
    def num_classes(self): return len(self.label_names)
    def __len__(self): return len(self.texts)

    def __getitem__(self, i):
        t = self.pipeline(self.texts[i]) if self.pipeline else self.texts[i]
        if self.pairs is not None:
            p = self.pipeline(self.pairs[i]) if self.pipeline else self.pairs[i]
            return t, p, self.labels[i]
        return t, self.labels[i]


class LanguageModelingDataset(torch.utils.data.Dataset):
    """A token stream cut into blocks of ``block_size + 1``: item i is (inputs, targets) shifted by one."""

    def __init__(self, token_ids, block_size: int, stride: int | None = None):
        self.ids = torch.as_tensor(token_ids, dtype=torch.long)
        self.block, self.stride = block_size, stride or block_size
        self.n = max((len(self.ids) - block_size - 1) // self.stride + 1, 0)

    @classmethod
    def from_text(cls, text: str, tokenizer, vocab, block_size: int, stride: int | None = None):
        return cls([vocab[t] for t in tokenizer(text)], block_size, stride)

    def __len__(self): return self.n

    def __getitem__(self, i):
        s = i * self.stride
        chunk = self.ids[s:s + self.block + 1]
        return chunk[:-1], chunk[1:]


class TranslationDataset(torch.utils.data.Dataset):
    """Line-aligned source / target files."""

    def __init__(self, src_path, tgt_path, src_pipeline=None, tgt_pipeline=None, max_length: int | None = None):
        src = Path(src_path).read_text(encoding="utf-8").splitlines()
        tgt = Path(tgt_path).read_text(encoding="utf-8").splitlines()
        if len(src) != len(tgt):
            raise ValueError(f"parallel files differ in length: {len(src)} vs {len(tgt)}")
        self.pairs = [(s, t) for s, t in zip(src, tgt) if s.strip() and t.strip()]
        self.sp, self.tp, self.max_length = src_pipeline, tgt_pipeline, max_length

    def __len__(self): return len(self.pairs)

    def __getitem__(self, i):
        s, t = self.pairs[i]
        s = self.sp(s) if self.sp else s
        t = self.tp(t) if self.tp else t
        if self.max_length is not None and not isinstance(s, str):
            s, t = s[:self.max_length], t[:self.max_length]
        return s, t


class SequenceLabelingDataset(torch.utils.data.Dataset):
    """CoNLL format: one ``token<sep>...<sep>tag`` per line, blank line between sentences."""

    def __init__(self, path, token_column: int = 0, tag_column: int = -1, sep: str | None = None):
        self.sentences, toks, tags = [], [], []
        for ln in Path(path).read_text(encoding="utf-8").splitlines() + [""]:
            if not ln.strip() or ln.startswith("-DOCSTART-"):
                if toks:
                    self.sentences.append((toks, tags))
                    toks, tags = [], []
                continue
            parts = ln.split(sep)
            toks.append(parts[token_column])
            tags.append(parts[tag_column])
        self.tag_names = sorted({t for _, ts in self.sentences for t in ts})

    def __len__(self): return len(self.sentences)
    def __getitem__(self, i): return self.sentences[i]


class CachedDataset(torch.utils.data.Dataset):
    """Memoises ``base[i]`` (tokenisation is usually the expensive part)."""

    def __init__(self, base, max_items: int | None = None):
        self.base, self.cache, self.max_items = base, {}, max_items
        self.hits = self.misses = 0

    def __len__(self): return len(self.base)

    def __getitem__(self, i):
        if i in self.cache:
            self.hits += 1
            return self.cache[i]
        self.misses += 1
        v = self.base[i]
        if self.max_items is None or len(self.cache) < self.max_items:
            self.cache[i] = v
        return v


def pad_sequences(seqs, pad_id: int = 0, max_length: int | None = None):
    """Right-pads lists of ids to a rectangle; returns (ids [N, T], attention mask [N, T], lengths [N])."""
    lens = [min(len(s), max_length) if max_length else len(s) for s in seqs]
    T = max(lens, default=0)
    ids = torch.full((len(seqs), T), pad_id, dtype=torch.long)
    for i, (s, n) in enumerate(zip(seqs, lens)):
        ids[i, :n] = torch.as_tensor(list(s)[:n], dtype=torch.long)
    lens_t = torch.tensor(lens, dtype=torch.long)
    return ids, (torch.arange(T)[None] < lens_t[:, None]), lens_t


class BatchIterator:
    """Batches of token-id sequences (optionally with labels), padded per batch. ``bucket=True`` sorts windows of
    ``bucket_size * batch_size`` examples by length first, which cuts the padding of mixed-length corpora."""

    def __init__(self, dataset, batch_size: int, pad_id: int = 0, shuffle: bool = False, bucket: bool = False, bucket_size: int = 50,
                 seed: int = 0, drop_last: bool = False):
        self.ds, self.bs, self.pad, self.shuffle, self.bucket, self.bsz, self.drop_last = dataset, batch_size, pad_id, shuffle, bucket, bucket_size, drop_last
        self.rng = random.Random(seed)

    def _seq(self, item):
        return item[0] if isinstance(item, tuple) else item

    def __iter__(self):
        idx = list(range(len(self.ds)))
        if self.shuffle:
            self.rng.shuffle(idx)
        if self.bucket:
            w = self.bs * self.bsz
            idx = [j for s in range(0, len(idx), w) for j in sorted(idx[s:s + w], key=lambda j: len(self._seq(self.ds[j])))]
        batches = [idx[s:s + self.bs] for s in range(0, len(idx), self.bs)]
        if self.drop_last and batches and len(batches[-1]) < self.bs:
            batches.pop()
        if self.shuffle and self.bucket:
            self.rng.shuffle(batches)
        for b in batches:
            items = [self.ds[j] for j in b]
            ids, mask, lens = pad_sequences([self._seq(it) for it in items], self.pad)
            out = {"input_ids": ids, "attention_mask": mask, "lengths": lens}
            if isinstance(items[0], tuple) and len(items[0]) > 1 and isinstance(items[0][-1], int):
                out["labels"] = torch.tensor([it[-1] for it in items])
            yield out


# ---- standard corpora in their published on-disk layouts (never downloaded) ------------------------------------------
def _need(path: Path, what: str) -> Path:
    if not path.exists():
        raise FileNotFoundError(f"{what} not found at {path}: place the corpus there (this library does not download)")
    return path


def ag_news(root, split: str = "train", pipeline=None) -> ClassificationDataset:
    """``root/{train,test}.csv`` with rows ``class index, title, description`` and no header."""
    p = _need(Path(root) / f"{split}.csv", "AG News")
    ds = ClassificationDataset(p, ColumnMapping(text=2, label=0), "csv", pipeline, has_header=False)
    return ds


class IMDBDataset(ClassificationDataset):
    """``root/{train,test}/{pos,neg}/*.txt``."""

    def __init__(self, root, split: str = "train", pipeline=None):
        base = _need(Path(root) / split, "IMDB")
        self.texts, self.labels, self.pairs = [], [], None
        self.label_names = ["neg", "pos"]
        for li, name in enumerate(self.label_names):
            for f in sorted((base / name).glob("*.txt")):
                self.texts.append(f.read_text(encoding="utf-8"))
                self.labels.append(li)
        self.pipeline = pipeline


def wikitext(root, split: str = "train", tokenizer=None, vocab=None, block_size: int = 128) -> LanguageModelingDataset:
    """``root/wiki.{train,valid,test}.tokens``."""
    p = _need(Path(root) / f"wiki.{split}.tokens", "WikiText")
    text = p.read_text(encoding="utf-8")
    tokenizer = tokenizer or (lambda s: s.split())
    if vocab is None:
        from . import Vocab
        vocab = Vocab.build([text], tokenizer=tokenizer)
    return LanguageModelingDataset.from_text(text, tokenizer, vocab, block_size)


def multi30k(root, split: str = "train", src: str = "de", tgt: str = "en", **kw) -> TranslationDataset:
    """``root/{train,val,test}.{de,en}``."""
    return TranslationDataset(_need(Path(root) / f"{split}.{src}", "Multi30k"), _need(Path(root) / f"{split}.{tgt}", "Multi30k"), **kw)
