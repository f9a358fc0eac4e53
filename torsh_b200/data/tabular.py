"""Tabular preprocessing, columnar file datasets, collate policies, fold splitters, text and audio sample transforms and
loader utilities (``crates/torsh-data/src/{tabular,arrow_integration,parquet_integration,collate/*,dataset/types,
text,text_processing,audio/transforms,sampler/advanced,privacy,federated,error,utils,builtin,zero_copy}.rs``).

Fitted statistics are tensors and ``transform`` is tensor arithmetic, so a fitted scaler or encoder can run on the device
inside the input pipeline; Arrow / Parquet columns are handed to ``torch.from_numpy`` without a copy when their layout
allows it."""
from __future__ import annotations

import csv
import math
import re
import threading
import time
from collections import Counter, OrderedDict
from pathlib import Path
from typing import Callable, Iterable, Sequence

import torch
from torch.utils.data import Dataset, Sampler

__all__ = [
    "StandardScaler", "MinMaxScaler", "RobustScaler", "LabelEncoder", "OneHotEncoder", "SimpleImputer", "VarianceThreshold",
    "SelectKBest", "f_classif", "CSVDataset", "ArrayDataset", "ArrowDataset", "ParquetDataset", "KFold", "StratifiedKFold",
    "GroupKFold", "DefaultCollate", "PadCollate", "SparseCollate", "MixedCollate", "DynamicBatchCollate", "CachedCollate",
    "TensorStacker", "AdaptiveBatchSampler", "GroupedSampler", "FederatedSampler", "PrivateSampler", "DatasetRegistry",
    "Vocabulary", "ToLowercase", "RemovePunctuation", "TrimWhitespace", "CollapseWhitespace", "RemoveNumbers",
    "RemoveStopwords", "Tokenize", "NGrams", "FilterByLength", "ReplacePattern", "AddSpecialTokens", "FixedLength",
    "TokenIdsToTensor", "SimpleBPE", "TextClassificationDataset", "TextFileDataset", "Resample", "AddNoise",
    "RandomBrightness", "RandomContrast", "GaussianNoise", "RetryStrategy", "ProgressTracker", "ConcurrentCache",
    "StatisticsCollector", "ZeroCopyTensor", "BufferManager", "OnlineAugmentationEngine",
]


# ================================================================================================ scalers and encoders
class _Fitted:
    def fit_transform(self, x, *a): return self.fit(x, *a).transform(x)


class StandardScaler(_Fitted):
    def __init__(self, with_mean: bool = True, with_std: bool = True): self.with_mean, self.with_std = with_mean, with_std
    def fit(self, x: torch.Tensor):
        x = x.double()
        self.mean_, self.var_ = x.mean(0), x.var(0, unbiased=False)
        self.scale_ = torch.where(self.var_ > 0, self.var_.sqrt(), torch.ones_like(self.var_))
        self.n_ = len(x)
        return self
    def partial_fit(self, x: torch.Tensor):
        """Chan's update of mean and variance with a new batch."""
        if not hasattr(self, "n_"):
            return self.fit(x)
        x = x.double()
        m, n = len(x), self.n_
        mean_b, var_b = x.mean(0), x.var(0, unbiased=False)
        delta = mean_b - self.mean_
        tot = n + m
        var = (self.var_ * n + var_b * m + delta ** 2 * n * m / tot) / tot
        self.mean_, self.n_, self.var_ = self.mean_ + delta * m / tot, tot, var
        self.scale_ = torch.where(var > 1e-30, var.sqrt(), torch.ones_like(var))
        return self
    def transform(self, x):
        out = x.double()
        if self.with_mean:
            out = out - self.mean_.to(x.device)
        if self.with_std:
            out = out / self.scale_.to(x.device)
        return out.to(x.dtype if x.is_floating_point() else torch.float32)
    def inverse_transform(self, z):
        out = z.double()
        if self.with_std:
            out = out * self.scale_.to(z.device)
        if self.with_mean:
            out = out + self.mean_.to(z.device)
        return out.to(z.dtype)


class MinMaxScaler(_Fitted):
    def __init__(self, feature_range=(0.0, 1.0)): self.lo, self.hi = feature_range
    def fit(self, x):
        x = x.double()
        self.min_, self.max_ = x.min(0).values, x.max(0).values
        return self
    def transform(self, x):
        span = (self.max_ - self.min_).to(x.device)
        span = torch.where(span > 0, span, torch.ones_like(span))
        return ((x.double() - self.min_.to(x.device)) / span * (self.hi - self.lo) + self.lo).to(x.dtype if x.is_floating_point() else torch.float32)
    def inverse_transform(self, z):
        span = (self.max_ - self.min_).to(z.device)
        return ((z.double() - self.lo) / (self.hi - self.lo) * span + self.min_.to(z.device)).to(z.dtype)


class RobustScaler(_Fitted):
    """Median and inter-quartile range."""
    def fit(self, x):
        q = torch.quantile(x.double(), torch.tensor([0.25, 0.5, 0.75], dtype=torch.float64), dim=0)
        self.center_, self.scale_ = q[1], torch.where(q[2] - q[0] > 0, q[2] - q[0], torch.ones_like(q[0]))
        return self
    def transform(self, x): return ((x.double() - self.center_) / self.scale_).to(x.dtype if x.is_floating_point() else torch.float32)


class LabelEncoder(_Fitted):
    """Sorted distinct values -> ``0 .. K-1``; works for strings, numbers and tensors."""
    def fit(self, values):
        vals = values.tolist() if isinstance(values, torch.Tensor) else list(values)
        self.classes_ = sorted(set(vals))
        self._index = {v: i for i, v in enumerate(self.classes_)}
        return self
    def transform(self, values) -> torch.Tensor:
        vals = values.tolist() if isinstance(values, torch.Tensor) else list(values)
        try:
            return torch.tensor([self._index[v] for v in vals], dtype=torch.long)
        except KeyError as e:
            raise ValueError(f"unseen label {e.args[0]!r}") from None
    def inverse_transform(self, ids): return [self.classes_[int(i)] for i in ids]


class OneHotEncoder(_Fitted):
    """Per-column categories; ``handle_unknown='ignore'`` encodes an unseen value as all zeros; ``drop_first`` removes the
    first category of every column (no collinearity with an intercept)."""
    def __init__(self, handle_unknown: str = "error", drop_first: bool = False): self.unknown, self.drop = handle_unknown, drop_first
    def fit(self, columns: Sequence[Sequence]):
        self.encoders_ = [LabelEncoder().fit(c) for c in columns]
        return self
    def transform(self, columns: Sequence[Sequence]) -> torch.Tensor:
        blocks = []
        for enc, col in zip(self.encoders_, columns):
            col = col.tolist() if isinstance(col, torch.Tensor) else list(col)
            k = len(enc.classes_)
            ids = []
            for v in col:
                if v in enc._index:
                    ids.append(enc._index[v])
                elif self.unknown == "ignore":
                    ids.append(k)
                else:
                    raise ValueError(f"unseen category {v!r}")
            oh = torch.nn.functional.one_hot(torch.tensor(ids), k + 1)[:, :k].float()
            blocks.append(oh[:, 1:] if self.drop else oh)
        return torch.cat(blocks, 1)
    def feature_names(self, names: Sequence[str]) -> list[str]:
        return [f"{n}={c}" for n, e in zip(names, self.encoders_) for c in (e.classes_[1:] if self.drop else e.classes_)]


class SimpleImputer(_Fitted):
    """NaN replacement by the column ``mean``, ``median``, ``most_frequent`` value or a ``constant``; ``add_indicator``
    appends one 0/1 column per feature that had gaps at fit time."""
    def __init__(self, strategy: str = "mean", fill_value: float = 0.0, add_indicator: bool = False): self.strategy, self.fill, self.indicator = strategy, fill_value, add_indicator
    def fit(self, x):
        x = x.double()
        stats = []
        for j in range(x.shape[1]):
            col = x[:, j][~torch.isnan(x[:, j])]
            if self.strategy == "constant" or len(col) == 0:
                stats.append(self.fill)
            elif self.strategy == "mean":
                stats.append(float(col.mean()))
            elif self.strategy == "median":
                stats.append(float(col.quantile(0.5)))
            else:
                v, c = torch.unique(col, return_counts=True)
                stats.append(float(v[c.argmax()]))
        self.statistics_ = torch.tensor(stats, dtype=torch.float64)
        self.missing_cols_ = torch.isnan(x).any(0)
        return self
    def transform(self, x):
        miss = torch.isnan(x)
        out = torch.where(miss, self.statistics_.to(x.dtype).expand_as(x), x)
        return torch.cat([out, miss[:, self.missing_cols_].to(x.dtype)], 1) if self.indicator else out


class VarianceThreshold(_Fitted):
    def __init__(self, threshold: float = 0.0): self.threshold = threshold
    def fit(self, x):
        self.variances_ = x.double().var(0, unbiased=False)
        self.support_ = self.variances_ > self.threshold
        return self
    def transform(self, x): return x[:, self.support_]


def f_classif(x: torch.Tensor, y: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """One-way ANOVA F statistic of every feature against the class label, with p-values."""
    x = x.double()
    classes = torch.unique(y)
    n, k = len(x), len(classes)
    grand = x.mean(0)
    ssb = sum((y == c).sum() * (x[y == c].mean(0) - grand) ** 2 for c in classes)
    ssw = sum(((x[y == c] - x[y == c].mean(0)) ** 2).sum(0) for c in classes)
    f = (ssb / (k - 1)) / (ssw / (n - k)).clamp(min=1e-300)
    from scipy import stats
    return f, torch.from_numpy(stats.f.sf(f.numpy(), k - 1, n - k))


class SelectKBest(_Fitted):
    def __init__(self, k: int, score_func: Callable = f_classif): self.k, self.score_func = k, score_func
    def fit(self, x, y):
        self.scores_ = self.score_func(x, y)[0]
        self.support_ = torch.zeros(x.shape[1], dtype=torch.bool)
        self.support_[self.scores_.topk(self.k).indices] = True
        return self
    def transform(self, x): return x[:, self.support_]
    def fit_transform(self, x, y): return self.fit(x, y).transform(x)


# ================================================================================================ datasets
class ArrayDataset(Dataset):
    """Features and optional targets held as tensors; ``transform`` is applied per sample."""
    def __init__(self, features, targets=None, transform: Callable | None = None):
        self.x, self.y, self.transform = torch.as_tensor(features), None if targets is None else torch.as_tensor(targets), transform
    def __len__(self): return len(self.x)
    def __getitem__(self, i):
        x = self.x[i] if self.transform is None else self.transform(self.x[i])
        return x if self.y is None else (x, self.y[i])


def _numeric(cell: str) -> float:
    try:
        return float(cell)
    except ValueError:
        return float("nan")


class CSVDataset(Dataset):
    """Delimited text -> float feature matrix.  Columns whose cells do not all parse as numbers are label-encoded (the
    encoders are kept in ``encoders``); empty cells and ``missing_values`` become NaN; ``target`` names or indexes the label."""
    def __init__(self, path, target: str | int | None = None, delimiter: str = ",", has_header: bool = True, missing_values=("", "NA", "NaN", "null"),
                 usecols: Sequence[str] | None = None, dtype=torch.float32):
        with open(path, newline="") as f:
            rows = list(csv.reader(f, delimiter=delimiter))
        header = rows[0] if has_header else [str(i) for i in range(len(rows[0]))]
        body = rows[1:] if has_header else rows
        cols = list(zip(*body)) if body else [()] * len(header)
        tcol = header.index(target) if isinstance(target, str) else target
        self.encoders, feats, names = {}, [], []
        self.targets = None
        for j, (name, col) in enumerate(zip(header, cols)):
            if usecols is not None and name not in usecols and j != tcol:
                continue
            cells = [c.strip() for c in col]
            present = [c for c in cells if c not in missing_values]
            numeric = all(not math.isnan(_numeric(c)) or c.lower() == "nan" for c in present)
            if numeric:
                vals = torch.tensor([float("nan") if c in missing_values else _numeric(c) for c in cells], dtype=torch.float64)
            else:
                enc = LabelEncoder().fit(present)
                self.encoders[name] = enc
                vals = torch.tensor([float("nan") if c in missing_values else enc._index[c] for c in cells], dtype=torch.float64)
            if j == tcol:
                self.targets = vals.long() if not torch.isnan(vals).any() and bool((vals == vals.round()).all()) else vals.to(dtype)
            else:
                feats.append(vals)
                names.append(name)
        self.feature_names = names
        self.features = torch.stack(feats, 1).to(dtype) if feats else torch.zeros(len(body), 0, dtype=dtype)
    def __len__(self): return len(self.features)
    def __getitem__(self, i): return self.features[i] if self.targets is None else (self.features[i], self.targets[i])


class ArrowDataset(Dataset):
    """A ``pyarrow.Table`` (or an Arrow IPC / Feather file) as tensors: numeric columns become one ``(rows, columns)`` matrix
    through ``to_numpy(zero_copy_only=...)``; dictionary and string columns are label-encoded."""
    def __init__(self, table_or_path, target: str | None = None, columns: Sequence[str] | None = None, dtype=torch.float32):
        import pyarrow as pa
        table = table_or_path
        if not isinstance(table, pa.Table):
            import pyarrow.feather as feather
            table = feather.read_table(str(table_or_path))
        self.schema = {f.name: str(f.type) for f in table.schema}
        self.encoders = {}
        feats, names = [], []
        self.targets = None
        for name in table.column_names:
            if columns is not None and name not in columns and name != target:
                continue
            col = table.column(name).combine_chunks()
            if pa.types.is_dictionary(col.type):
                col = col.dictionary_decode()
            if pa.types.is_string(col.type) or pa.types.is_large_string(col.type):
                vals = col.to_pylist()
                enc = LabelEncoder().fit([v for v in vals if v is not None])
                self.encoders[name] = enc
                t = torch.tensor([float("nan") if v is None else enc._index[v] for v in vals], dtype=torch.float64)
            else:
                zero_copy = col.null_count == 0 and not pa.types.is_boolean(col.type)
                arr = col.to_numpy(zero_copy_only=zero_copy)
                t = torch.from_numpy(arr if arr.flags.writeable else arr.copy())
            if name == target:
                self.targets = t.long() if not t.is_floating_point() or (not torch.isnan(t).any() and bool((t == t.round()).all())) else t.to(dtype)
            else:
                feats.append(t.to(dtype))
                names.append(name)
        self.feature_names = names
        self.features = torch.stack(feats, 1) if feats else torch.zeros(table.num_rows, 0, dtype=dtype)
    def __len__(self): return len(self.features)
    def __getitem__(self, i): return self.features[i] if self.targets is None else (self.features[i], self.targets[i])


class ParquetDataset(torch.utils.data.IterableDataset):
    """Streams a Parquet file row group by row group (``row_groups`` restricts them, which is how ranks and workers shard a
    file), with column projection and an optional ``filters`` predicate pushed into the reader.  ``materialize`` loads all."""
    def __init__(self, path, target: str | None = None, columns: Sequence[str] | None = None, row_groups: Sequence[int] | None = None, batch_rows: int | None = None, dtype=torch.float32):
        import pyarrow.parquet as pq
        self.path, self.target, self.columns, self.dtype, self.batch_rows = str(path), target, columns, dtype, batch_rows
        self.file = pq.ParquetFile(self.path)
        self.num_row_groups, self.num_rows = self.file.num_row_groups, self.file.metadata.num_rows
        self.row_groups = list(range(self.num_row_groups)) if row_groups is None else list(row_groups)

    def shard(self, rank: int, world: int) -> "ParquetDataset":
        return ParquetDataset(self.path, self.target, self.columns, self.row_groups[rank::world], self.batch_rows, self.dtype)

    def _tables(self):
        cols = None if self.columns is None else list(self.columns) + ([self.target] if self.target and self.target not in self.columns else [])
        for g in self.row_groups:
            yield self.file.read_row_group(g, columns=cols)

    def __iter__(self):
        for t in self._tables():
            ds = ArrowDataset(t, self.target, dtype=self.dtype)
            if self.batch_rows:
                for lo in range(0, len(ds), self.batch_rows):
                    yield (ds.features[lo:lo + self.batch_rows],) if ds.targets is None else (ds.features[lo:lo + self.batch_rows], ds.targets[lo:lo + self.batch_rows])
            else:
                for i in range(len(ds)):
                    yield ds[i]

    def materialize(self) -> ArrowDataset:
        import pyarrow as pa
        return ArrowDataset(pa.concat_tables(list(self._tables())), self.target, dtype=self.dtype)


# ================================================================================================ fold splitters
class KFold:
    def __init__(self, n_splits: int = 5, shuffle: bool = False, seed: int = 0): self.k, self.shuffle, self.seed = n_splits, shuffle, seed
    def split(self, n: int):
        idx = torch.randperm(n, generator=torch.Generator().manual_seed(self.seed)) if self.shuffle else torch.arange(n)
        sizes = [n // self.k + (1 if i < n % self.k else 0) for i in range(self.k)]
        lo = 0
        for s in sizes:
            yield torch.cat([idx[:lo], idx[lo + s:]]), idx[lo:lo + s]
            lo += s
    def subsets(self, dataset):
        for tr, te in self.split(len(dataset)):
            yield torch.utils.data.Subset(dataset, tr.tolist()), torch.utils.data.Subset(dataset, te.tolist())


class StratifiedKFold(KFold):
    def split(self, labels):
        labels = torch.as_tensor(labels)
        g = torch.Generator().manual_seed(self.seed)
        folds = [[] for _ in range(self.k)]
        for off, c in enumerate(torch.unique(labels).tolist()):
            idx = (labels == c).nonzero().flatten()
            if self.shuffle:
                idx = idx[torch.randperm(len(idx), generator=g)]
            for i, v in enumerate(idx.tolist()):
                folds[(i + off) % self.k].append(v)
        for f in range(self.k):
            yield torch.tensor(sorted(v for j in range(self.k) if j != f for v in folds[j])), torch.tensor(sorted(folds[f]))


class GroupKFold(KFold):
    """No group appears on both sides; groups are dealt largest-first to the lightest fold."""
    def split(self, groups):
        groups = list(groups.tolist() if isinstance(groups, torch.Tensor) else groups)
        counts = Counter(groups)
        load, assign = [0] * self.k, {}
        for gname, c in sorted(counts.items(), key=lambda kv: (-kv[1], str(kv[0]))):
            f = load.index(min(load))
            assign[gname], load[f] = f, load[f] + c
        for f in range(self.k):
            yield torch.tensor([i for i, gname in enumerate(groups) if assign[gname] != f]), torch.tensor([i for i, gname in enumerate(groups) if assign[gname] == f])


# ================================================================================================ collate
class TensorStacker:
    """Stacks equal-shape tensors into one pre-sized output (optionally pinned) with a single ``torch.stack(out=...)``."""
    def __init__(self, pin_memory: bool = False): self.pin = pin_memory and torch.cuda.is_available()
    def __call__(self, tensors: Sequence[torch.Tensor]) -> torch.Tensor:
        first = tensors[0]
        out = torch.empty((len(tensors), *first.shape), dtype=first.dtype, pin_memory=self.pin)
        return torch.stack(list(tensors), out=out)


class DefaultCollate:
    """Recursive: tensors are stacked, numbers become tensors, strings stay lists, mappings and tuples are collated field
    by field."""
    def __init__(self, pin_memory: bool = False): self.stack = TensorStacker(pin_memory)
    def __call__(self, batch):
        first = batch[0]
        if isinstance(first, torch.Tensor):
            return self.stack(batch)
        if isinstance(first, (int, float, bool)):
            return torch.tensor(batch)
        if isinstance(first, str):
            return list(batch)
        if isinstance(first, dict):
            return {k: self([b[k] for b in batch]) for k in first}
        if isinstance(first, (tuple, list)):
            return type(first)(self(list(f)) for f in zip(*batch)) if isinstance(first, tuple) else [self(list(f)) for f in zip(*batch)]
        return list(batch)


class PadCollate:
    """Pads dimension ``dim`` of every tensor field to the batch maximum (rounded up to ``pad_to_multiple``) and returns
    the lengths; non-tensor fields go through ``DefaultCollate``."""
    def __init__(self, padding_value=0, dim: int = 0, pad_to_multiple: int = 1, side: str = "right"):
        self.value, self.dim, self.mult, self.side, self.default = padding_value, dim, pad_to_multiple, side, DefaultCollate()
    def _pad(self, seqs):
        lens = torch.tensor([s.shape[self.dim] for s in seqs])
        L = int(math.ceil(int(lens.max()) / self.mult) * self.mult)
        out = []
        for s in seqs:
            pad = [0, 0] * s.dim()
            pad[2 * (s.dim() - 1 - self.dim) + (1 if self.side == "right" else 0)] = L - s.shape[self.dim]
            out.append(torch.nn.functional.pad(s, pad, value=self.value))
        return torch.stack(out), lens
    def __call__(self, batch):
        first = batch[0]
        if isinstance(first, torch.Tensor):
            return self._pad(batch)
        if isinstance(first, dict):
            out = {}
            for k in first:
                vals = [b[k] for b in batch]
                if isinstance(vals[0], torch.Tensor) and vals[0].dim() > 0 and len({v.shape for v in vals}) > 1:
                    out[k], out[k + "_lengths"] = self._pad(vals)
                else:
                    out[k] = self.default(vals)
            return out
        fields = list(zip(*batch))
        res = []
        for f in fields:
            if isinstance(f[0], torch.Tensor) and f[0].dim() > 0 and len({v.shape for v in f}) > 1:
                res.extend(self._pad(list(f)))
            else:
                res.append(self.default(list(f)))
        return tuple(res)


class SparseCollate:
    """Samples given as ``(indices, values)`` or sparse tensors -> one batched COO tensor ``(batch, *shape)``."""
    def __init__(self, shape: Sequence[int]): self.shape = tuple(shape)
    def __call__(self, batch):
        idx, val = [], []
        for b, item in enumerate(batch):
            if isinstance(item, torch.Tensor) and item.is_sparse:
                item = item.coalesce()
                i, v = item.indices(), item.values()
            else:
                i, v = item
                i = i.reshape(len(self.shape), -1) if i.dim() > 1 else i[None]
            idx.append(torch.cat([torch.full((1, i.shape[1]), b, dtype=torch.long), i.long()]))
            val.append(v)
        return torch.sparse_coo_tensor(torch.cat(idx, 1), torch.cat(val), (len(batch), *self.shape), check_invariants=True).coalesce()


class MixedCollate:
    """A collate function per field name (dict samples) or position (tuple samples); unnamed fields use the default."""
    def __init__(self, rules: dict, default: Callable | None = None): self.rules, self.default = rules, default or DefaultCollate()
    def __call__(self, batch):
        first = batch[0]
        if isinstance(first, dict):
            return {k: self.rules.get(k, self.default)([b[k] for b in batch]) for k in first}
        return tuple(self.rules.get(i, self.default)(list(f)) for i, f in enumerate(zip(*batch)))


class DynamicBatchCollate:
    """Splits an over-full list of variable-length samples into batches whose padded size ``max_len * count`` stays within
    ``max_tokens``, after sorting by length so that padding is small."""
    def __init__(self, max_tokens: int, length_fn: Callable = len, collate: Callable | None = None): self.max_tokens, self.length_fn, self.collate = max_tokens, length_fn, collate or PadCollate()
    def __call__(self, samples) -> list:
        order = sorted(range(len(samples)), key=lambda i: self.length_fn(samples[i]))
        out, cur, longest = [], [], 0
        for i in order:
            L = self.length_fn(samples[i])
            if cur and max(longest, L) * (len(cur) + 1) > self.max_tokens:
                out.append(self.collate([samples[j] for j in cur]))
                cur, longest = [], 0
            cur.append(i)
            longest = max(longest, L)
        if cur:
            out.append(self.collate([samples[j] for j in cur]))
        return out


class CachedCollate:
    """Memoises collated batches by a key of the batch (default: the ids of its samples), LRU-bounded: repeated epochs over
    fixed batches skip the stacking."""
    def __init__(self, collate: Callable | None = None, capacity: int = 256, key: Callable | None = None):
        self.collate, self.capacity, self.key = collate or DefaultCollate(), capacity, key or (lambda b: tuple(id(s) for s in b))
        self.cache, self.hits, self.misses = OrderedDict(), 0, 0
    def __call__(self, batch):
        k = self.key(batch)
        if k in self.cache:
            self.hits += 1
            self.cache.move_to_end(k)
            return self.cache[k]
        self.misses += 1
        out = self.cache[k] = self.collate(batch)
        if len(self.cache) > self.capacity:
            self.cache.popitem(last=False)
        return out


# ================================================================================================ samplers
class AdaptiveBatchSampler(Sampler):
    """Batches of indices under a memory budget: ``cost(i)`` estimates a sample's size and a batch closes before the sum
    would exceed ``budget``; ``report(seconds)`` after every step tunes the budget toward ``target_seconds`` per batch."""
    def __init__(self, n: int, cost: Callable[[int], float], budget: float, target_seconds: float | None = None, shuffle: bool = True, seed: int = 0):
        self.n, self.cost, self.budget, self.target, self.shuffle, self.seed, self.epoch = n, cost, budget, target_seconds, shuffle, seed, 0
    def report(self, seconds: float):
        if self.target:
            self.budget *= min(max(self.target / max(seconds, 1e-9), 0.5), 2.0) ** 0.5
    def __iter__(self):
        order = torch.randperm(self.n, generator=torch.Generator().manual_seed(self.seed + self.epoch)).tolist() if self.shuffle else list(range(self.n))
        self.epoch += 1
        cur, tot = [], 0.0
        for i in order:
            c = self.cost(i)
            if cur and tot + c > self.budget:
                yield cur
                cur, tot = [], 0.0
            cur.append(i)
            tot += c
        if cur:
            yield cur
    def __len__(self): return sum(1 for _ in iter(self))


class GroupedSampler(Sampler):
    """Every batch holds samples of a single group (same image size, same language, ...); groups are visited in shuffled
    batch order."""
    def __init__(self, groups: Sequence, batch_size: int, drop_last: bool = False, seed: int = 0):
        self.groups, self.bs, self.drop, self.seed, self.epoch = list(groups), batch_size, drop_last, seed, 0
    def __iter__(self):
        g = torch.Generator().manual_seed(self.seed + self.epoch)
        self.epoch += 1
        by = {}
        for i, k in enumerate(self.groups):
            by.setdefault(k, []).append(i)
        batches = []
        for k, idx in by.items():
            idx = [idx[j] for j in torch.randperm(len(idx), generator=g).tolist()]
            for lo in range(0, len(idx), self.bs):
                b = idx[lo:lo + self.bs]
                if len(b) == self.bs or not self.drop:
                    batches.append(b)
        for j in torch.randperm(len(batches), generator=g).tolist():
            yield batches[j]
    def __len__(self): return sum(1 for _ in iter(self))


class FederatedSampler:
    """Chooses the clients of a round: uniformly, proportionally to their data size, or by a capability score
    (``capabilities[c] = {"compute": .., "bandwidth": .., "battery": ..}``, clients below ``min_battery`` are skipped)."""
    def __init__(self, client_sizes: Sequence[int], clients_per_round: int, strategy: str = "uniform", capabilities: Sequence[dict] | None = None, min_battery: float = 0.2, seed: int = 0):
        self.sizes, self.m, self.strategy, self.caps, self.min_battery = list(client_sizes), clients_per_round, strategy, capabilities, min_battery
        self.gen = torch.Generator().manual_seed(seed)
    def sample(self) -> list[int]:
        n = len(self.sizes)
        if self.strategy == "uniform":
            w = torch.ones(n)
        elif self.strategy == "proportional":
            w = torch.tensor(self.sizes, dtype=torch.float)
        else:
            w = torch.tensor([0.0 if c.get("battery", 1.0) < self.min_battery else c.get("compute", 1.0) * c.get("bandwidth", 1.0) for c in self.caps])
        m = min(self.m, int((w > 0).sum()))
        return sorted(torch.multinomial(w, m, replacement=False, generator=self.gen).tolist())
    def aggregation_weights(self, chosen: Sequence[int]) -> torch.Tensor:
        s = torch.tensor([self.sizes[c] for c in chosen], dtype=torch.float)
        return s / s.sum()


class PrivateSampler(Sampler):
    """Poisson sampling (every index independently with probability ``rate``), the scheme differential-privacy accounting
    assumes; batch sizes therefore vary."""
    def __init__(self, n: int, rate: float, steps: int, seed: int = 0): self.n, self.rate, self.steps, self.gen = n, rate, steps, torch.Generator().manual_seed(seed)
    def __iter__(self):
        for _ in range(self.steps):
            yield (torch.rand(self.n, generator=self.gen) < self.rate).nonzero().flatten().tolist()
    def __len__(self): return self.steps


class DatasetRegistry:
    """Name -> factory, with decorator registration and keyword overrides at build time."""
    def __init__(self): self._f, self._doc = {}, {}
    def register(self, name: str, factory: Callable | None = None, description: str = ""):
        def deco(fn):
            if name in self._f:
                raise KeyError(f"dataset {name!r} already registered")
            self._f[name], self._doc[name] = fn, description or (fn.__doc__ or "").strip().split("\n")[0]
            return fn
        return deco(factory) if factory is not None else deco
    def build(self, name: str, **kw):
        if name not in self._f:
            raise KeyError(f"unknown dataset {name!r}; known: {sorted(self._f)}")
        return self._f[name](**kw)
    def list(self) -> dict: return dict(sorted(self._doc.items()))
    def __contains__(self, name): return name in self._f


# ================================================================================================ text
_PUNCT = re.compile(r"[^\w\s]", re.UNICODE)
_STOP = frozenset("a an the and or but if while of at by for with about against between into through during before after above below to from up down in out on off over under "
                  "again further then once here there when where why how all any both each few more most other some such no nor not only own same so than too very is are was were be been "
                  "being have has had do does did this that these those i you he she it we they me him her us them my your his its our their".split())


class ToLowercase:
    def __call__(self, s: str) -> str: return s.lower()
class RemovePunctuation:
    def __call__(self, s: str) -> str: return _PUNCT.sub("", s)
class TrimWhitespace:
    def __call__(self, s: str) -> str: return s.strip()
class CollapseWhitespace:
    def __call__(self, s: str) -> str: return re.sub(r"\s+", " ", s)
class RemoveNumbers:
    def __call__(self, s: str) -> str: return re.sub(r"\d+([.,]\d+)*", "", s)
class ReplacePattern:
    def __init__(self, pattern: str, replacement: str): self.p, self.r = re.compile(pattern), replacement
    def __call__(self, s: str) -> str: return self.p.sub(self.r, s)
class Tokenize:
    def __init__(self, pattern: str = r"\w+|[^\w\s]"): self.p = re.compile(pattern, re.UNICODE)
    def __call__(self, s: str) -> list[str]: return self.p.findall(s)
class RemoveStopwords:
    def __init__(self, stopwords: Iterable[str] | None = None): self.stop = frozenset(stopwords) if stopwords is not None else _STOP
    def __call__(self, tokens: list[str]) -> list[str]: return [t for t in tokens if t.lower() not in self.stop]
class FilterByLength:
    def __init__(self, min_len: int = 1, max_len: int = 10 ** 9): self.lo, self.hi = min_len, max_len
    def __call__(self, tokens: list[str]) -> list[str]: return [t for t in tokens if self.lo <= len(t) <= self.hi]
class NGrams:
    def __init__(self, n: int = 2, join: str | None = " ", include_lower: bool = False): self.n, self.join, self.lower = n, join, include_lower
    def __call__(self, tokens: list[str]) -> list:
        out = []
        for k in (range(1, self.n + 1) if self.lower else (self.n,)):
            for i in range(len(tokens) - k + 1):
                g = tokens[i:i + k]
                out.append(self.join.join(g) if self.join is not None else tuple(g))
        return out


class Vocabulary:
    """Token <-> id with the four special entries first; built from counts with ``min_freq`` and ``max_size``."""
    PAD, UNK, BOS, EOS = "<pad>", "<unk>", "<bos>", "<eos>"
    def __init__(self, tokens: Iterable[str] = ()):
        self.itos = [self.PAD, self.UNK, self.BOS, self.EOS]
        self.stoi = {t: i for i, t in enumerate(self.itos)}
        for t in tokens:
            self.add(t)
    @classmethod
    def build(cls, corpus: Iterable[Sequence[str]], min_freq: int = 1, max_size: int | None = None) -> "Vocabulary":
        c = Counter(t for doc in corpus for t in doc)
        items = sorted(((t, n) for t, n in c.items() if n >= min_freq), key=lambda kv: (-kv[1], kv[0]))
        v = cls(t for t, _ in (items[:max_size - 4] if max_size else items))
        v.freqs = c
        return v
    def add(self, t: str) -> int:
        if t not in self.stoi:
            self.stoi[t] = len(self.itos)
            self.itos.append(t)
        return self.stoi[t]
    def __len__(self): return len(self.itos)
    def __contains__(self, t): return t in self.stoi
    def encode(self, tokens: Sequence[str]) -> list[int]: return [self.stoi.get(t, 1) for t in tokens]
    def decode(self, ids: Sequence[int], skip_special: bool = True) -> list[str]: return [self.itos[int(i)] for i in ids if not (skip_special and int(i) < 4)]


class AddSpecialTokens:
    def __init__(self, bos: int = 2, eos: int = 3): self.bos, self.eos = bos, eos
    def __call__(self, ids: list[int]) -> list[int]: return [self.bos, *ids, self.eos]
class FixedLength:
    """Truncates or pads a list / 1-D tensor to ``length``."""
    def __init__(self, length: int, pad_value=0, truncate: str = "right"): self.L, self.pad, self.trunc = length, pad_value, truncate
    def __call__(self, seq):
        if isinstance(seq, torch.Tensor):
            seq = seq[..., :self.L] if self.trunc == "right" else seq[..., -self.L:]
            return torch.nn.functional.pad(seq, (0, self.L - seq.shape[-1]), value=self.pad)
        seq = list(seq[:self.L] if self.trunc == "right" else seq[-self.L:])
        return seq + [self.pad] * (self.L - len(seq))
class TokenIdsToTensor:
    def __call__(self, ids) -> torch.Tensor: return torch.tensor(ids, dtype=torch.long)


class SimpleBPE:
    """Byte-pair merges learned on word counts (end-of-word marker ``</w>``); ``encode`` applies the merges in the order
    they were learned."""
    def __init__(self, num_merges: int = 100): self.num_merges, self.merges = num_merges, []
    def fit(self, corpus: Iterable[str]) -> "SimpleBPE":
        words = Counter(w for line in corpus for w in line.split())
        vocab = {tuple(w) + ("</w>",): c for w, c in words.items()}
        for _ in range(self.num_merges):
            pairs = Counter()
            for sym, c in vocab.items():
                for a, b in zip(sym, sym[1:]):
                    pairs[(a, b)] += c
            if not pairs:
                break
            best = min(pairs, key=lambda p: (-pairs[p], p))
            if pairs[best] < 2:
                break
            self.merges.append(best)
            vocab = {self._merge(sym, best): c for sym, c in vocab.items()}
        self.ranks = {m: i for i, m in enumerate(self.merges)}
        return self
    @staticmethod
    def _merge(sym, pair):
        out, i = [], 0
        while i < len(sym):
            if i + 1 < len(sym) and (sym[i], sym[i + 1]) == pair:
                out.append(sym[i] + sym[i + 1]); i += 2
            else:
                out.append(sym[i]); i += 1
        return tuple(out)
    def encode_word(self, w: str) -> list[str]:
        sym = tuple(w) + ("</w>",)
        while len(sym) > 1:
            cand = [(self.ranks[p], p) for p in zip(sym, sym[1:]) if p in self.ranks]
            if not cand:
                break
            sym = self._merge(sym, min(cand)[1])
        return list(sym)
    def encode(self, text: str) -> list[str]: return [s for w in text.split() for s in self.encode_word(w)]
    def decode(self, pieces: Sequence[str]) -> str: return "".join(pieces).replace("</w>", " ").strip()


class TextClassificationDataset(Dataset):
    """``(text, label)`` pairs -> ``(token ids, label id)`` through a transform chain, vocabulary and fixed length."""
    def __init__(self, texts: Sequence[str], labels: Sequence, transforms: Sequence[Callable] = (ToLowercase(), RemovePunctuation(), Tokenize()), vocab: Vocabulary | None = None,
                 max_len: int = 64, min_freq: int = 1):
        self.transforms = list(transforms)
        toks = [self._apply(t) for t in texts]
        self.vocab = vocab or Vocabulary.build(toks, min_freq)
        self.label_encoder = LabelEncoder().fit(labels)
        fix = FixedLength(max_len)
        self.ids = torch.tensor([fix(self.vocab.encode(t)) for t in toks], dtype=torch.long)
        self.lengths = torch.tensor([min(len(t), max_len) for t in toks])
        self.labels = self.label_encoder.transform(labels)
    def _apply(self, s):
        for t in self.transforms:
            s = t(s)
        return s
    def __len__(self): return len(self.ids)
    def __getitem__(self, i): return self.ids[i], self.labels[i]


class TextFileDataset(Dataset):
    """One sample per line, addressed through a byte-offset index so that only the requested line is read."""
    def __init__(self, path, transform: Callable | None = None, encoding: str = "utf-8"):
        self.path, self.transform, self.encoding = str(path), transform, encoding
        self.offsets, pos = [], 0
        with open(self.path, "rb") as f:
            for line in f:
                if line.strip():
                    self.offsets.append(pos)
                pos += len(line)
    def __len__(self): return len(self.offsets)
    def __getitem__(self, i):
        with open(self.path, "rb") as f:
            f.seek(self.offsets[i])
            s = f.readline().decode(self.encoding).rstrip("\r\n")
        return s if self.transform is None else self.transform(s)


# ================================================================================================ audio and image sample transforms
class Resample:
    """Band-limited sample-rate conversion by a windowed-sinc polyphase filter."""
    def __init__(self, orig_rate: int, new_rate: int, taps_per_phase: int = 16):
        g = math.gcd(orig_rate, new_rate)
        self.up, self.down = new_rate // g, orig_rate // g
        self.tpp = taps_per_phase
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.up == self.down:
            return x
        up, down = self.up, self.down
        half = self.tpp * max(up, down)
        t = torch.arange(-half, half + 1, dtype=torch.float64)
        cutoff = 1.0 / max(up, down)
        h = cutoff * torch.sinc(cutoff * t) * torch.hann_window(len(t), periodic=False, dtype=torch.float64) * up
        # polyphase form: output n sits at m = n * down on the up-sampled grid and only every up-th filter tap meets a sample
        n_in = x.shape[-1]
        n_out = math.ceil(n_in * up / down)
        m = torch.arange(n_out, device=x.device) * down + half
        k0, phase = m // up, m % up
        J = (2 * half) // up + 1
        j = torch.arange(J, device=x.device)
        tap = phase[:, None] + j[None] * up
        src = k0[:, None] - j[None]
        ok = (tap <= 2 * half) & (src >= 0) & (src < n_in)
        w = torch.where(ok, h.to(x.device)[tap.clamp(max=2 * half)], torch.zeros((), dtype=torch.float64, device=x.device))
        xs = x.double().reshape(-1, n_in)[:, src.clamp(0, n_in - 1)]
        return (xs * w[None]).sum(-1).reshape(*x.shape[:-1], n_out).to(x.dtype)


class AddNoise:
    """White noise at a signal-to-noise ratio drawn uniformly from ``snr_db``."""
    def __init__(self, snr_db=(10.0, 30.0), seed: int | None = None): self.snr, self.gen = snr_db, None if seed is None else torch.Generator().manual_seed(seed)
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        snr = self.snr[0] + (self.snr[1] - self.snr[0]) * float(torch.rand((), generator=self.gen))
        power = x.double().pow(2).mean()
        noise = torch.randn(x.shape, generator=self.gen, dtype=torch.float64) * torch.sqrt(power / 10 ** (snr / 10))
        return (x.double() + noise).to(x.dtype)


class RandomBrightness:
    def __init__(self, delta: float = 0.2, seed: int | None = None): self.d, self.gen = delta, None if seed is None else torch.Generator().manual_seed(seed)
    def __call__(self, img): return (img * (1 + self.d * (2 * float(torch.rand((), generator=self.gen)) - 1))).clamp(0, 1)
class RandomContrast:
    def __init__(self, delta: float = 0.2, seed: int | None = None): self.d, self.gen = delta, None if seed is None else torch.Generator().manual_seed(seed)
    def __call__(self, img):
        f = 1 + self.d * (2 * float(torch.rand((), generator=self.gen)) - 1)
        m = img.mean((-1, -2, -3), keepdim=True)
        return ((img - m) * f + m).clamp(0, 1)
class GaussianNoise:
    def __init__(self, std: float = 0.05, seed: int | None = None): self.std, self.gen = std, None if seed is None else torch.Generator().manual_seed(seed)
    def __call__(self, x): return x + self.std * torch.randn(x.shape, generator=self.gen, dtype=x.dtype)


class OnlineAugmentationEngine:
    """Adjusts augmentation strength while training: ``report(train_metric, val_metric)`` raises the strength when the
    generalisation gap grows beyond ``target_gap`` and lowers it when training itself stalls; ``__call__`` applies each
    registered transform with probability ``strength``."""
    def __init__(self, transforms: Sequence[Callable], strength: float = 0.3, target_gap: float = 0.05, step: float = 0.05, seed: int = 0):
        self.transforms, self.strength, self.target_gap, self.step, self.gen, self.history = list(transforms), strength, target_gap, step, torch.Generator().manual_seed(seed), []
    def report(self, train_metric: float, val_metric: float):
        gap = train_metric - val_metric
        if gap > self.target_gap:
            self.strength = min(1.0, self.strength + self.step)
        elif gap < self.target_gap / 2:
            self.strength = max(0.0, self.strength - self.step)
        self.history.append((gap, self.strength))
    def __call__(self, x):
        for t in self.transforms:
            if float(torch.rand((), generator=self.gen)) < self.strength:
                x = t(x)
        return x


# ================================================================================================ loader utilities
class RetryStrategy:
    """Retries a flaky read with exponential back-off and jitter; only ``retry_on`` exceptions are retried."""
    def __init__(self, max_attempts: int = 3, base_delay: float = 0.05, factor: float = 2.0, max_delay: float = 2.0, retry_on=(OSError, TimeoutError), sleep: Callable = time.sleep):
        self.n, self.base, self.factor, self.cap, self.retry_on, self.sleep, self.attempts = max_attempts, base_delay, factor, max_delay, retry_on, sleep, 0
    def delays(self) -> list[float]: return [min(self.base * self.factor ** i, self.cap) for i in range(self.n - 1)]
    def run(self, fn: Callable, *a, **k):
        for i in range(self.n):
            self.attempts += 1
            try:
                return fn(*a, **k)
            except self.retry_on:
                if i == self.n - 1:
                    raise
                self.sleep(min(self.base * self.factor ** i, self.cap))


class ProgressTracker:
    def __init__(self, total: int, clock: Callable = time.perf_counter): self.total, self.done, self.clock, self.t0 = total, 0, clock, clock()
    def update(self, n: int = 1): self.done += n
    def rate(self) -> float: return self.done / max(self.clock() - self.t0, 1e-12)
    def eta(self) -> float: return (self.total - self.done) / max(self.rate(), 1e-12)
    def fraction(self) -> float: return self.done / max(self.total, 1)
    def __str__(self): return f"{self.done}/{self.total} ({100 * self.fraction():.1f}%) {self.rate():.1f}/s eta {self.eta():.0f}s"


class ConcurrentCache:
    """Thread-safe LRU; ``get_or_compute`` runs the producer once per key even when several workers ask at once."""
    def __init__(self, capacity: int = 1024):
        self.capacity, self.data, self.lock, self.pending, self.hits, self.misses = capacity, OrderedDict(), threading.Lock(), {}, 0, 0
    def get_or_compute(self, key, producer: Callable):
        with self.lock:
            if key in self.data:
                self.hits += 1
                self.data.move_to_end(key)
                return self.data[key]
            ev = self.pending.get(key)
            owner = ev is None
            if owner:
                ev = self.pending[key] = threading.Event()
                self.misses += 1
        if not owner:
            ev.wait()
            with self.lock:
                if key in self.data:
                    self.hits += 1
                    return self.data[key]
            return self.get_or_compute(key, producer)
        try:
            value = producer()
            with self.lock:
                self.data[key] = value
                if len(self.data) > self.capacity:
                    self.data.popitem(last=False)
            return value
        finally:
            with self.lock:
                self.pending.pop(key, None)
            ev.set()
    def __len__(self): return len(self.data)


class StatisticsCollector:
    """Per-channel mean / std / min / max of a dataset in one streaming pass (for normalisation constants)."""
    def __init__(self, channel_dim: int = 0): self.cd, self.n, self.s, self.ss, self.lo, self.hi = channel_dim, 0, None, None, None, None
    def update(self, x: torch.Tensor):
        x = x.double().movedim(self.cd, 0).reshape(x.shape[self.cd], -1)
        if self.s is None:
            self.s, self.ss = torch.zeros(len(x), dtype=torch.float64), torch.zeros(len(x), dtype=torch.float64)
            self.lo, self.hi = torch.full((len(x),), float("inf"), dtype=torch.float64), torch.full((len(x),), float("-inf"), dtype=torch.float64)
        self.n += x.shape[1]
        self.s += x.sum(1); self.ss += (x * x).sum(1)
        self.lo, self.hi = torch.minimum(self.lo, x.min(1).values), torch.maximum(self.hi, x.max(1).values)
    def compute(self) -> dict:
        mean = self.s / self.n
        return {"mean": mean, "std": (self.ss / self.n - mean ** 2).clamp(min=0).sqrt(), "min": self.lo, "max": self.hi, "count": self.n}


class ZeroCopyTensor:
    """A tensor view over a foreign buffer (``bytes``-like, ``mmap``, numpy array) that shares its memory; ``owner`` keeps
    the buffer alive for the lifetime of the view."""
    def __init__(self, buffer, dtype: torch.dtype, shape: Sequence[int], offset: int = 0):
        self.owner = buffer
        n = int(math.prod(shape))
        self.tensor = torch.frombuffer(buffer, dtype=dtype, count=n, offset=offset).reshape(tuple(shape))
    def shares_memory_with(self, other: torch.Tensor) -> bool: return self.tensor.untyped_storage().data_ptr() == other.untyped_storage().data_ptr()


class BufferManager:
    """Reusable byte buffers by size class (powers of two): ``acquire`` hands out a ``bytearray`` of at least the asked
    size, ``release`` returns it; avoids reallocating staging buffers per batch."""
    def __init__(self, max_per_class: int = 8): self.free, self.max, self.allocated, self.reused = {}, max_per_class, 0, 0
    @staticmethod
    def _cls(n: int) -> int: return 1 << max(n - 1, 1).bit_length()
    def acquire(self, nbytes: int) -> bytearray:
        c = self._cls(nbytes)
        pool = self.free.get(c)
        if pool:
            self.reused += 1
            return pool.pop()
        self.allocated += 1
        return bytearray(c)
    def release(self, buf: bytearray):
        pool = self.free.setdefault(len(buf), [])
        if len(pool) < self.max:
            pool.append(buf)
