"""Dataset combinators, transform framework and data services (``crates/torsh-data/src``): the ``Transform`` algebra
(``core_framework.rs``), dataset wrappers (``dataset/*_traits.rs``), text cleaning with a Porter stemmer
(``text_processing.rs``), progressive / adaptive augmentation schedules (``online_transforms.rs``,
``augmentation_pipeline.rs``), SQL-backed datasets (``database_integration.rs``), differentially private release
(``privacy.rs``), federated partitions and aggregation (``federated.rs``), pooled and memory-mapped batches
(``zero_copy.rs``), batched device-side preprocessing (``gpu_acceleration.rs``) and padding / nested collation (``collate/``)."""
from __future__ import annotations

import itertools
import math
import re
import sqlite3
import time
from collections import OrderedDict, deque
from pathlib import Path
from typing import Callable, Iterable, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset, IterableDataset


# ================================================================================================ transforms
class Transform:
    """Callable with ``then`` / ``when`` / ``|`` combinators."""

    def __call__(self, x): raise NotImplementedError
    def then(self, other) -> "Chain": return Chain(self, other)
    def __or__(self, other): return self.then(other)
    def when(self, predicate: Callable) -> "Conditional": return Conditional(predicate, self)
    def with_probability(self, p: float, seed: int = 0) -> "Conditional":
        g = torch.Generator().manual_seed(seed)
        return Conditional(lambda _: float(torch.rand((), generator=g)) < p, self)


class Lambda(Transform):
    def __init__(self, fn, name: str = "lambda"): self.fn, self.name = fn, name
    def __call__(self, x): return self.fn(x)
    def __repr__(self): return f"Lambda({self.name})"


class Chain(Transform):
    def __init__(self, *ts): self.ts = [t for x in ts for t in (x.ts if isinstance(x, Chain) else [x])]
    def __call__(self, x):
        for t in self.ts:
            x = t(x)
        return x
    def __repr__(self): return " | ".join(map(repr, self.ts))


Compose = Chain


class Conditional(Transform):
    def __init__(self, predicate, t, otherwise=None): self.predicate, self.t, self.otherwise = predicate, t, otherwise
    def __call__(self, x): return self.t(x) if self.predicate(x) else (self.otherwise(x) if self.otherwise else x)


class ToType(Transform):
    def __init__(self, dtype): self.dtype = dtype
    def __call__(self, x): return x.to(self.dtype)


class Normalize(Transform):
    def __init__(self, mean, std): self.mean, self.std = torch.as_tensor(mean, dtype=torch.float32), torch.as_tensor(std, dtype=torch.float32)
    def __call__(self, x):
        shape = (-1,) + (1,) * (x.dim() - 1) if self.mean.dim() else ()
        return (x - self.mean.reshape(shape)) / self.std.reshape(shape)


# ================================================================================================ datasets
class TensorDataset(Dataset):
    def __init__(self, *tensors):
        if len({len(t) for t in tensors}) != 1:
            raise ValueError("all tensors must have the same first dimension")
        self.tensors = tensors
    def __len__(self): return len(self.tensors[0])
    def __getitem__(self, i): return tuple(t[i] for t in self.tensors) if len(self.tensors) > 1 else self.tensors[0][i]


class TransformedDataset(Dataset):
    def __init__(self, base, transform, target_transform=None): self.base, self.transform, self.target_transform = base, transform, target_transform
    def __len__(self): return len(self.base)
    def __getitem__(self, i):
        item = self.base[i]
        if isinstance(item, tuple):
            return (self.transform(item[0]), *(self.target_transform(v) if self.target_transform else v for v in item[1:]))
        return self.transform(item)


class ChainDataset(IterableDataset):
    def __init__(self, *parts): self.parts = parts
    def __iter__(self): return itertools.chain.from_iterable(self.parts)


class InfiniteDataset(IterableDataset):
    """Cycles a map-style dataset forever, reshuffling every pass when ``shuffle``."""

    def __init__(self, base, shuffle=False, seed=0): self.base, self.shuffle, self.seed = base, shuffle, seed
    def __iter__(self):
        epoch = 0
        while True:
            order = torch.randperm(len(self.base), generator=torch.Generator().manual_seed(self.seed + epoch)).tolist() if self.shuffle else range(len(self.base))
            for i in order:
                yield self.base[i]
            epoch += 1


class BufferedStreamingDataset(IterableDataset):
    """Shuffle buffer over a stream: holds ``buffer_size`` items and emits a random one as each new item arrives."""

    def __init__(self, source: Iterable, buffer_size: int = 1000, seed: int = 0): self.source, self.buffer_size, self.seed = source, buffer_size, seed
    def __iter__(self):
        g, buf = torch.Generator().manual_seed(self.seed), []
        for item in self.source:
            if len(buf) < self.buffer_size:
                buf.append(item)
                continue
            j = int(torch.randint(0, len(buf), (), generator=g))
            yield buf[j]
            buf[j] = item
        for j in torch.randperm(len(buf), generator=g).tolist():
            yield buf[j]


class DataPipeline(IterableDataset):
    """Lazy stream stages: ``map`` / ``filter`` / ``batch`` / ``shuffle`` / ``take`` / ``skip`` / ``shard``, composed by chaining."""

    def __init__(self, source: Iterable, stages=()): self.source, self.stages = source, list(stages)
    def _with(self, stage): return DataPipeline(self.source, self.stages + [stage])
    def map(self, fn): return self._with(lambda it: (fn(x) for x in it))
    def filter(self, fn): return self._with(lambda it: (x for x in it if fn(x)))
    def take(self, n): return self._with(lambda it: itertools.islice(it, n))
    def skip(self, n): return self._with(lambda it: itertools.islice(it, n, None))
    def shard(self, num_shards, index): return self._with(lambda it: itertools.islice(it, index, None, num_shards))
    def shuffle(self, buffer_size, seed=0): return self._with(lambda it: iter(BufferedStreamingDataset(it, buffer_size, seed)))

    def batch(self, n, drop_last=False, collate=None):
        def stage(it):
            it = iter(it)
            while chunk := list(itertools.islice(it, n)):
                if len(chunk) == n or not drop_last:
                    yield collate(chunk) if collate else chunk
        return self._with(stage)

    def __iter__(self):
        it = iter(self.source)
        for s in self.stages:
            it = s(it)
        return iter(it)


class ProfiledDataset(Dataset):
    """Times every ``__getitem__`` and reports count, mean, p95 and the slowest indices."""

    def __init__(self, base, clock=time.perf_counter): self.base, self.clock, self.times = base, clock, {}
    def __len__(self): return len(self.base)
    def __getitem__(self, i):
        t0 = self.clock()
        item = self.base[i]
        self.times.setdefault(i, []).append(self.clock() - t0)
        return item

    def stats(self):
        allt = sorted(t for v in self.times.values() for t in v)
        if not allt:
            return {"count": 0}
        return {"count": len(allt), "mean": sum(allt) / len(allt), "p95": allt[min(len(allt) - 1, int(0.95 * len(allt)))], "total": sum(allt),
                "slowest": sorted(self.times, key=lambda i: -max(self.times[i]))[:5]}


class RealTimeDataset(IterableDataset):
    """Bounded queue fed by a producer (``push``); iteration yields items as they arrive and ends after ``close``."""

    def __init__(self, capacity: int = 1024, policy: str = "drop_oldest"): self.q, self.capacity, self.policy, self.closed, self.dropped = deque(), capacity, policy, False, 0
    def push(self, item) -> bool:
        if len(self.q) >= self.capacity:
            self.dropped += 1
            if self.policy == "drop_newest":
                return False
            self.q.popleft()
        self.q.append(item)
        return True
    def close(self): self.closed = True
    def __iter__(self):
        while self.q or not self.closed:
            if self.q:
                yield self.q.popleft()
            else:
                time.sleep(0.001)


class SharedMemoryDataset(Dataset):
    """Tensors moved to shared memory once, so worker processes read the same pages instead of copies."""

    def __init__(self, *tensors): self.tensors = tuple(t.contiguous().share_memory_() for t in tensors)
    def __len__(self): return len(self.tensors[0])
    def __getitem__(self, i): return tuple(t[i] for t in self.tensors)
    def is_shared(self): return all(t.is_shared() for t in self.tensors)


def random_split(dataset, fractions: Sequence[float], seed: int = 0):
    from torch.utils.data import Subset
    n = len(dataset)
    sizes = [int(math.floor(f * n)) for f in fractions]
    for i in range(n - sum(sizes)):
        sizes[i % len(sizes)] += 1
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed)).tolist()
    out, s = [], 0
    for k in sizes:
        out.append(Subset(dataset, perm[s:s + k]))
        s += k
    return out


# ================================================================================================ text cleaning
STOPWORDS = frozenset("a an and are as at be but by for from has have he her his i if in into is it its me my no not of on or our she so that the "
                      "their them then there these they this to up was we were what when which who will with you your".split())


class PorterStemmer:
    """The 1980 Porter algorithm, steps 1a to 5b."""

    _V = "aeiou"

    def _cons(self, w, i): return w[i] not in self._V and not (w[i] == "y" and i > 0 and self._cons(w, i - 1))

    def _m(self, w):
        forms = "".join("c" if self._cons(w, i) else "v" for i in range(len(w)))
        return len(re.findall("vc", re.sub(r"(.)\1+", r"\1", forms)))

    def _has_vowel(self, w): return any(not self._cons(w, i) for i in range(len(w)))
    def _double(self, w): return len(w) >= 2 and w[-1] == w[-2] and self._cons(w, len(w) - 1)
    def _cvc(self, w): return len(w) >= 3 and self._cons(w, len(w) - 3) and not self._cons(w, len(w) - 2) and self._cons(w, len(w) - 1) and w[-1] not in "wxy"

    def _replace(self, w, rules, cond):
        for suf, rep in rules:
            if w.endswith(suf):
                stem = w[:len(w) - len(suf)]
                return stem + rep if cond(stem) else w
        return w

    def stem(self, w: str) -> str:
        w = w.lower()
        if len(w) <= 2:
            return w
        if w.endswith("sses") or w.endswith("ies"):
            w = w[:-2]
        elif w.endswith("ss"):
            pass
        elif w.endswith("s"):
            w = w[:-1]
        if w.endswith("eed"):
            if self._m(w[:-3]) > 0:
                w = w[:-1]
        else:
            for suf in ("ed", "ing"):
                if w.endswith(suf) and self._has_vowel(w[:-len(suf)]):
                    w = w[:-len(suf)]
                    if w.endswith(("at", "bl", "iz")):
                        w += "e"
                    elif self._double(w) and w[-1] not in "lsz":
                        w = w[:-1]
                    elif self._m(w) == 1 and self._cvc(w):
                        w += "e"
                    break
        if w.endswith("y") and self._has_vowel(w[:-1]):
            w = w[:-1] + "i"
        m0 = lambda s: self._m(s) > 0
        w = self._replace(w, [("ational", "ate"), ("tional", "tion"), ("enci", "ence"), ("anci", "ance"), ("izer", "ize"), ("abli", "able"), ("alli", "al"),
                              ("entli", "ent"), ("eli", "e"), ("ousli", "ous"), ("ization", "ize"), ("ation", "ate"), ("ator", "ate"), ("alism", "al"),
                              ("iveness", "ive"), ("fulness", "ful"), ("ousness", "ous"), ("aliti", "al"), ("iviti", "ive"), ("biliti", "ble")], m0)
        w = self._replace(w, [("icate", "ic"), ("ative", ""), ("alize", "al"), ("iciti", "ic"), ("ical", "ic"), ("ful", ""), ("ness", "")], m0)
        for suf in ("al", "ance", "ence", "er", "ic", "able", "ible", "ant", "ement", "ment", "ent", "ion", "ou", "ism", "ate", "iti", "ous", "ive", "ize"):
            if w.endswith(suf):
                stem = w[:-len(suf)]
                if self._m(stem) > 1 and (suf != "ion" or stem.endswith(("s", "t"))):
                    w = stem
                break
        if w.endswith("e"):
            stem = w[:-1]
            if self._m(stem) > 1 or (self._m(stem) == 1 and not self._cvc(stem)):
                w = stem
        if self._m(w) > 1 and self._double(w) and w.endswith("l"):
            w = w[:-1]
        return w


class TextPipeline(Transform):
    """String cleaning steps in order; ``tokenize`` switches the value to a token list, later steps act on tokens."""

    def __init__(self): self.steps = []
    def _add(self, fn): self.steps.append(fn); return self
    def lowercase(self): return self._add(lambda s: s.lower() if isinstance(s, str) else [t.lower() for t in s])
    def remove_punctuation(self): return self._add(lambda s: re.sub(r"[^\w\s]", "", s))
    def remove_numbers(self): return self._add(lambda s: re.sub(r"\d+", "", s))
    def collapse_whitespace(self): return self._add(lambda s: re.sub(r"\s+", " ", s).strip())
    def replace_pattern(self, pattern, repl): return self._add(lambda s: re.sub(pattern, repl, s))
    def tokenize(self, pattern=r"\s+"): return self._add(lambda s: [t for t in re.split(pattern, s) if t])
    def remove_stopwords(self, words=STOPWORDS): return self._add(lambda ts: [t for t in ts if t not in words])
    def filter_by_length(self, lo=1, hi=10 ** 9): return self._add(lambda ts: [t for t in ts if lo <= len(t) <= hi])
    def stem(self): st = PorterStemmer(); return self._add(lambda ts: [st.stem(t) for t in ts])
    def ngrams(self, n, join=" "): return self._add(lambda ts: [join.join(ts[i:i + n]) for i in range(len(ts) - n + 1)])
    def __call__(self, s):
        for f in self.steps:
            s = f(s)
        return s


# ================================================================================================ augmentation schedules
class ProgressiveAugmentation:
    """Augmentation strength as a function of training progress: ``linear``, ``cosine`` or ``step`` ramp from ``start`` to
    ``end`` over ``total_steps``; ``transform_factory(strength)`` builds the transform for the current strength."""

    def __init__(self, transform_factory, start=0.0, end=1.0, total_steps=1000, mode="linear", steps=4):
        self.factory, self.start, self.end, self.total, self.mode, self.nsteps, self.step_count = transform_factory, start, end, total_steps, mode, steps, 0

    def strength(self) -> float:
        t = min(1.0, self.step_count / max(self.total, 1))
        if self.mode == "cosine":
            t = 0.5 * (1 - math.cos(math.pi * t))
        elif self.mode == "step":
            t = math.floor(t * self.nsteps) / self.nsteps
        return self.start + (self.end - self.start) * t

    def step(self): self.step_count += 1
    def __call__(self, x): return self.factory(self.strength())(x)


class AdaptiveAugmentation:
    """Closed loop on the train / validation gap: strength goes up while the model over-fits (gap above ``target_gap``) and
    down when it under-fits, by ``rate`` per update, inside ``[lo, hi]``."""

    def __init__(self, transform_factory, strength=0.3, target_gap=0.05, rate=0.05, lo=0.0, hi=1.0):
        self.factory, self.strength, self.target, self.rate, self.lo, self.hi, self.history = transform_factory, strength, target_gap, rate, lo, hi, []

    def update(self, train_metric: float, val_metric: float):
        gap = train_metric - val_metric
        self.strength = min(self.hi, max(self.lo, self.strength + (self.rate if gap > self.target else -self.rate)))
        self.history.append((gap, self.strength))

    def __call__(self, x): return self.factory(self.strength)(x)


class AugmentationPipeline(Transform):
    """Named stages with individual probabilities and usage statistics."""

    def __init__(self, seed=0): self.stages, self.gen, self.stats = [], torch.Generator().manual_seed(seed), OrderedDict()
    def add(self, name, fn, p=1.0): self.stages.append((name, fn, p)); self.stats[name] = 0; return self
    def __call__(self, x):
        for name, fn, p in self.stages:
            if p >= 1.0 or float(torch.rand((), generator=self.gen)) < p:
                x = fn(x)
                self.stats[name] += 1
        return x


# ================================================================================================ SQL datasets
class DatabaseDataset(Dataset):
    """Rows of a SQL query as a map-style dataset over ``sqlite3`` (file or ``:memory:`` connection).  Keys are read once;
    rows are fetched in pages of ``page_size`` by key and cached (LRU of ``cache_pages``).  Numeric ``feature_columns``
    become a float tensor, ``target_column`` the label."""

    def __init__(self, conn_or_path, table: str, feature_columns: Sequence[str], target_column: str | None = None, key: str = "rowid", where: str = "",
                 page_size: int = 256, cache_pages: int = 8):
        self.conn = conn_or_path if isinstance(conn_or_path, sqlite3.Connection) else sqlite3.connect(str(conn_or_path))
        ident = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")
        for name in (table, key, *feature_columns, *( [target_column] if target_column else [])):
            if not ident.match(name):
                raise ValueError(f"bad SQL identifier {name!r}")
        self.table, self.features, self.target, self.key, self.page_size, self.cache_pages = table, list(feature_columns), target_column, key, page_size, cache_pages
        self.keys = [r[0] for r in self.conn.execute(f"SELECT {key} FROM {table} {('WHERE ' + where) if where else ''} ORDER BY {key}")]
        self.cache: OrderedDict[int, list] = OrderedDict()
        self.queries = 0

    def __len__(self): return len(self.keys)

    def _page(self, p):
        if p in self.cache:
            self.cache.move_to_end(p)
            return self.cache[p]
        ks = self.keys[p * self.page_size:(p + 1) * self.page_size]
        cols = ", ".join([self.key] + self.features + ([self.target] if self.target else []))
        rows = {r[0]: r[1:] for r in self.conn.execute(f"SELECT {cols} FROM {self.table} WHERE {self.key} IN ({','.join('?' * len(ks))})", ks)}
        self.queries += 1
        self.cache[p] = [rows[k] for k in ks]
        if len(self.cache) > self.cache_pages:
            self.cache.popitem(last=False)
        return self.cache[p]

    def __getitem__(self, i):
        row = self._page(i // self.page_size)[i % self.page_size]
        x = torch.tensor([float(v) for v in row[:len(self.features)]])
        return (x, row[-1]) if self.target else x


# ================================================================================================ privacy
class PrivacyBudget:
    """Tracks (epsilon, delta) spending under ``basic`` (sums) or ``advanced`` composition
    (``eps * sqrt(2 k ln(1/delta')) + k eps (e^eps - 1)`` for ``k`` equal queries) and refuses queries beyond the total."""

    def __init__(self, epsilon: float, delta: float = 0.0, composition: str = "basic", delta_slack: float = 1e-6):
        self.total_eps, self.total_delta, self.composition, self.slack, self.spent = epsilon, delta, composition, delta_slack, []

    def consumed(self) -> tuple[float, float]:
        if not self.spent:
            return 0.0, 0.0
        eps, delta = [e for e, _ in self.spent], sum(d for _, d in self.spent)
        if self.composition == "advanced" and len(set(eps)) == 1 and len(eps) > 1:
            e, k = eps[0], len(eps)
            adv = e * math.sqrt(2 * k * math.log(1 / self.slack)) + k * e * (math.exp(e) - 1)
            if adv < sum(eps):
                return adv, delta + self.slack
        return sum(eps), delta

    def remaining(self): e, d = self.consumed(); return self.total_eps - e, self.total_delta - d

    def spend(self, epsilon: float, delta: float = 0.0):
        self.spent.append((epsilon, delta))
        e, d = self.consumed()
        if e > self.total_eps + 1e-12 or d > self.total_delta + 1e-12:
            self.spent.pop()
            raise PermissionError(f"privacy budget exceeded: would reach eps={e:.4g}, delta={d:.3g} of ({self.total_eps}, {self.total_delta})")


def laplace_mechanism(value, sensitivity: float, epsilon: float, generator=None):
    v = torch.as_tensor(value, dtype=torch.float64)
    u = torch.rand(v.shape, generator=generator, dtype=torch.float64) - 0.5
    return v - (sensitivity / epsilon) * torch.sign(u) * torch.log1p(-2 * u.abs())


def gaussian_mechanism(value, sensitivity: float, epsilon: float, delta: float, generator=None):
    """Classical calibration ``sigma = sensitivity * sqrt(2 ln(1.25 / delta)) / epsilon`` (valid for ``epsilon < 1``)."""
    v = torch.as_tensor(value, dtype=torch.float64)
    sigma = sensitivity * math.sqrt(2 * math.log(1.25 / delta)) / epsilon
    return v + sigma * torch.randn(v.shape, generator=generator, dtype=torch.float64)


def randomized_response(bits: torch.Tensor, epsilon: float, generator=None):
    """Each bit is kept with probability ``e^eps / (1 + e^eps)``; returns the noisy bits and an unbiased estimate of the mean."""
    p = math.exp(epsilon) / (1 + math.exp(epsilon))
    keep = torch.rand(bits.shape, generator=generator) < p
    noisy = torch.where(keep, bits.bool(), ~bits.bool())
    return noisy, (noisy.float().mean().item() - (1 - p)) / (2 * p - 1)


class PrivateDataset:
    """Answers bounded-sensitivity queries about a numeric tensor under a budget: ``count``, ``sum``, ``mean`` (clipped to
    ``[lo, hi]``) and ``histogram``; raw rows are never returned."""

    def __init__(self, data: torch.Tensor, lo: float, hi: float, budget: PrivacyBudget, seed: int = 0):
        self.data, self.lo, self.hi, self.budget, self.gen = data.double().clamp(lo, hi), lo, hi, budget, torch.Generator().manual_seed(seed)

    def count(self, predicate, epsilon): self.budget.spend(epsilon); return float(laplace_mechanism(float(predicate(self.data).sum()), 1.0, epsilon, self.gen))
    def sum(self, epsilon): self.budget.spend(epsilon); return float(laplace_mechanism(float(self.data.sum()), max(abs(self.lo), abs(self.hi)), epsilon, self.gen))

    def mean(self, epsilon):
        self.budget.spend(epsilon)
        return float(laplace_mechanism(float(self.data.mean()), (self.hi - self.lo) / len(self.data), epsilon, self.gen))

    def histogram(self, bins: int, epsilon):
        self.budget.spend(epsilon)
        h = torch.histc(self.data.float(), bins, self.lo, self.hi).double()
        return laplace_mechanism(h, 1.0, epsilon, self.gen).clamp(min=0)          # one row changes one bin by one (add / remove)


# ================================================================================================ federated
def partition_iid(n: int, clients: int, seed: int = 0) -> list[list[int]]:
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed)).tolist()
    return [perm[i::clients] for i in range(clients)]


def partition_dirichlet(labels, clients: int, alpha: float = 0.5, seed: int = 0) -> list[list[int]]:
    """Label-skewed split: the share of each class that a client receives is drawn from ``Dirichlet(alpha)``."""
    rng, labels = np.random.default_rng(seed), np.asarray(labels)
    out: list[list[int]] = [[] for _ in range(clients)]
    for c in np.unique(labels):
        idx = rng.permutation(np.nonzero(labels == c)[0])
        cuts = (np.cumsum(rng.dirichlet([alpha] * clients)) * len(idx)).astype(int)[:-1]
        for k, part in enumerate(np.split(idx, cuts)):
            out[k] += part.tolist()
    return out


def partition_shards(labels, clients: int, shards_per_client: int = 2, seed: int = 0) -> list[list[int]]:
    """Sort by label, cut into ``clients * shards_per_client`` shards, deal shards at random (the FedAvg paper's split)."""
    order = np.argsort(np.asarray(labels), kind="stable")
    shards = np.array_split(order, clients * shards_per_client)
    perm = np.random.default_rng(seed).permutation(len(shards))
    return [sorted(np.concatenate([shards[j] for j in perm[k * shards_per_client:(k + 1) * shards_per_client]]).tolist()) for k in range(clients)]


class FederatedDataset:
    """A dataset split over simulated clients with capability records; ``select_clients`` draws a round's participants
    (``random``, ``weighted`` by data size, or ``capable``: fastest first), ``client(k)`` is that client's subset."""

    def __init__(self, base, partitions, capabilities: Sequence[dict] | None = None):
        self.base, self.partitions = base, partitions
        self.capabilities = list(capabilities or [{"compute": 1.0, "bandwidth": 1.0} for _ in partitions])

    def client(self, k):
        from torch.utils.data import Subset
        return Subset(self.base, self.partitions[k])

    def sizes(self): return [len(p) for p in self.partitions]

    def select_clients(self, n: int, strategy: str = "random", seed: int = 0) -> list[int]:
        g = torch.Generator().manual_seed(seed)
        if strategy == "weighted":
            return torch.multinomial(torch.tensor(self.sizes(), dtype=torch.float64), n, False, generator=g).tolist()
        if strategy == "capable":
            return sorted(range(len(self.partitions)), key=lambda k: -(self.capabilities[k]["compute"] * self.capabilities[k]["bandwidth"]))[:n]
        return torch.randperm(len(self.partitions), generator=g)[:n].tolist()

    def label_distribution(self, labels) -> torch.Tensor:
        labels = torch.as_tensor(labels)
        c = int(labels.max()) + 1
        return torch.stack([torch.bincount(labels[p], minlength=c).float() / max(len(p), 1) for p in self.partitions])


def federated_average(states: Sequence[dict], weights: Sequence[float] | None = None, strategy: str = "fedavg", trim: float = 0.2) -> dict:
    """``fedavg`` (weighted mean), ``median`` (coordinate-wise) or ``trimmed_mean`` (drops the ``trim`` share at each end)."""
    w = torch.tensor(weights if weights is not None else [1.0] * len(states), dtype=torch.float64)
    w = w / w.sum()
    out = {}
    for k in states[0]:
        stack = torch.stack([s[k].double() for s in states])
        if strategy == "median":
            v = stack.median(0).values
        elif strategy == "trimmed_mean":
            cut = int(trim * len(states))
            v = stack.sort(0).values[cut:len(states) - cut].mean(0)
        else:
            v = (stack * w.reshape(-1, *[1] * (stack.dim() - 1))).sum(0)
        out[k] = v.to(states[0][k].dtype)
    return out


# ================================================================================================ zero copy / device preprocessing
class TensorPool:
    """Reusable batch buffers keyed by ``(shape, dtype, pinned)``: ``acquire`` hands out a free buffer or allocates one,
    ``release`` returns it; a loader that recycles buffers stops allocating after the first few batches."""

    def __init__(self, pin_memory: bool = False): self.free, self.pin, self.allocated, self.reused = {}, pin_memory, 0, 0

    def acquire(self, shape, dtype=torch.float32) -> torch.Tensor:
        key = (tuple(shape), dtype)
        if self.free.get(key):
            self.reused += 1
            return self.free[key].pop()
        self.allocated += 1
        return torch.empty(shape, dtype=dtype, pin_memory=self.pin and torch.cuda.is_available())

    def release(self, t: torch.Tensor): self.free.setdefault((tuple(t.shape), t.dtype), []).append(t)


class MemoryMappedLoader:
    """Batches as views of a ``.npy`` file opened with ``mmap_mode='r'``: a contiguous batch is a slice of the mapping (no
    copy until the tensor is moved); an index list gathers rows."""

    def __init__(self, path, batch_size: int): self.arr, self.batch_size = np.load(path, mmap_mode="r"), batch_size
    def __len__(self): return math.ceil(len(self.arr) / self.batch_size)
    def batch(self, i) -> torch.Tensor:
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")                                     # read-only mapping: torch warns that writes are undefined
            return torch.from_numpy(self.arr[i * self.batch_size:(i + 1) * self.batch_size])
    def gather(self, indices) -> torch.Tensor: return torch.from_numpy(np.ascontiguousarray(self.arr[np.sort(np.asarray(indices))]))
    def __iter__(self): return (self.batch(i) for i in range(len(self)))


class DevicePreprocessingPipeline:
    """Batched preprocessing on the model's device: uint8 ``[N, H, W, C]`` batches are uploaded once (non-blocking from
    pinned memory), then converted, resized, flipped, jittered and normalised there, so the host does no per-image work."""

    def __init__(self, device="cpu", size=None, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225), flip_p=0.0, brightness=0.0, seed=0, dtype=torch.float32):
        self.device, self.size, self.flip_p, self.brightness, self.dtype = torch.device(device), size, flip_p, brightness, dtype
        self.mean, self.std = torch.tensor(mean, device=self.device).reshape(1, -1, 1, 1), torch.tensor(std, device=self.device).reshape(1, -1, 1, 1)
        self.gen = torch.Generator(device="cpu").manual_seed(seed)
        self.batches = self.bytes_uploaded = 0

    def __call__(self, batch_u8: torch.Tensor) -> torch.Tensor:
        x = batch_u8.to(self.device, non_blocking=True)
        self.batches += 1
        self.bytes_uploaded += batch_u8.numel()
        x = x.permute(0, 3, 1, 2).float() / 255
        if self.size and tuple(x.shape[-2:]) != tuple(self.size):
            x = torch.nn.functional.interpolate(x, size=self.size, mode="bilinear", align_corners=False, antialias=True)
        n = x.shape[0]
        if self.flip_p > 0:
            flip = (torch.rand(n, generator=self.gen) < self.flip_p).to(self.device)
            x = torch.where(flip.reshape(n, 1, 1, 1), x.flip(-1), x)
        if self.brightness > 0:
            f = (1 + (torch.rand(n, generator=self.gen) * 2 - 1) * self.brightness).to(self.device)
            x = (x * f.reshape(n, 1, 1, 1)).clamp(0, 1)
        return ((x - self.mean) / self.std).to(self.dtype)


# ================================================================================================ collation
def pad_sequence_collate(batch, padding_value=0, pad_to_multiple: int = 1, left: bool = False):
    """Variable-length 1-D (or ``[L, ...]``) tensors to a padded batch, lengths and a boolean mask (true = real)."""
    seqs = [b[0] if isinstance(b, tuple) else b for b in batch]
    lengths = torch.tensor([len(s) for s in seqs])
    width = int(math.ceil(int(lengths.max()) / pad_to_multiple) * pad_to_multiple)
    out = seqs[0].new_full((len(seqs), width, *seqs[0].shape[1:]), padding_value)
    for i, s in enumerate(seqs):
        if left:
            out[i, width - len(s):] = s
        else:
            out[i, :len(s)] = s
    ar = torch.arange(width)[None]
    mask = ar >= (width - lengths)[:, None] if left else ar < lengths[:, None]
    rest = tuple(torch.as_tensor([b[k] for b in batch]) for k in range(1, len(batch[0]))) if isinstance(batch[0], tuple) else ()
    return (out, lengths, mask, *rest)


def nested_collate(batch):
    """Recursively stacks tensors / numbers inside dicts, tuples and lists; strings and ragged tensors stay as lists."""
    first = batch[0]
    if isinstance(first, torch.Tensor):
        return torch.stack(batch) if all(b.shape == first.shape for b in batch) else list(batch)
    if isinstance(first, (int, float, bool, np.number)):
        return torch.tensor(batch)
    if isinstance(first, dict):
        return {k: nested_collate([b[k] for b in batch]) for k in first}
    if isinstance(first, (tuple, list)) and not isinstance(first, str):
        return type(first)(nested_collate(list(col)) for col in zip(*batch))
    return list(batch)
