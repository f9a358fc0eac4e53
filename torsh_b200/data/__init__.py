"""Datasets, samplers and the DataLoader (``crates/torsh-data``).

``DataLoaderConfig`` defaults follow ``crates/torsh-data/src/dataloader/mod.rs:128-160`` (batch_size 1, shuffle
false, num_workers 0, pin_memory false, drop_last false, prefetch_buffer_size 0, persistent_workers false).
``DistributedSampler`` follows ``crates/torsh-data/src/sampler/distributed.rs:194-330``: pad by wrap-around (or drop
the tail), Fisher-Yates shuffle with seed 42 by default, and each rank takes a CONTIGUOUS block
``[rank*k, (rank+1)*k)`` (not a strided one). Batches can be staged through pinned host buffers and copied to the
device on a side stream (``PrefetchToDevice``), the role of ``dataloader/memory.rs`` and ``prefetch.rs``.
"""
from __future__ import annotations

import math
import random
from dataclasses import dataclass

import torch
from torch.utils.data import (BatchSampler, ConcatDataset, Dataset, IterableDataset, RandomSampler, Sampler,
                              SequentialSampler, Subset, TensorDataset, WeightedRandomSampler, random_split)
from torch.utils.data import DataLoader as _TorchLoader
from torch.utils.data import default_collate


@dataclass
class DataLoaderConfig:
    batch_size: int = 1
    shuffle: bool = False
    num_workers: int = 0
    pin_memory: bool = False
    drop_last: bool = False
    timeout: float | None = None
    generator: int | None = None
    prefetch_buffer_size: int = 0
    persistent_workers: bool = False


class DataLoader(_TorchLoader):
    """``DataLoader(dataset, config)`` or PyTorch-style keyword arguments."""

    def __init__(self, dataset, config: DataLoaderConfig | None = None, **kw):
        if config is not None:
            g = torch.Generator().manual_seed(config.generator) if config.generator is not None else None
            kw = dict(batch_size=config.batch_size, shuffle=config.shuffle, num_workers=config.num_workers,
                      pin_memory=config.pin_memory, drop_last=config.drop_last, timeout=config.timeout or 0,
                      generator=g, persistent_workers=config.persistent_workers and config.num_workers > 0,
                      prefetch_factor=config.prefetch_buffer_size if (config.prefetch_buffer_size and config.num_workers) else None,
                      **kw)
        super().__init__(dataset, **kw)


class DistributedSampler(Sampler):
    def __init__(self, num_samples: int, num_replicas: int, rank: int, shuffle: bool = True, seed: int = 42,
                 drop_last: bool = False):
        if not 0 <= rank < num_replicas:
            raise ValueError(f"rank {rank} not in [0, {num_replicas})")
        self.n, self.replicas, self.rank, self.shuffle, self.seed, self.drop_last = num_samples, num_replicas, rank, shuffle, seed, drop_last
        self.epoch = 0
        self.per_replica = num_samples // num_replicas if drop_last else math.ceil(num_samples / num_replicas)
        self.total = self.per_replica * num_replicas

    def with_generator(self, seed: int):
        self.seed = seed
        return self

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def indices(self) -> list[int]:
        idx = list(range(self.n))
        if self.shuffle:
            rng = random.Random(self.seed + self.epoch)
            for i in range(len(idx) - 1, 0, -1):  # Fisher-Yates
                j = rng.randint(0, i)
                idx[i], idx[j] = idx[j], idx[i]
        if self.drop_last:
            idx = idx[: self.total]
        else:
            k = 0
            while len(idx) < self.total:  # wrap-around padding
                idx.append(idx[k])
                k += 1
        return idx[self.rank * self.per_replica:(self.rank + 1) * self.per_replica]

    def __iter__(self):
        return iter(self.indices())

    def __len__(self):
        return self.per_replica


class CachedDataset(Dataset):
    """Memoises items of a slow dataset (``crates/torsh-data/src/dataset/types.rs``)."""

    def __init__(self, base: Dataset, max_items: int | None = None):
        self.base, self.cache, self.max_items = base, {}, max_items

    def __len__(self):
        return len(self.base)

    def __getitem__(self, i):
        if i not in self.cache:
            if self.max_items is not None and len(self.cache) >= self.max_items:
                self.cache.pop(next(iter(self.cache)))
            self.cache[i] = self.base[i]
        return self.cache[i]


class MemoryMappedDataset(Dataset):
    """Fixed-shape records in a flat binary file, read through ``numpy.memmap``."""

    def __init__(self, path, dtype, record_shape):
        import numpy as np
        self.arr = np.memmap(path, dtype=dtype, mode="r")
        self.record_shape = tuple(record_shape)
        self.rec = int(math.prod(self.record_shape))
        self.n = self.arr.size // self.rec

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        import numpy as np
        return torch.from_numpy(np.array(self.arr[i * self.rec:(i + 1) * self.rec]).reshape(self.record_shape))


class StreamingDataset(IterableDataset):
    """Wraps a generator factory; each worker sees every ``num_workers``-th item."""

    def __init__(self, make_iter):
        self.make_iter = make_iter

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        it = self.make_iter()
        if info is None:
            yield from it
        else:
            for i, x in enumerate(it):
                if i % info.num_workers == info.id:
                    yield x


class SyntheticTokenDataset(Dataset):
    """Uniform random token ids with next-token targets (benchmark data)."""

    def __init__(self, vocab_size: int, seq_len: int, length: int, seed: int = 0):
        self.v, self.s, self.n, self.seed = vocab_size, seq_len, length, seed

    def __len__(self):
        return self.n

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + i)
        t = torch.randint(0, self.v, (self.s + 1,), generator=g)
        return t[:-1], t[1:]


class PrefetchToDevice:
    """Iterates a loader one batch ahead: pinned staging + H2D copy on a side stream."""

    def __init__(self, loader, device):
        self.loader, self.device = loader, torch.device(device)
        self.stream = torch.cuda.Stream() if self.device.type == "cuda" else None

    def _move(self, batch):
        if isinstance(batch, torch.Tensor):
            if self.stream is not None and not batch.is_pinned():
                batch = batch.pin_memory()
            return batch.to(self.device, non_blocking=True)
        if isinstance(batch, (list, tuple)):
            return type(batch)(self._move(b) for b in batch)
        if isinstance(batch, dict):
            return {k: self._move(v) for k, v in batch.items()}
        return batch

    def __iter__(self):
        it = iter(self.loader)
        nxt = None

        def fetch():
            try:
                b = next(it)
            except StopIteration:
                return None
            if self.stream is None:
                return self._move(b)
            with torch.cuda.stream(self.stream):
                return self._move(b)

        nxt = fetch()
        while nxt is not None:
            if self.stream is not None:
                torch.cuda.current_stream().wait_stream(self.stream)
            cur, nxt = nxt, fetch()
            yield cur

    def __len__(self):
        return len(self.loader)


def collate(batch):
    return default_collate(batch)


# ----------------------------------------------------------------------------------------- tabular / audio / columnar
class TabularDataset(Dataset):
    """Rows of numeric and categorical columns (``crates/torsh-data``: tabular datasets): numeric columns are
    standardised with statistics of the data given at construction, categorical ones mapped to integer codes.
    ``__getitem__`` returns ``(numeric [F], categorical [C], target)``."""

    def __init__(self, columns: dict, target: str, categorical=(), standardize: bool = True):
        self.target_name, self.categorical = target, list(categorical)
        self.numeric = [c for c in columns if c != target and c not in self.categorical]
        n = len(columns[target])
        num = torch.tensor([[float(columns[c][i]) for c in self.numeric] for i in range(n)], dtype=torch.float32).reshape(n, len(self.numeric))
        self.mean = num.mean(0) if standardize and n else torch.zeros(len(self.numeric))
        self.std = num.std(0, unbiased=False).clamp(min=1e-8) if standardize and n else torch.ones(len(self.numeric))
        self.num = (num - self.mean) / self.std
        self.vocab = {c: {v: i for i, v in enumerate(sorted(set(columns[c]), key=str))} for c in self.categorical}
        self.cat = torch.tensor([[self.vocab[c][columns[c][i]] for c in self.categorical] for i in range(n)],
                                dtype=torch.int64).reshape(n, len(self.categorical))
        t = columns[target]
        self.y = torch.tensor(t) if not isinstance(t, torch.Tensor) else t

    @classmethod
    def from_csv(cls, path: str, target: str, categorical=(), **kw):
        import csv
        with open(path, newline="") as f:
            rows = list(csv.DictReader(f))
        cols = {k: [r[k] for r in rows] for k in rows[0]}
        for k in cols:
            if k not in categorical:
                cols[k] = [float(v) for v in cols[k]]
        return cls(cols, target, categorical, **kw)

    @classmethod
    def from_parquet(cls, path: str, target: str, categorical=(), **kw):
        import pyarrow.parquet as pq
        table = pq.read_table(path)
        return cls({name: table.column(name).to_pylist() for name in table.column_names}, target, categorical, **kw)

    def cardinalities(self) -> list[int]:
        return [len(self.vocab[c]) for c in self.categorical]

    def __len__(self):
        return len(self.y)

    def __getitem__(self, i):
        return self.num[i], self.cat[i], self.y[i]


class AudioDataset(Dataset):
    """Waveforms with labels (``crates/torsh-data``: audio datasets): clips are cropped or zero-padded to ``num_samples``
    and optionally turned into log-mel-free log-magnitude spectrograms (``n_fft``, ``hop``). Sources are in-memory tensors
    or ``.npy`` files; ``synthetic`` makes labelled sine mixtures for tests and examples."""

    def __init__(self, waveforms, labels, sample_rate: int = 16000, num_samples: int | None = None, n_fft: int | None = None,
                 hop: int | None = None):
        self.items, self.labels, self.sr = list(waveforms), list(labels), sample_rate
        self.num_samples, self.n_fft, self.hop = num_samples, n_fft, hop or (n_fft // 4 if n_fft else None)

    @classmethod
    def synthetic(cls, n: int = 32, classes: int = 4, sample_rate: int = 8000, seconds: float = 0.25, seed: int = 0, **kw):
        g = torch.Generator().manual_seed(seed)
        t = torch.arange(int(sample_rate * seconds)) / sample_rate
        labels = torch.randint(0, classes, (n,), generator=g).tolist()
        waves = [torch.sin(2 * torch.pi * (220.0 * (c + 1)) * t) + 0.05 * torch.randn(t.shape, generator=g) for c in labels]
        return cls(waves, labels, sample_rate, **kw)

    def _load(self, item):
        if isinstance(item, str):
            import numpy as np
            return torch.from_numpy(np.load(item)).float()
        return item.float()

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        w = self._load(self.items[i]).reshape(-1)
        if self.num_samples is not None:
            w = w[: self.num_samples] if w.numel() >= self.num_samples else torch.nn.functional.pad(w, (0, self.num_samples - w.numel()))
        if self.n_fft:
            spec = torch.stft(w, self.n_fft, self.hop, window=torch.hann_window(self.n_fft), return_complex=True).abs()
            w = torch.log1p(spec)
        return w, self.labels[i]


class NativeTokenLoader:
    """Batches of token windows cut from a memory-mapped token file by native worker threads
    (``csrc/host/token_loader.cpp``): ``[batch, seq + 1]`` int64 windows land in a ring of (pinned, when a GPU is
    present) host buffers; iteration yields ``(inputs, targets)`` views of the current buffer. A buffer goes back to the
    workers ``hold`` batches later (default 1: it stays valid until the call after the next one), which covers an
    asynchronous host→device copy of a training loop that keeps one step in flight. Deterministic in ``(seed, rank)``;
    ranks read disjoint random streams."""

    def __init__(self, path: str, batch: int, seq: int, token_bytes: int = 2, slots: int = 4, workers: int = 2, seed: int = 0,
                 rank: int = 0, world: int = 1, pin: bool | None = None, timeout_s: float = 30.0, hold: int = 1):
        import ctypes

        from .. import _native as nv
        if slots < hold + 2:
            raise ValueError(f"slots ({slots}) must be at least hold + 2 ({hold + 2})")
        self.lib = nv.host()
        L = self.lib
        L.tsh_tokens_open.restype = ctypes.c_void_p
        L.tsh_tokens_open.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_int]
        L.tsh_tokens_next.argtypes = [ctypes.c_void_p, ctypes.c_double, ctypes.POINTER(ctypes.c_longlong)]
        L.tsh_tokens_release.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.tsh_tokens_count.restype, L.tsh_tokens_count.argtypes = ctypes.c_longlong, [ctypes.c_void_p]
        L.tsh_tokens_filled.restype, L.tsh_tokens_filled.argtypes = ctypes.c_longlong, [ctypes.c_void_p]
        L.tsh_tokens_close.argtypes = [ctypes.c_void_p]
        pin = torch.cuda.is_available() if pin is None else pin
        self.buffers = [torch.zeros(batch, seq + 1, dtype=torch.int64) for _ in range(slots)]
        if pin:
            self.buffers = [b.pin_memory() for b in self.buffers]
        ptrs = (ctypes.c_void_p * slots)(*[b.data_ptr() for b in self.buffers])
        self.h = L.tsh_tokens_open(str(path).encode(), token_bytes, batch, seq, slots, ptrs, workers, seed, rank, world)
        if not self.h:
            L.tsh_last_error.restype = ctypes.c_char_p
            raise OSError((L.tsh_last_error() or b"token loader: open failed").decode())
        self.timeout_s, self._held, self.batch_number, self.hold = timeout_s, [], -1, hold

    @property
    def num_tokens(self) -> int:
        return self.lib.tsh_tokens_count(self.h)

    def __iter__(self):
        return self

    def __next__(self):
        import ctypes
        while len(self._held) > self.hold:
            self.lib.tsh_tokens_release(self.h, self._held.pop(0))
        n = ctypes.c_longlong()
        slot = self.lib.tsh_tokens_next(self.h, self.timeout_s, ctypes.byref(n))
        if slot < 0:
            raise TimeoutError(f"no batch within {self.timeout_s}s")
        self._held.append(slot)
        self.batch_number = n.value
        buf = self.buffers[slot]
        return buf[:, :-1], buf[:, 1:]

    def close(self):
        if getattr(self, "h", None):
            self.lib.tsh_tokens_close(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


from . import pipeline, samplers, tabular  # noqa: E402,F401  (index samplers, dataset / transform combinators, tabular and columnar-file tools)
