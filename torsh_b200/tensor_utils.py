"""Runtime helpers of the tensor layer (``crates/torsh-tensor/src/{memory_pool,lockfree_cache,auto_batching,async_ops,
op_logging,tensor_tracker}.rs``): a pool of reusable scratch tensors, a small cache that readers never lock, a batcher
that groups single requests into one batched call, a thread-backed asynchronous op runner, an operation log and a
tracker of live tensors. Device memory itself is managed by the native caching pools (``core.runtime``); these are the
host-side conveniences built on top."""
from __future__ import annotations

import threading
import time
import weakref
from collections import OrderedDict, defaultdict, deque
from concurrent.futures import Future, ThreadPoolExecutor
from contextlib import contextmanager
from dataclasses import dataclass, field

import torch


class ReusedBuffer:
    """A tensor on loan from :class:`GlobalMemoryPool`; give it back with ``release()`` or use it as a context manager."""

    def __init__(self, pool: "GlobalMemoryPool", tensor: torch.Tensor, key, base: torch.Tensor):
        self.pool, self.tensor, self._key, self._base = pool, tensor, key, base

    def release(self):
        if self.tensor is not None:
            self.pool._give_back(self._key, self._base)
            self.tensor = self._base = None

    def __enter__(self):
        return self.tensor

    def __exit__(self, *exc):
        self.release()


class GlobalMemoryPool:
    """Scratch tensors keyed by (numel rounded up to a power of two, dtype, device); at most ``max_per_key`` are kept."""

    _instance = None

    def __init__(self, max_per_key: int = 8):
        self.max_per_key = max_per_key
        self._free: dict[tuple, list[torch.Tensor]] = defaultdict(list)
        self._lock = threading.Lock()
        self.stats = {"hits": 0, "misses": 0, "returned": 0, "dropped": 0}

    @classmethod
    def instance(cls) -> "GlobalMemoryPool":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def acquire(self, shape, dtype=torch.float32, device="cpu") -> ReusedBuffer:
        n = 1
        for s in (shape if isinstance(shape, (tuple, list)) else (shape,)):
            n *= int(s)
        cap = 1 << max(n - 1, 0).bit_length()
        key = (cap, dtype, str(device))
        with self._lock:
            if self._free[key]:
                base = self._free[key].pop()
                self.stats["hits"] += 1
            else:
                base = None
                self.stats["misses"] += 1
        if base is None:
            base = torch.empty(cap, dtype=dtype, device=device)
        return ReusedBuffer(self, base[:n].view(shape), key, base)

    def _give_back(self, key, base):
        with self._lock:
            if len(self._free[key]) < self.max_per_key:
                self._free[key].append(base)
                self.stats["returned"] += 1
            else:
                self.stats["dropped"] += 1

    def clear(self):
        with self._lock:
            self._free.clear()


class LockFreeCache:
    """Read-mostly cache: readers take a reference to an immutable snapshot dict without locking; writers copy, modify
    and swap the snapshot under a lock (``lockfree_cache.rs``'s role: no reader ever blocks on a writer)."""

    def __init__(self, capacity: int = 1024):
        self.capacity, self._snap, self._wlock = capacity, OrderedDict(), threading.Lock()
        self.hits = self.misses = 0

    def get(self, key, default=None):
        v = self._snap.get(key, default)
        if v is default:
            self.misses += 1
        else:
            self.hits += 1
        return v

    def put(self, key, value):
        with self._wlock:
            new = OrderedDict(self._snap)
            new[key] = value
            new.move_to_end(key)
            while len(new) > self.capacity:
                new.popitem(last=False)
            self._snap = new

    def get_or_insert(self, key, factory):
        v = self._snap.get(key)
        if v is None:
            v = factory()
            self.put(key, v)
        return v

    def __len__(self):
        return len(self._snap)


class AutoBatcher:
    """Collects single-sample requests and runs ``fn`` once per batch of up to ``max_batch`` samples or after
    ``max_wait_s`` (``auto_batching.rs``): callers get futures; a worker thread stacks the inputs, calls ``fn(batch)`` and
    splits the result."""

    def __init__(self, fn, max_batch: int = 32, max_wait_s: float = 0.002):
        self.fn, self.max_batch, self.max_wait = fn, max_batch, max_wait_s
        self._q: deque = deque()
        self._cv = threading.Condition()
        self._stop = False
        self.batches: list[int] = []
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def submit(self, x: torch.Tensor) -> Future:
        f: Future = Future()
        with self._cv:
            self._q.append((x, f))
            self._cv.notify()
        return f

    def _run(self):
        while True:
            with self._cv:
                while not self._q and not self._stop:
                    self._cv.wait()
                if self._stop and not self._q:
                    return
                deadline = time.monotonic() + self.max_wait
                while len(self._q) < self.max_batch and not self._stop:
                    left = deadline - time.monotonic()
                    if left <= 0:
                        break
                    self._cv.wait(left)
                items = [self._q.popleft() for _ in range(min(self.max_batch, len(self._q)))]
            try:
                out = self.fn(torch.stack([x for x, _ in items]))
                self.batches.append(len(items))
                for i, (_, f) in enumerate(items):
                    f.set_result(out[i])
            except Exception as e:       # noqa: BLE001
                for _, f in items:
                    f.set_exception(e)

    def shutdown(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        self._t.join(2)


class AsyncOps:
    """Runs tensor functions on a thread pool and returns futures (``async_ops.rs``); on a GPU every worker uses its own
    stream so that independent ops overlap."""

    def __init__(self, workers: int = 4):
        self._pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="torsh-async")
        self._streams = threading.local()

    def _call(self, fn, args, kwargs):
        if torch.cuda.is_available():
            s = getattr(self._streams, "s", None)
            if s is None:
                s = self._streams.s = torch.cuda.Stream()
            with torch.cuda.stream(s):
                out = fn(*args, **kwargs)
            s.synchronize()
            return out
        return fn(*args, **kwargs)

    def submit(self, fn, *args, **kwargs) -> Future:
        return self._pool.submit(self._call, fn, args, kwargs)

    def map(self, fn, items) -> list:
        return [f.result() for f in [self.submit(fn, it) for it in items]]

    def shutdown(self):
        self._pool.shutdown(wait=True)


@dataclass
class OpRecord:
    name: str
    shapes: list
    duration_ms: float
    thread: str
    extra: dict = field(default_factory=dict)


class OperationLog:
    """Bounded log of executed operations with shapes and durations (``op_logging.rs``)."""

    def __init__(self, capacity: int = 10000):
        self.records: deque[OpRecord] = deque(maxlen=capacity)
        self.enabled = True

    @contextmanager
    def record(self, name: str, *tensors, **extra):
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.records.append(OpRecord(name, [tuple(t.shape) for t in tensors if isinstance(t, torch.Tensor)],
                                         (time.perf_counter() - t0) * 1e3, threading.current_thread().name, extra))

    def summary(self) -> dict[str, dict]:
        out: dict[str, dict] = {}
        for r in self.records:
            s = out.setdefault(r.name, {"count": 0, "total_ms": 0.0})
            s["count"] += 1
            s["total_ms"] += r.duration_ms
        return out


class TensorTracker:
    """Tracks tensors by weak reference with a tag and creation site; reports what is still alive (``tensor_tracker.rs``)."""

    def __init__(self):
        self._live: dict[int, tuple] = {}
        self.created = self.freed = 0

    def track(self, t: torch.Tensor, tag: str = "") -> torch.Tensor:
        key = id(t)
        nbytes = t.numel() * t.element_size()
        self._live[key] = (tag, tuple(t.shape), str(t.dtype), nbytes)
        self.created += 1
        weakref.finalize(t, self._gone, key)
        return t

    def _gone(self, key):
        if self._live.pop(key, None) is not None:
            self.freed += 1

    def live(self) -> list[tuple]:
        return list(self._live.values())

    def live_bytes(self, tag: str | None = None) -> int:
        return sum(v[3] for v in self._live.values() if tag is None or v[0] == tag)
