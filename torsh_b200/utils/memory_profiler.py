"""Memory profiling and leak detection (``crates/torsh-backend/src/memory_profiler/*``, ``memory_profiling/*`` and
``crates/torsh-core/src/memory_debug.rs``): named scopes record how much device (or, without a GPU, Python heap) memory
they allocated and kept, a timeline of samples can be exported, and two snapshots of the live tensors are compared to
name what leaked between them."""
from __future__ import annotations

import gc
import json
import time
import tracemalloc
from collections import Counter
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field

import torch


def _device_bytes() -> tuple[int, int]:
    if torch.cuda.is_available():
        return torch.cuda.memory_allocated(), torch.cuda.max_memory_allocated()
    if not tracemalloc.is_tracing():
        tracemalloc.start()
    cur, peak = tracemalloc.get_traced_memory()
    return cur, peak


@dataclass
class ScopeRecord:
    name: str
    start_bytes: int
    end_bytes: int
    peak_bytes: int
    duration_ms: float

    @property
    def retained(self) -> int:
        return self.end_bytes - self.start_bytes


@dataclass
class TensorSnapshot:
    """Live tensors grouped by (shape, dtype, device)."""
    counts: Counter = field(default_factory=Counter)
    nbytes: int = 0


class MemoryProfiler:
    def __init__(self):
        self.scopes: list[ScopeRecord] = []
        self.timeline: list[tuple[float, int]] = []
        self._t0 = time.perf_counter()

    @contextmanager
    def scope(self, name: str):
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
        elif tracemalloc.is_tracing():
            tracemalloc.reset_peak()
        start, _ = _device_bytes()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            end, peak = _device_bytes()
            self.scopes.append(ScopeRecord(name, start, end, max(peak, end), (time.perf_counter() - t0) * 1e3))
            self.sample()

    def sample(self):
        self.timeline.append((time.perf_counter() - self._t0, _device_bytes()[0]))

    @staticmethod
    def snapshot() -> TensorSnapshot:
        gc.collect()
        snap, seen = TensorSnapshot(), set()
        for o in gc.get_objects():
            try:
                if isinstance(o, torch.Tensor) and o.data_ptr() and o.untyped_storage().data_ptr() not in seen:
                    seen.add(o.untyped_storage().data_ptr())
                    snap.counts[(tuple(o.shape), str(o.dtype), str(o.device))] += 1
                    snap.nbytes += o.untyped_storage().nbytes()
            except Exception:
                continue
        return snap

    @staticmethod
    def leaks(before: TensorSnapshot, after: TensorSnapshot) -> list[tuple[tuple, int]]:
        """Tensor groups that exist more often in ``after`` than in ``before``, largest growth first."""
        grown = [(k, n - before.counts.get(k, 0)) for k, n in after.counts.items() if n > before.counts.get(k, 0)]
        return sorted(grown, key=lambda kv: -kv[1])

    def report(self) -> dict:
        return {"scopes": [dict(asdict(s), retained=s.retained) for s in self.scopes],
                "peak_bytes": max((s.peak_bytes for s in self.scopes), default=0),
                "timeline": self.timeline}

    def export_json(self, path: str):
        with open(path, "w") as f:
            json.dump(self.report(), f, indent=1)
