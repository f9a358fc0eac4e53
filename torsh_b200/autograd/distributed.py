"""Distributed gradient accumulation and synchronisation scheduling
(``crates/torsh-autograd/src/distributed/accumulator.rs:24-1009``, ``sync.rs:10-357``): parameter groups whose gradients
are accumulated over micro-batches and synchronised every ``sync_every`` steps, a priority scheduler that keeps at most
``max_concurrent`` synchronisations in flight and returns handles, and a network-health record that decides whether to
compress. The reductions themselves go through ``torch.distributed`` (NCCL / gloo) or, for flat symmetric buffers on
GPUs, the fused kernels of ``parallel.collectives``; with no process group everything degrades to a single rank."""
from __future__ import annotations

import heapq
import itertools
import threading
import time
from collections import deque
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class NetworkHealth:
    """Rolling latency / bandwidth / failure record; ``should_compress`` turns on when the link degrades."""
    window: int = 32
    latencies_ms: deque = field(default_factory=lambda: deque(maxlen=32))
    bandwidths_gbs: deque = field(default_factory=lambda: deque(maxlen=32))
    failures: int = 0
    successes: int = 0

    def record(self, nbytes: int, seconds: float, ok: bool = True):
        if ok:
            self.successes += 1
            self.latencies_ms.append(seconds * 1e3)
            if seconds > 0:
                self.bandwidths_gbs.append(nbytes / seconds / 1e9)
        else:
            self.failures += 1

    @property
    def failure_rate(self) -> float:
        n = self.failures + self.successes
        return self.failures / n if n else 0.0

    @property
    def mean_bandwidth_gbs(self) -> float:
        return sum(self.bandwidths_gbs) / len(self.bandwidths_gbs) if self.bandwidths_gbs else 0.0

    def should_compress(self, min_gbs: float = 1.0, max_failure_rate: float = 0.05) -> bool:
        return bool(self.bandwidths_gbs) and (self.mean_bandwidth_gbs < min_gbs or self.failure_rate > max_failure_rate)


class AsyncSyncHandle:
    """Result of a scheduled synchronisation: ``wait()`` blocks until the reduction has finished."""

    def __init__(self, name: str):
        self.name, self._done, self.error, self.seconds = name, threading.Event(), None, 0.0

    def _finish(self, seconds: float, error=None):
        self.seconds, self.error = seconds, error
        self._done.set()

    def is_done(self) -> bool:
        return self._done.is_set()

    def wait(self, timeout: float | None = 30.0) -> bool:
        if not self._done.wait(timeout):
            raise TimeoutError(f"gradient synchronisation of {self.name!r} did not finish in {timeout}s")
        if self.error is not None:
            raise self.error
        return True


class GradientSyncScheduler:
    """Priority queue of pending reductions (lower value first; ties in submission order) with at most
    ``max_concurrent`` running at a time on worker threads."""

    def __init__(self, max_concurrent: int = 2, health: NetworkHealth | None = None):
        self.max_concurrent, self.health = max_concurrent, health or NetworkHealth()
        self._heap, self._seq = [], itertools.count()
        self._cv = threading.Condition()
        self._running, self._stop = 0, False
        self.order: list[str] = []
        self._workers = [threading.Thread(target=self._run, daemon=True) for _ in range(max_concurrent)]
        for w in self._workers:
            w.start()

    def schedule(self, name: str, fn, nbytes: int = 0, priority: int = 10) -> AsyncSyncHandle:
        h = AsyncSyncHandle(name)
        with self._cv:
            heapq.heappush(self._heap, (priority, next(self._seq), name, fn, nbytes, h))
            self._cv.notify()
        return h

    def _run(self):
        while True:
            with self._cv:
                while not self._heap and not self._stop:
                    self._cv.wait()
                if self._stop and not self._heap:
                    return
                _, _, name, fn, nbytes, h = heapq.heappop(self._heap)
                self.order.append(name)
            t0 = time.perf_counter()
            try:
                fn()
                dt = time.perf_counter() - t0
                self.health.record(nbytes, dt, True)
                h._finish(dt)
            except Exception as e:      # noqa: BLE001
                self.health.record(nbytes, 0.0, False)
                h._finish(time.perf_counter() - t0, e)

    def shutdown(self):
        with self._cv:
            self._stop = True
            self._cv.notify_all()
        for w in self._workers:
            w.join(2)


SyncCoordinator = GradientSyncScheduler


@dataclass
class GradParamGroup:
    name: str
    params: list
    sync_every: int = 1
    priority: int = 10
    compressor: object | None = None


class DistributedGradAccumulator:
    """Accumulates gradients of named parameter groups over micro-batches and averages them across ranks every
    ``sync_every`` calls of :meth:`step` (``GradientAccumulation`` + ``DistributedGradAccumulator``)."""

    def __init__(self, group=None, scheduler: GradientSyncScheduler | None = None):
        self.group, self.scheduler = group, scheduler
        self.groups: dict[str, GradParamGroup] = {}
        self.acc: dict[int, torch.Tensor] = {}
        self.micro_steps = 0
        self.stats = {"syncs": 0, "bytes": 0, "compressed": 0}

    def add_param_group(self, name: str, params, sync_every: int = 1, priority: int = 10, compressor=None):
        self.groups[name] = GradParamGroup(name, [p for p in params if p.requires_grad], sync_every, priority, compressor)

    def accumulate(self):
        """Fold the current ``p.grad`` of every group into the accumulators and clear ``p.grad``."""
        for g in self.groups.values():
            for p in g.params:
                if p.grad is None:
                    continue
                a = self.acc.get(id(p))
                if a is None:
                    self.acc[id(p)] = p.grad.detach().clone()
                else:
                    a.add_(p.grad)
                p.grad = None
        self.micro_steps += 1

    def _world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _reduce_group(self, g: GradParamGroup, scale: float):
        world = self._world()
        for p in g.params:
            a = self.acc.get(id(p))
            if a is None:
                continue
            a.mul_(scale)
            if g.compressor is not None:
                payload = g.compressor.compress(a)
                a.copy_(g.compressor.decompress(payload, a.shape, a.dtype, a.device))
                self.stats["compressed"] += 1
            if world > 1:
                dist.all_reduce(a, group=self.group)
                a.div_(world)
            self.stats["bytes"] += a.numel() * a.element_size()
            p.grad = a
            self.acc.pop(id(p))
        self.stats["syncs"] += 1

    def step(self) -> list[AsyncSyncHandle]:
        """Call once per optimizer step (after the last ``accumulate``): groups whose period has come are averaged over
        the micro-batches and the ranks and written back to ``p.grad``. Returns the handles of scheduled reductions
        (empty without a scheduler: the reductions have already run)."""
        handles = []
        scale = 1.0 / max(self.micro_steps, 1)
        self._opt_steps = getattr(self, "_opt_steps", 0) + 1
        for g in sorted(self.groups.values(), key=lambda x: x.priority):
            if self._opt_steps % g.sync_every:
                continue
            if self.scheduler is None:
                self._reduce_group(g, scale)
            else:
                nbytes = sum(self.acc[id(p)].numel() * 4 for p in g.params if id(p) in self.acc)
                handles.append(self.scheduler.schedule(g.name, lambda g=g: self._reduce_group(g, scale), nbytes, g.priority))
        self.micro_steps = 0
        return handles
