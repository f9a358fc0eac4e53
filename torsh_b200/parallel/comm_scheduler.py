"""Communication scheduler (``crates/torsh-distributed/src/communication_scheduler.rs:37-1256``): a priority queue of
collective tasks executed by a worker thread on a dedicated CUDA stream (or inline on CPU), with FIFO / priority /
smallest-first strategies, an optional bandwidth budget and per-task futures.  Gradient buckets enter with high
priority, parameter prefetches with low priority, so a late bucket is never stuck behind a prefetch."""
from __future__ import annotations

import enum
import heapq
import itertools
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable


class Priority(enum.IntEnum):
    CRITICAL = 0
    HIGH = 1
    NORMAL = 2
    LOW = 3


class Strategy(enum.Enum):
    FIFO = "fifo"
    PRIORITY = "priority"
    SMALLEST_FIRST = "smallest_first"


@dataclass(order=True)
class _Task:
    key: tuple
    fn: Callable = field(compare=False)
    nbytes: int = field(compare=False)
    future: Future = field(compare=False)
    name: str = field(compare=False, default="")


class CommunicationScheduler:
    def __init__(self, strategy: Strategy = Strategy.PRIORITY, bandwidth_limit_gbs: float | None = None, stream=None,
                 max_in_flight: int = 4):
        self.strategy, self.bw_limit, self.stream = strategy, bandwidth_limit_gbs, stream
        self._heap: list[_Task] = []
        self._seq = itertools.count()
        self._cv = threading.Condition()
        self._stop = False
        self.stats = {"submitted": 0, "completed": 0, "bytes": 0, "failed": 0, "throttle_s": 0.0}
        self.order: list[str] = []   # names in execution order (observability, tests)
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def submit(self, fn: Callable, nbytes: int = 0, priority: Priority = Priority.NORMAL, name: str = "") -> Future:
        fut: Future = Future()
        seq = next(self._seq)
        key = {Strategy.FIFO: (seq,), Strategy.PRIORITY: (int(priority), seq), Strategy.SMALLEST_FIRST: (nbytes, seq)}[self.strategy]
        with self._cv:
            heapq.heappush(self._heap, _Task(key, fn, nbytes, fut, name))
            self.stats["submitted"] += 1
            self._cv.notify()
        return fut

    def _run(self):
        window_start, window_bytes = time.perf_counter(), 0
        while True:
            with self._cv:
                while not self._heap and not self._stop:
                    self._cv.wait()
                if self._stop and not self._heap:
                    return
                task = heapq.heappop(self._heap)
            if self.bw_limit:
                budget = self.bw_limit * 1e9
                elapsed = time.perf_counter() - window_start
                need = (window_bytes + task.nbytes) / budget
                if need > elapsed:
                    time.sleep(need - elapsed)
                    self.stats["throttle_s"] += need - elapsed
                window_bytes += task.nbytes
            try:
                if self.stream is not None:
                    import torch
                    with torch.cuda.stream(self.stream):
                        out = task.fn()
                else:
                    out = task.fn()
                self.order.append(task.name)
                self.stats["completed"] += 1
                self.stats["bytes"] += task.nbytes
                task.future.set_result(out)
            except Exception as e:
                self.stats["failed"] += 1
                task.future.set_exception(e)

    def pause(self):
        """Hold the queue (tasks keep accumulating); returns a function that releases it."""
        gate = threading.Event()
        self.submit(gate.wait, priority=Priority.CRITICAL, name="__gate")
        return gate.set

    def drain(self, timeout: float = 30.0) -> None:
        self.submit(lambda: None, priority=Priority.LOW, name="__drain").result(timeout)

    def shutdown(self):
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._thread.join(5)


class CollectiveAlgorithm(enum.Enum):
    """``crates/torsh-distributed/src/nccl_optimization.rs``: ring / tree / hierarchical selection. On one NVSwitch box
    the device-side choice is between the one-shot kernel (latency-bound sizes), the two-shot kernel over peer memory,
    and the in-switch (NVLS ``multimem``) reduction."""
    ONE_SHOT = "one_shot"
    TWO_SHOT_PEER = "two_shot_peer"
    NVLS = "nvls"
    RING = "ring"
    TREE = "tree"
    HIERARCHICAL = "hierarchical"


@dataclass
class _PendingOp:
    name: str
    nbytes: int
    priority: Priority
    fn: Callable
    fusable: bool = True


class NcclScheduler:
    """Multi-stream collective scheduler with op fusion (``nccl_optimization.rs:22-1170``: ``NcclScheduler``,
    ``FusedNcclOp``): ops are queued, small fusable ops of equal priority are merged until ``fusion_bytes``, every
    (fused) op goes to the least-loaded of ``num_streams`` streams, and the algorithm is chosen from the message size
    and the topology. Streams are CUDA streams when a GPU is present, otherwise plain counters (the logic is the same
    and is what the CPU tests drive)."""

    def __init__(self, num_streams: int = 2, fusion_bytes: int = 4 << 20, world: int = 1, ranks_per_node: int | None = None,
                 has_multicast: bool = False, streams=None):
        self.num_streams, self.fusion_bytes, self.world = num_streams, fusion_bytes, world
        self.ranks_per_node = ranks_per_node or world
        self.has_multicast = has_multicast
        self.streams = streams
        self.load = [0] * num_streams                # bytes queued per stream
        self.queue: list[_PendingOp] = []
        self.stats = {"ops": 0, "fused_groups": 0, "fused_ops": 0, "bytes": 0, "per_stream": [0] * num_streams}
        self.log: list[tuple[int, list[str], CollectiveAlgorithm]] = []

    def choose_algorithm(self, nbytes: int) -> CollectiveAlgorithm:
        if self.world > self.ranks_per_node:
            return CollectiveAlgorithm.HIERARCHICAL if nbytes >= (256 << 10) else CollectiveAlgorithm.TREE
        if nbytes <= (128 << 10):
            return CollectiveAlgorithm.ONE_SHOT
        if self.has_multicast and self.world > 2:
            return CollectiveAlgorithm.NVLS
        return CollectiveAlgorithm.TWO_SHOT_PEER

    def enqueue(self, name: str, nbytes: int, fn: Callable, priority: Priority = Priority.NORMAL, fusable: bool = True):
        self.queue.append(_PendingOp(name, nbytes, priority, fn, fusable))
        self.stats["ops"] += 1

    def _groups(self) -> list[list[_PendingOp]]:
        ops = sorted(self.queue, key=lambda o: int(o.priority))       # stable: submission order inside a priority
        groups: list[list[_PendingOp]] = []
        for op in ops:
            last = groups[-1] if groups else None
            if (last is not None and op.fusable and last[0].fusable and last[0].priority == op.priority
                    and sum(o.nbytes for o in last) + op.nbytes <= self.fusion_bytes):
                last.append(op)
            else:
                groups.append([op])
        return groups

    def flush(self) -> list:
        """Issue everything queued; returns the results of the ops in issue order."""
        results = []
        for grp in self._groups():
            nbytes = sum(o.nbytes for o in grp)
            sid = min(range(self.num_streams), key=lambda i: self.load[i])
            self.load[sid] += nbytes
            alg = self.choose_algorithm(nbytes)
            self.log.append((sid, [o.name for o in grp], alg))
            if len(grp) > 1:
                self.stats["fused_groups"] += 1
                self.stats["fused_ops"] += len(grp)
            self.stats["bytes"] += nbytes
            self.stats["per_stream"][sid] += 1
            if self.streams is not None:
                import torch
                with torch.cuda.stream(self.streams[sid]):
                    results.extend(o.fn() for o in grp)
            else:
                results.extend(o.fn() for o in grp)
        self.queue.clear()
        return results

    def complete(self, stream_id: int, nbytes: int):
        """Bookkeeping when a stream has drained ``nbytes`` (called from an event callback or after a synchronise)."""
        self.load[stream_id] = max(0, self.load[stream_id] - nbytes)
