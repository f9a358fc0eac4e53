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
