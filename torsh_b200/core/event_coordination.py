"""Cross-stream coordination (``crates/torsh-backend/src/cuda/event_coordination.rs:53-686``): an
:class:`OperationCoordinator` that turns declared dependencies between operations on different streams into event
record / wait pairs and refuses dependency cycles (the deadlock check of ``:407-478``), a :class:`CrossStreamBarrier`
and an :class:`AsyncEventWaiter` that runs callbacks when events complete.

Streams and events are anything with ``record(stream)`` / ``wait(stream)`` / ``query()``: ``core.runtime.Event`` and
``torch.cuda`` streams on a GPU, or the :class:`HostEvent` stand-in that the CPU tests (and CPU-only runs) use."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field


class HostEvent:
    """Event for code paths without a GPU: complete as soon as it has been recorded."""

    def __init__(self):
        self._done = threading.Event()
        self.recorded_on = None
        self.waited_by: list = []

    def record(self, stream=None):
        self.recorded_on = stream
        self._done.set()

    def wait(self, stream=None):
        self.waited_by.append(stream)

    def query(self) -> bool:
        return self._done.is_set()

    def synchronize(self):
        self._done.wait()


def _new_event():
    try:
        import torch
        if torch.cuda.is_available():
            from .runtime import Event
            return Event()
    except Exception:
        pass
    return HostEvent()


class DependencyCycleError(RuntimeError):
    """Raised when a new dependency would make two streams wait for each other for ever."""


@dataclass
class _Op:
    name: str
    stream: object
    deps: list[str] = field(default_factory=list)
    event: object | None = None
    issued: bool = False


class OperationCoordinator:
    """Declare operations (``add_operation(name, stream, depends_on=[...])``), then ``issue(name, fn)``: before ``fn``
    runs, the operation's stream waits for the events of its dependencies on other streams; afterwards an event is
    recorded for its own dependants. Same-stream dependencies need no event (stream order already gives them)."""

    def __init__(self, event_factory=_new_event):
        self.ops: dict[str, _Op] = {}
        self._event_factory = event_factory
        self.stats = {"events_recorded": 0, "cross_stream_waits": 0, "same_stream_skipped": 0}

    def add_operation(self, name: str, stream, depends_on=()):
        if name in self.ops:
            raise ValueError(f"operation {name!r} already declared")
        for d in depends_on:
            if d not in self.ops:
                raise KeyError(f"{name!r} depends on undeclared operation {d!r}")
        self.ops[name] = _Op(name, stream, list(depends_on))

    def add_dependency(self, name: str, on: str):
        """Late edge; rejected when ``on`` already (transitively) depends on ``name``."""
        if self._reaches(on, name):
            raise DependencyCycleError(f"{name!r} -> {on!r} would close a cycle: {' -> '.join(self._path(on, name))} -> {on}")
        self.ops[name].deps.append(on)

    def _reaches(self, src: str, dst: str) -> bool:
        return bool(self._path(src, dst))

    def _path(self, src: str, dst: str) -> list[str]:
        stack, seen = [(src, [src])], set()
        while stack:
            cur, path = stack.pop()
            if cur == dst:
                return path
            if cur in seen:
                continue
            seen.add(cur)
            stack.extend((d, path + [d]) for d in self.ops[cur].deps)
        return []

    def detect_deadlocks(self) -> list[list[str]]:
        """Cycles among the declared operations (empty when the graph is a DAG)."""
        cycles, state = [], {}

        def visit(n, path):
            state[n] = 1
            for d in self.ops[n].deps:
                if state.get(d) == 1:
                    cycles.append(path[path.index(d):] + [d] if d in path else [n, d])
                elif d not in state:
                    visit(d, path + [d])
            state[n] = 2
        for n in self.ops:
            if n not in state:
                visit(n, [n])
        return cycles

    def order(self) -> list[str]:
        """A valid issue order (topological); raises on cycles."""
        if self.detect_deadlocks():
            raise DependencyCycleError(f"dependency cycle: {self.detect_deadlocks()[0]}")
        out, done = [], set()

        def visit(n):
            if n in done:
                return
            for d in self.ops[n].deps:
                visit(d)
            done.add(n)
            out.append(n)
        for n in self.ops:
            visit(n)
        return out

    def issue(self, name: str, fn=None):
        op = self.ops[name]
        for d in op.deps:
            dep = self.ops[d]
            if not dep.issued:
                raise RuntimeError(f"{name!r} issued before its dependency {d!r}")
            if dep.stream is op.stream:
                self.stats["same_stream_skipped"] += 1
                continue
            dep.event.wait(op.stream)
            self.stats["cross_stream_waits"] += 1
        out = fn() if fn is not None else None
        op.event = self._event_factory()
        op.event.record(op.stream)
        op.issued = True
        self.stats["events_recorded"] += 1
        return out

    def run(self, fns: dict):
        """Issue every declared operation in dependency order; ``fns[name]`` is its body."""
        return {n: self.issue(n, fns.get(n)) for n in self.order()}


class CrossStreamBarrier:
    """All participating streams continue only after every one of them has reached the barrier: each records an event,
    and each waits for the events of all the others."""

    def __init__(self, streams, event_factory=_new_event):
        self.streams, self._event_factory = list(streams), event_factory

    def arrive_and_wait(self):
        events = []
        for s in self.streams:
            e = self._event_factory()
            e.record(s)
            events.append(e)
        for i, s in enumerate(self.streams):
            for j, e in enumerate(events):
                if i != j:
                    e.wait(s)
        return events


class AsyncEventWaiter:
    """Polls registered events on a helper thread and runs their callbacks on completion (the reference's
    ``AsyncEventWaiter``); ``timeout_s`` bounds every wait and reports the event as timed out instead of blocking."""

    def __init__(self, poll_interval_s: float = 0.0005):
        self.poll, self._items, self._lock = poll_interval_s, [], threading.Lock()
        self._stop = threading.Event()
        self.completed, self.timed_out = 0, 0
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def on_complete(self, event, callback, timeout_s: float = 30.0, on_timeout=None):
        with self._lock:
            self._items.append((event, callback, time.monotonic() + timeout_s, on_timeout))

    def _run(self):
        while not self._stop.is_set():
            with self._lock:
                items, self._items = self._items, []
            keep = []
            for ev, cb, deadline, on_to in items:
                if ev.query():
                    self.completed += 1
                    cb()
                elif time.monotonic() >= deadline:
                    self.timed_out += 1
                    if on_to is not None:
                        on_to()
                else:
                    keep.append((ev, cb, deadline, on_to))
            with self._lock:
                self._items = keep + self._items
            time.sleep(self.poll)

    def pending(self) -> int:
        with self._lock:
            return len(self._items)

    def shutdown(self):
        self._stop.set()
        self._thread.join(2)
