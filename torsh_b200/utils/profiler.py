"""Profiler: scoped events, CUDA-event device timing, NVTX ranges, Chrome-trace / JSON / Prometheus export.

Reference: global ``Profiler`` + RAII ``ScopeGuard`` recording ``ProfileEvent{name, category, start_us, duration_us,
thread_id, op_count, flops, bytes}`` (``crates/torsh-profiler/src/core/profiler.rs:14-240``, ``core/scope.rs``), macros
``profile_block! / profile_cuda! / profile_tensor_op!`` (``src/macros.rs:21-417``), Chrome-trace export
(``src/chrome_trace.rs:10-68``); its CUDA side only records what it is told (``src/cuda.rs:21-437``). Here a scope on a
CUDA device brackets the region with CUDA events (resolved lazily, no sync inside the region) and pushes an NVTX
range; ``CommunicationProfiler`` keeps per-collective records with achieved bandwidth
(``crates/torsh-distributed/src/profiling.rs:14-619``).
"""
from __future__ import annotations

import functools
import json
import os
import threading
import time
from contextlib import contextmanager
from dataclasses import asdict, dataclass, field

import torch


@dataclass
class ProfileEvent:
    name: str
    category: str
    start_us: float
    duration_us: float
    thread_id: int
    device_us: float | None = None
    op_count: int = 0
    flops: float = 0.0
    bytes: float = 0.0
    args: dict = field(default_factory=dict)


class Profiler:
    _global = None

    def __init__(self, enabled: bool = True, use_cuda: bool | None = None, nvtx: bool = True):
        self.enabled = enabled
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self.nvtx = nvtx and self.use_cuda
        self.events: list[ProfileEvent] = []
        self._pending: list = []
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()

    @classmethod
    def global_(cls) -> "Profiler":
        if cls._global is None:
            cls._global = cls(enabled=os.environ.get("TORSH_PROFILE", "0") not in ("0", ""))
        return cls._global

    @contextmanager
    def scope(self, name: str, category: str = "op", flops: float = 0.0, bytes: float = 0.0, **args):
        if not self.enabled:
            yield
            return
        ev = None
        if self.use_cuda:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
            if self.nvtx:
                torch.cuda.nvtx.range_push(name)
        t0 = time.perf_counter()
        try:
            yield
        finally:
            dur = (time.perf_counter() - t0) * 1e6
            if ev is not None:
                ev[1].record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
            e = ProfileEvent(name, category, (t0 - self._t0) * 1e6, dur, threading.get_ident(), None, 1, flops, bytes, args)
            with self._lock:
                self.events.append(e)
                if ev is not None:
                    self._pending.append((e, ev))

    def profile(self, name: str | None = None, category: str = "fn"):
        def deco(fn):
            @functools.wraps(fn)
            def wrapped(*a, **kw):
                with self.scope(name or fn.__qualname__, category):
                    return fn(*a, **kw)
            return wrapped
        return deco

    def resolve(self):
        """Synchronise once and fill in the device durations of all finished scopes."""
        if self._pending:
            torch.cuda.synchronize()
            for e, (a, b) in self._pending:
                e.device_us = a.elapsed_time(b) * 1e3
            self._pending.clear()

    def summary(self) -> dict:
        self.resolve()
        out: dict = {}
        for e in self.events:
            s = out.setdefault(e.name, {"count": 0, "host_us": 0.0, "device_us": 0.0, "flops": 0.0, "bytes": 0.0})
            s["count"] += 1
            s["host_us"] += e.duration_us
            s["device_us"] += e.device_us or 0.0
            s["flops"] += e.flops
            s["bytes"] += e.bytes
        for s in out.values():
            t = (s["device_us"] or s["host_us"]) * 1e-6
            s["tflops"] = s["flops"] / t / 1e12 if t > 0 and s["flops"] else 0.0
            s["gbps"] = s["bytes"] / t / 1e9 if t > 0 and s["bytes"] else 0.0
        return out

    def export_chrome_trace(self, path):
        self.resolve()
        tr = [{"name": e.name, "cat": e.category, "ph": "X", "ts": e.start_us, "dur": e.device_us or e.duration_us,
               "pid": os.getpid(), "tid": e.thread_id % 100000, "args": e.args} for e in self.events]
        with open(path, "w") as f:
            json.dump({"traceEvents": tr, "displayTimeUnit": "us"}, f)

    def export_json(self, path):
        self.resolve()
        with open(path, "w") as f:
            json.dump([asdict(e) for e in self.events], f, indent=1)

    def prometheus_text(self, prefix: str = "torsh") -> str:
        lines = []
        for name, s in self.summary().items():
            lab = name.replace('"', "'")
            lines.append(f'{prefix}_scope_count{{name="{lab}"}} {s["count"]}')
            lines.append(f'{prefix}_scope_device_seconds{{name="{lab}"}} {s["device_us"] * 1e-6:.9f}')
            lines.append(f'{prefix}_scope_host_seconds{{name="{lab}"}} {s["host_us"] * 1e-6:.9f}')
        return "\n".join(lines) + "\n"

    def clear(self):
        self.events.clear()
        self._pending.clear()


def profile_block(name: str, category: str = "block", **kw):
    """``profile_block!`` equivalent on the global profiler."""
    return Profiler.global_().scope(name, category, **kw)


@dataclass
class CommunicationEvent:
    op_type: str
    rank: int
    bytes: int
    duration_us: float
    algo: str = ""


class CommunicationProfiler:
    def __init__(self, rank: int = 0):
        self.rank, self.events = rank, []

    @contextmanager
    def record(self, op_type: str, nbytes: int, algo: str = ""):
        if torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            yield
            b.record()
            b.synchronize()
            us = a.elapsed_time(b) * 1e3
        else:
            t0 = time.perf_counter()
            yield
            us = (time.perf_counter() - t0) * 1e6
        self.events.append(CommunicationEvent(op_type, self.rank, nbytes, us, algo))

    def stats(self) -> dict:
        out = {}
        for e in self.events:
            s = out.setdefault(e.op_type, {"count": 0, "bytes": 0, "us": []})
            s["count"] += 1
            s["bytes"] += e.bytes
            s["us"].append(e.duration_us)
        for s in out.values():
            u = sorted(s.pop("us"))
            s["p50_us"], s["p99_us"] = u[len(u) // 2], u[min(len(u) - 1, int(len(u) * 0.99))]
            s["gbps"] = s["bytes"] / (sum(u) * 1e-6) / 1e9 if sum(u) > 0 else 0.0
        return out

    def export_json(self, path):
        with open(path, "w") as f:
            json.dump({"events": [asdict(e) for e in self.events], "stats": self.stats()}, f, indent=1)



class DeviceRangeProfiler:
    """Native scoped ranges (``csrc/kernels/runtime.cu``): every range is an NVTX range for Nsight tools and a pair of
    CUDA events on the launching stream; ``collect()`` returns device durations, ``chrome_trace()`` the trace JSON."""

    def __init__(self):
        import ctypes

        from .. import _native as nv
        self._nv, self._ct = nv, ctypes
        self._lib = nv.require_cuda()
        self._lib.tb_prof_push.argtypes = [ctypes.c_char_p, ctypes.c_void_p]
        self._lib.tb_prof_pop.argtypes = [ctypes.c_void_p]
        self.records: list[dict] = []

    def range(self, name: str):
        prof = self

        class _R:
            def __enter__(self_inner):
                prof._nv.check(prof._lib.tb_prof_push(name.encode()[:63], prof._nv.stream_ptr()), "prof_push")

            def __exit__(self_inner, *a):
                prof._nv.check(prof._lib.tb_prof_pop(prof._nv.stream_ptr()), "prof_pop")
        return _R()

    def collect(self, cap: int = 4096) -> list[dict]:
        ct = self._ct
        names = ct.create_string_buffer(64 * cap)
        depth, host, dev = (ct.c_int * cap)(), (ct.c_double * cap)(), (ct.c_float * cap)()
        n = self._lib.tb_prof_collect(names, depth, host, dev, cap)
        out = [{"name": names.raw[64 * i: 64 * i + 64].split(b"\0", 1)[0].decode(), "depth": depth[i], "host_us": host[i],
                "device_us": dev[i]} for i in range(n)]
        self.records += out
        return out

    def chrome_trace(self) -> str:
        import json
        return json.dumps({"traceEvents": [{"name": r["name"], "ph": "X", "ts": r["host_us"], "dur": r["device_us"], "pid": 0,
                                            "tid": r["depth"], "cat": "cuda"} for r in self.records]})


# ------------------------------------------------------------------------------------------------ core profiling API
def profile_closure(fn, *args, name: str | None = None, repeats: int = 1, **kwargs):
    """``crates/torsh-core/src/profiling.rs``: run ``fn`` under the global profiler and return ``(result, mean ms)``;
    on a GPU the time is taken after a synchronise so that it covers the launched work."""
    import time as _time

    import torch
    label = name or getattr(fn, "__name__", "closure")
    out, t0 = None, _time.perf_counter()
    with profile_block(label, category="closure"):
        for _ in range(repeats):
            out = fn(*args, **kwargs)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    return out, (_time.perf_counter() - t0) * 1e3 / repeats


class PerformanceProfiler:
    """Named timers with call counts and simple statistics (``PerformanceProfiler`` of ``torsh-core``)."""

    def __init__(self):
        self.samples: dict[str, list[float]] = {}

    def time(self, name: str):
        import contextlib
        import time as _time

        @contextlib.contextmanager
        def cm():
            t0 = _time.perf_counter()
            try:
                yield
            finally:
                self.samples.setdefault(name, []).append((_time.perf_counter() - t0) * 1e3)
        return cm()

    def stats(self, name: str) -> dict:
        xs = sorted(self.samples.get(name, []))
        if not xs:
            return {"count": 0}
        return {"count": len(xs), "mean_ms": sum(xs) / len(xs), "min_ms": xs[0], "max_ms": xs[-1],
                "p50_ms": xs[len(xs) // 2], "p95_ms": xs[min(len(xs) - 1, int(0.95 * len(xs)))]}

    def report(self) -> dict:
        return {k: self.stats(k) for k in self.samples}


class OperationTrace:
    """``trace_operation`` (``crates/torsh-core/src/op_trace.rs``): a bounded, nestable trace of operations with inputs'
    shapes and dtypes; ``format()`` prints the call tree."""

    def __init__(self, capacity: int = 4096):
        self.capacity, self.events, self._depth = capacity, [], 0

    def trace_operation(self, name: str, *tensors):
        import contextlib

        @contextlib.contextmanager
        def cm():
            if len(self.events) < self.capacity:
                self.events.append((self._depth, name, [(tuple(t.shape), str(t.dtype)) for t in tensors if hasattr(t, "shape")]))
            self._depth += 1
            try:
                yield
            finally:
                self._depth -= 1
        return cm()

    def format(self) -> str:
        return "\n".join("  " * d + f"{n} {sig}" for d, n, sig in self.events)


class PerfRegressionDetector:
    """Compares fresh timings with stored baselines (``perf_regression`` of ``torsh-core`` / the profiler crate's regression
    detection): a measurement slower than ``baseline x (1 + tolerance)`` is a regression; baselines live in a JSON file and
    improve monotonically when ``update_on_improvement`` is set."""

    def __init__(self, path: str | None = None, tolerance: float = 0.10, update_on_improvement: bool = True):
        import json
        import os
        self.path, self.tolerance, self.update = path, tolerance, update_on_improvement
        self.baselines: dict[str, float] = {}
        if path and os.path.exists(path):
            with open(path) as f:
                self.baselines = json.load(f)

    def check(self, name: str, value_ms: float) -> dict:
        base = self.baselines.get(name)
        if base is None:
            self.baselines[name] = value_ms
            verdict = {"name": name, "status": "new", "baseline_ms": None, "value_ms": value_ms, "ratio": None}
        else:
            ratio = value_ms / base
            status = "regression" if ratio > 1 + self.tolerance else "improvement" if ratio < 1 - self.tolerance else "ok"
            if status == "improvement" and self.update:
                self.baselines[name] = value_ms
            verdict = {"name": name, "status": status, "baseline_ms": base, "value_ms": value_ms, "ratio": ratio}
        if self.path:
            import json
            with open(self.path, "w") as f:
                json.dump(self.baselines, f, indent=1)
        return verdict
