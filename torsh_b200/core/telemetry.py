"""Structured telemetry: levelled log events with fields and error codes, spans with attributes / events / parent links,
and readiness / liveness health checks with a JSON report. Reference: crates/torsh-core/src/{telemetry,health}.rs.
"""
from __future__ import annotations

import enum
import json
import threading
import time
from dataclasses import dataclass, field


class LogLevel(enum.IntEnum):
    TRACE = 0
    DEBUG = 1
    INFO = 2
    WARN = 3
    ERROR = 4

    def is_enabled(self, minimum: "LogLevel") -> bool:
        return self >= minimum


class ErrorCode(enum.IntEnum):
    OK = 0
    INVALID_ARGUMENT = 1001
    SHAPE_MISMATCH = 1002
    DTYPE_MISMATCH = 1003
    DEVICE_MISMATCH = 1004
    OUT_OF_MEMORY = 2001
    KERNEL_TIMEOUT = 2002
    KERNEL_CHECK_FAILED = 2003
    COMMUNICATION = 3001
    RANK_FAILURE = 3002
    IO = 4001
    NOT_IMPLEMENTED = 5001
    INTERNAL = 9001

    @staticmethod
    def from_exception(e: BaseException) -> "ErrorCode":
        name = type(e).__name__
        table = {"ShapeMismatch": ErrorCode.SHAPE_MISMATCH, "KernelTimeout": ErrorCode.KERNEL_TIMEOUT, "KernelCheckFailed": ErrorCode.KERNEL_CHECK_FAILED,
                 "MemoryError": ErrorCode.OUT_OF_MEMORY, "OutOfMemoryError": ErrorCode.OUT_OF_MEMORY, "NotImplementedError": ErrorCode.NOT_IMPLEMENTED,
                 "ValueError": ErrorCode.INVALID_ARGUMENT, "TypeError": ErrorCode.DTYPE_MISMATCH, "OSError": ErrorCode.IO, "FileNotFoundError": ErrorCode.IO,
                 "TimeoutError": ErrorCode.COMMUNICATION, "ConnectionError": ErrorCode.COMMUNICATION}
        for k, v in table.items():
            if k in name or any(k == b.__name__ for b in type(e).__mro__):
                return v
        return ErrorCode.INTERNAL


@dataclass
class LogEvent:
    level: LogLevel
    message: str
    module: str = ""
    fields: dict = field(default_factory=dict)
    span_id: int | None = None
    error_code: ErrorCode | None = None
    timestamp: float = field(default_factory=time.time)

    def format_structured(self) -> str:
        d = {"ts": round(self.timestamp, 6), "level": self.level.name, "module": self.module, "msg": self.message, **self.fields}
        if self.span_id is not None:
            d["span_id"] = self.span_id
        if self.error_code is not None:
            d["error_code"] = int(self.error_code)
        return json.dumps(d, default=str)


@dataclass
class SpanMetrics:
    span_id: int
    name: str
    parent_id: int | None
    duration_s: float
    attributes: dict
    events: list


@dataclass
class TelemetryConfig:
    min_level: LogLevel = LogLevel.INFO
    max_events: int = 10000
    sink: object = None                 # callable(str) receiving each structured line


class TelemetrySystem:
    def __init__(self, config: TelemetryConfig | None = None):
        self.cfg = config or TelemetryConfig()
        self._lock = threading.Lock()
        self.events: list[LogEvent] = []
        self._open: dict[int, dict] = {}
        self.finished: list[SpanMetrics] = []
        self._next = 1
        self.dropped = 0

    def log(self, level: LogLevel, message: str, module: str = "", span_id: int | None = None, error_code: ErrorCode | None = None, **fields):
        if not LogLevel(level).is_enabled(self.cfg.min_level):
            return None
        ev = LogEvent(LogLevel(level), message, module, fields, span_id, error_code)
        with self._lock:
            if len(self.events) >= self.cfg.max_events:
                self.events.pop(0)
                self.dropped += 1
            self.events.append(ev)
        if self.cfg.sink is not None:
            self.cfg.sink(ev.format_structured())
        return ev

    def start_span(self, name: str, parent_id: int | None = None) -> int:
        with self._lock:
            sid = self._next
            self._next += 1
            self._open[sid] = {"name": name, "parent": parent_id, "t0": time.perf_counter(), "attrs": {}, "events": []}
        return sid

    def span_add_attribute(self, span_id: int, key: str, value):
        self._open[span_id]["attrs"][key] = value

    def span_add_event(self, span_id: int, name: str, **fields):
        s = self._open[span_id]
        s["events"].append({"name": name, "at_s": time.perf_counter() - s["t0"], **fields})

    def end_span(self, span_id: int) -> SpanMetrics | None:
        with self._lock:
            s = self._open.pop(span_id, None)
            if s is None:
                return None
            m = SpanMetrics(span_id, s["name"], s["parent"], time.perf_counter() - s["t0"], s["attrs"], s["events"])
            self.finished.append(m)
            return m

    def span(self, name: str, parent_id: int | None = None):
        sys_ = self

        class _Ctx:
            def __enter__(self_inner):
                self_inner.id = sys_.start_span(name, parent_id)
                return self_inner.id

            def __exit__(self_inner, et, ev, tb):
                if ev is not None:
                    sys_.span_add_attribute(self_inner.id, "error", repr(ev))
                    sys_.log(LogLevel.ERROR, str(ev), span_id=self_inner.id, error_code=ErrorCode.from_exception(ev))
                sys_.end_span(self_inner.id)
                return False
        return _Ctx()

    def get_events(self, level: LogLevel | None = None):
        return [e for e in self.events if level is None or e.level >= level]


_global = TelemetrySystem()


def telemetry() -> TelemetrySystem:
    return _global


# ---- health --------------------------------------------------------------------------------------------------------
class HealthStatus(enum.Enum):
    HEALTHY = "healthy"
    DEGRADED = "degraded"
    UNHEALTHY = "unhealthy"

    def is_operational(self) -> bool:
        return self is not HealthStatus.UNHEALTHY

    def http_status_code(self) -> int:
        return 200 if self.is_operational() else 503


@dataclass
class HealthCheckResult:
    name: str
    status: HealthStatus
    message: str = ""
    error_code: ErrorCode | None = None
    metadata: dict = field(default_factory=dict)
    duration_s: float = 0.0


@dataclass
class HealthReport:
    checks: list
    timestamp: float = field(default_factory=time.time)

    @property
    def status(self) -> HealthStatus:
        if any(c.status is HealthStatus.UNHEALTHY for c in self.checks):
            return HealthStatus.UNHEALTHY
        if any(c.status is HealthStatus.DEGRADED for c in self.checks):
            return HealthStatus.DEGRADED
        return HealthStatus.HEALTHY

    def failing_checks(self):
        return [c for c in self.checks if c.status is not HealthStatus.HEALTHY]

    def summary(self) -> str:
        bad = self.failing_checks()
        return f"{self.status.value}: {len(self.checks) - len(bad)}/{len(self.checks)} checks passing" + (
            "; failing: " + ", ".join(c.name for c in bad) if bad else "")

    def to_json(self) -> str:
        return json.dumps({"status": self.status.value, "http": self.status.http_status_code(), "timestamp": self.timestamp,
                           "checks": [{"name": c.name, "status": c.status.value, "message": c.message, "duration_s": c.duration_s,
                                       "error_code": None if c.error_code is None else int(c.error_code), **c.metadata} for c in self.checks]})


class HealthChecker:
    """Named checks (callables returning a ``HealthCheckResult``, a bool, or raising). ``is_alive`` = the checker itself
    runs; ``is_ready`` = the last report is operational. Built-in checks: host memory head-room, device presence and
    free memory, and the kernel status word (a recorded kernel timeout makes the process unhealthy)."""

    def __init__(self, min_free_host_fraction: float = 0.05, min_free_device_fraction: float = 0.02):
        self.checks: dict[str, object] = {}
        self.last: HealthReport | None = None
        self.count = 0
        self.register("host_memory", lambda: self._host_memory(min_free_host_fraction))
        self.register("device", lambda: self._device(min_free_device_fraction))
        self.register("kernel_status", self._kernel_status)

    def register(self, name: str, fn):
        self.checks[name] = fn

    @staticmethod
    def _host_memory(min_free):
        import psutil
        vm = psutil.virtual_memory()
        frac = vm.available / vm.total
        st = HealthStatus.HEALTHY if frac >= 2 * min_free else (HealthStatus.DEGRADED if frac >= min_free else HealthStatus.UNHEALTHY)
        return HealthCheckResult("host_memory", st, f"{frac:.1%} of host memory available", metadata={"available_bytes": vm.available})

    @staticmethod
    def _device(min_free):
        import torch
        if not torch.cuda.is_available():
            return HealthCheckResult("device", HealthStatus.DEGRADED, "no CUDA device visible: kernels fall back to PyTorch CPU paths")
        free, total = torch.cuda.mem_get_info()
        st = HealthStatus.HEALTHY if free / total >= min_free else HealthStatus.DEGRADED
        return HealthCheckResult("device", st, f"{free / total:.1%} of device memory free", metadata={"free_bytes": free, "devices": torch.cuda.device_count()})

    @staticmethod
    def _kernel_status():
        import torch
        from .. import _native as nv
        if not torch.cuda.is_available() or not nv._status:
            return HealthCheckResult("kernel_status", HealthStatus.HEALTHY, "no kernel status recorded")
        codes = {k: int(v[0]) for k, v in nv._status.items()}
        bad = {k: c for k, c in codes.items() if c != 0}
        if bad:
            return HealthCheckResult("kernel_status", HealthStatus.UNHEALTHY, f"device status words set: {bad}", ErrorCode.KERNEL_TIMEOUT)
        return HealthCheckResult("kernel_status", HealthStatus.HEALTHY, "all status words clear")

    def check_health(self) -> HealthReport:
        out = []
        for name, fn in self.checks.items():
            t0 = time.perf_counter()
            try:
                r = fn()
                if isinstance(r, bool):
                    r = HealthCheckResult(name, HealthStatus.HEALTHY if r else HealthStatus.UNHEALTHY)
            except Exception as e:
                r = HealthCheckResult(name, HealthStatus.UNHEALTHY, f"{type(e).__name__}: {e}", ErrorCode.from_exception(e))
            r.name, r.duration_s = name, time.perf_counter() - t0
            out.append(r)
        self.last = HealthReport(out)
        self.count += 1
        return self.last

    def is_alive(self) -> bool:
        return True

    def is_ready(self) -> bool:
        return (self.last or self.check_health()).status.is_operational()
