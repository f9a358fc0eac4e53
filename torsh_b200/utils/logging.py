"""Structured and audit logging, and graceful degradation (``crates/torsh-autograd/src/{structured_logging,
audit_logging,graceful_degradation,automatic_error_recovery}.rs``; ``crates/torsh-core/src/telemetry.rs``): JSON-lines
records with fixed fields and spans, a tamper-evident audit trail (each record carries the SHA-256 of its predecessor),
and a runner that falls back through cheaper implementations when one fails."""
from __future__ import annotations

import hashlib
import json
import os
import threading
import time
from contextlib import contextmanager


class StructuredLogger:
    """One JSON object per line: ``ts, level, event, rank, span`` + user fields. ``path=None`` keeps records in memory."""

    LEVELS = {"debug": 10, "info": 20, "warning": 30, "error": 40}

    def __init__(self, path: str | None = None, level: str = "info", rank: int | None = None):
        self.path, self.level = path, self.LEVELS[level]
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.records: list[dict] = []
        self._lock = threading.Lock()
        self._spans = threading.local()

    def log(self, level: str, event: str, **fields):
        if self.LEVELS[level] < self.level:
            return None
        rec = {"ts": time.time(), "level": level, "event": event, "rank": self.rank,
               "span": "/".join(getattr(self._spans, "stack", [])) or None, **fields}
        with self._lock:
            self.records.append(rec)
            if self.path:
                with open(self.path, "a") as f:
                    f.write(json.dumps(rec, default=str) + "\n")
        return rec

    def info(self, event, **f): return self.log("info", event, **f)
    def warning(self, event, **f): return self.log("warning", event, **f)
    def error(self, event, **f): return self.log("error", event, **f)
    def debug(self, event, **f): return self.log("debug", event, **f)

    @contextmanager
    def span(self, name: str, **fields):
        stack = getattr(self._spans, "stack", None)
        if stack is None:
            stack = self._spans.stack = []
        stack.append(name)
        t0 = time.perf_counter()
        try:
            yield
        except Exception as e:
            self.error("span_failed", error=repr(e), **fields)
            raise
        finally:
            self.info("span_end", duration_ms=(time.perf_counter() - t0) * 1e3, **fields)
            stack.pop()


class AuditLog:
    """Append-only trail: record ``i`` stores ``prev`` = SHA-256 of record ``i-1``'s canonical JSON, so any edit or
    removal breaks :meth:`verify`."""

    def __init__(self, path: str | None = None):
        self.path, self.records, self._last = path, [], "0" * 64
        if path and os.path.exists(path):
            with open(path) as f:
                self.records = [json.loads(ln) for ln in f if ln.strip()]
            if self.records:
                self._last = self._digest(self.records[-1])

    @staticmethod
    def _digest(rec: dict) -> str:
        return hashlib.sha256(json.dumps(rec, sort_keys=True, default=str).encode()).hexdigest()

    def append(self, actor: str, action: str, **details) -> dict:
        rec = {"seq": len(self.records), "ts": time.time(), "actor": actor, "action": action, "details": details, "prev": self._last}
        self.records.append(rec)
        self._last = self._digest(rec)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec, sort_keys=True, default=str) + "\n")
        return rec

    def verify(self) -> bool:
        prev = "0" * 64
        for i, rec in enumerate(self.records):
            if rec.get("seq") != i or rec.get("prev") != prev:
                return False
            prev = self._digest(rec)
        return True


class GracefulDegradation:
    """Runs the first implementation that works: ``add("kernel", fn)``, ``add("torch", fn2)`` …; a failure is logged and
    the next level tried, and a level that failed ``disable_after`` times in a row is skipped from then on."""

    def __init__(self, logger: StructuredLogger | None = None, disable_after: int = 3):
        self.levels: list[tuple[str, object]] = []
        self.failures: dict[str, int] = {}
        self.logger, self.disable_after = logger, disable_after
        self.used: list[str] = []

    def add(self, name: str, fn):
        self.levels.append((name, fn))
        self.failures[name] = 0
        return self

    def run(self, *args, **kwargs):
        last = None
        for name, fn in self.levels:
            if self.failures[name] >= self.disable_after:
                continue
            try:
                out = fn(*args, **kwargs)
                self.failures[name] = 0
                self.used.append(name)
                return out
            except Exception as e:       # noqa: BLE001
                last = e
                self.failures[name] += 1
                if self.logger:
                    self.logger.warning("degraded", implementation=name, error=repr(e), consecutive=self.failures[name])
        raise RuntimeError(f"every implementation failed; last error: {last!r}")
