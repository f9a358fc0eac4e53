"""Failure detection, retry / circuit breaking, heartbeats and elastic membership — all on the host.

Reference: ``error_recovery.rs`` — ``RetryConfig`` (3 attempts, 100 ms → ×2 → ≤ 10 s, jitter 0.1), ``CircuitBreaker``
``{Closed, Open, HalfOpen}`` (5 failures open it, 3 successes close it, 30 s timeout, 60 s window: ``:49-216``),
``RetryExecutor`` (``:223-366``), ``HealthChecker`` (``:377-497``), ``FailureDetector.execute_with_recovery`` (``:501-570``);
``fault_tolerance.rs`` — ``ElasticConfig`` (min 1, max 64 workers, scaling timeout 300 s, check 30 s, heartbeat timeout
60 s: ``:55-87``) and ``ElasticTrainingManager`` with the state machine ``Stable → Scaling → Synchronizing → Stable``
and events ``WorkerFailure / WorkerJoin / ManualScale / AutoScale`` (``:451-855``). Fault injection exists only in the
reference's tests (``tests/test_fault_injection.rs:22-229``) and is host-side; it is host-side here too: no kernel is
ever made to fault, trap or hang. Device-side waits are bounded and report through a status word
(``torsh_b200._native.check_status``), which :class:`FailureDetector` turns into ``OperationTimeout``.
"""
from __future__ import annotations

import random
import threading
import time
from collections import deque
from dataclasses import dataclass
from enum import Enum

from ..core.error import TorshDistributedError


@dataclass
class RetryConfig:
    max_attempts: int = 3
    initial_delay_s: float = 0.1
    backoff_multiplier: float = 2.0
    max_delay_s: float = 10.0
    jitter: float = 0.1

    def delay(self, attempt: int) -> float:
        d = min(self.initial_delay_s * self.backoff_multiplier ** attempt, self.max_delay_s)
        return d * (1 + random.uniform(-self.jitter, self.jitter))


class CircuitState(Enum):
    CLOSED = "closed"; OPEN = "open"; HALF_OPEN = "half_open"


class CircuitBreaker:
    def __init__(self, failure_threshold: int = 5, success_threshold: int = 3, timeout_s: float = 30.0, window_s: float = 60.0,
                 clock=time.monotonic):
        self.failure_threshold, self.success_threshold, self.timeout_s, self.window_s = failure_threshold, success_threshold, timeout_s, window_s
        self.clock, self.state = clock, CircuitState.CLOSED
        self.failures: deque = deque()
        self.successes, self.opened_at = 0, 0.0

    def allow(self) -> bool:
        if self.state is CircuitState.OPEN and self.clock() - self.opened_at >= self.timeout_s:
            self.state, self.successes = CircuitState.HALF_OPEN, 0
        return self.state is not CircuitState.OPEN

    def record_success(self):
        if self.state is CircuitState.HALF_OPEN:
            self.successes += 1
            if self.successes >= self.success_threshold:
                self.state = CircuitState.CLOSED
                self.failures.clear()

    def record_failure(self):
        now = self.clock()
        if self.state is CircuitState.HALF_OPEN:
            self.state, self.opened_at = CircuitState.OPEN, now
            return
        self.failures.append(now)
        while self.failures and now - self.failures[0] > self.window_s:
            self.failures.popleft()
        if len(self.failures) >= self.failure_threshold:
            self.state, self.opened_at = CircuitState.OPEN, now


class RetryExecutor:
    def __init__(self, config: RetryConfig | None = None, breaker: CircuitBreaker | None = None, sleep=time.sleep):
        self.cfg, self.breaker, self.sleep = config or RetryConfig(), breaker, sleep
        self.stats = {"attempts": 0, "retries": 0, "failures": 0}

    def execute(self, fn, *args, **kw):
        last = None
        for attempt in range(self.cfg.max_attempts):
            if self.breaker is not None and not self.breaker.allow():
                raise TorshDistributedError.communication_error("circuit breaker is open")
            self.stats["attempts"] += 1
            try:
                out = fn(*args, **kw)
                if self.breaker is not None:
                    self.breaker.record_success()
                return out
            except Exception as e:  # noqa: BLE001
                last = e
                if self.breaker is not None:
                    self.breaker.record_failure()
                retryable = not isinstance(e, TorshDistributedError) or e.is_retryable()
                if not retryable or attempt + 1 == self.cfg.max_attempts:
                    break
                self.stats["retries"] += 1
                self.sleep(self.cfg.delay(attempt))
        self.stats["failures"] += 1
        raise last


class HealthChecker:
    """rank → last-seen time; ranks silent for longer than ``timeout_s`` are unhealthy."""

    def __init__(self, timeout_s: float = 60.0, clock=time.monotonic):
        self.timeout_s, self.clock, self.last_seen = timeout_s, clock, {}

    def heartbeat(self, rank: int):
        self.last_seen[rank] = self.clock()

    def is_healthy(self, rank: int) -> bool:
        t = self.last_seen.get(rank)
        return t is not None and self.clock() - t <= self.timeout_s

    def unhealthy(self) -> list[int]:
        return sorted(r for r in self.last_seen if not self.is_healthy(r))

    def cleanup_stale(self, factor: float = 5.0):
        now = self.clock()
        for r in [r for r, t in self.last_seen.items() if now - t > factor * self.timeout_s]:
            del self.last_seen[r]


class FailureDetector:
    def __init__(self, retry: RetryConfig | None = None, breaker: CircuitBreaker | None = None, health: HealthChecker | None = None):
        self.executor = RetryExecutor(retry, breaker or CircuitBreaker())
        self.health = health or HealthChecker()
        self.incidents: list[dict] = []

    def execute_with_recovery(self, fn, *args, description: str = "", **kw):
        try:
            return self.executor.execute(fn, *args, **kw)
        except Exception as e:  # noqa: BLE001
            self.incidents.append({"what": description or getattr(fn, "__name__", "op"), "error": repr(e), "time": time.time()})
            raise

    def check_device(self):
        """Turns a bounded-wait expiry recorded by a kernel into ``OperationTimeout``."""
        from .. import _native as nv
        try:
            nv.check_status()
        except nv.KernelTimeout as e:
            self.incidents.append({"what": "device wait", "error": str(e), "time": time.time()})
            raise TorshDistributedError.operation_timeout(str(e)) from e


# ---- elastic membership over a Store --------------------------------------------------------------------
@dataclass
class ElasticConfig:
    min_workers: int = 1
    max_workers: int = 64
    scaling_timeout_s: float = 300.0
    check_interval_s: float = 30.0
    heartbeat_timeout_s: float = 60.0
    rendezvous_backend: str = "tcp"
    rendezvous_endpoint: str = "127.0.0.1:29500"


class ElasticState(Enum):
    STABLE = "stable"; SCALING = "scaling"; SYNCHRONIZING = "synchronizing"


class ScalingEvent(Enum):
    WORKER_FAILURE = "worker_failure"; WORKER_JOIN = "worker_join"; MANUAL_SCALE = "manual_scale"; AUTO_SCALE = "auto_scale"


class HeartbeatPublisher:
    """Background thread writing ``hb/{rank}`` = wall time into the store every ``interval_s``."""

    def __init__(self, store, rank: int, interval_s: float = 1.0):
        self.store, self.rank, self.interval_s = store, rank, interval_s
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.store.set(f"hb/{self.rank}", repr(time.time()).encode())
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(self.interval_s)

    def start(self):
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        self._thread.join(2.0)


class ElasticTrainingManager:
    """Watches heartbeats in the store and decides when the job has to re-form with a new world size."""

    def __init__(self, store, rank: int, world_size: int, config: ElasticConfig | None = None, on_checkpoint=None):
        self.store, self.rank, self.world_size = store, rank, world_size
        self.cfg = config or ElasticConfig()
        self.state, self.events, self.on_checkpoint = ElasticState.STABLE, [], on_checkpoint
        self.generation = 0

    def alive_workers(self, now: float | None = None) -> list[int]:
        now = time.time() if now is None else now
        alive = []
        for r in range(self.cfg.max_workers):
            v = self.store.get(f"hb/{r}")
            if v is not None and now - float(v.decode()) <= self.cfg.heartbeat_timeout_s:
                alive.append(r)
        return alive

    def check_scaling_needs(self, now: float | None = None) -> ScalingEvent | None:
        alive = self.alive_workers(now)
        expected = set(range(self.world_size))
        if expected - set(alive):
            return self._begin(ScalingEvent.WORKER_FAILURE, len([r for r in alive if r in expected]))
        if set(alive) - expected and len(alive) <= self.cfg.max_workers:
            return self._begin(ScalingEvent.WORKER_JOIN, len(alive))
        return None

    def request_scale(self, target: int) -> ScalingEvent:
        if not self.cfg.min_workers <= target <= self.cfg.max_workers:
            raise TorshDistributedError.invalid_argument(f"target {target} outside [{self.cfg.min_workers}, {self.cfg.max_workers}]")
        return self._begin(ScalingEvent.MANUAL_SCALE, target)

    def _begin(self, ev: ScalingEvent, target: int) -> ScalingEvent:
        if target < self.cfg.min_workers:
            raise TorshDistributedError.process_failure(f"only {target} workers alive, need {self.cfg.min_workers}")
        if self.on_checkpoint is not None:  # checkpoint-before-scale
            self.on_checkpoint()
        self.state = ElasticState.SCALING
        self.events.append({"event": ev.value, "from": self.world_size, "to": target, "time": time.time()})
        self.pending_world = target
        return ev

    def complete_scaling(self):
        """Re-rendezvous finished: ranks synchronise (store barrier keyed by generation) and training resumes."""
        self.state = ElasticState.SYNCHRONIZING
        self.generation += 1
        self.world_size = self.pending_world
        self.state = ElasticState.STABLE


class FaultKind(Enum):
    NETWORK_FAILURE = "network"; PROCESS_CRASH = "crash"; MEMORY_FAILURE = "memory"; TIMEOUT = "timeout"
    DATA_CORRUPTION = "corruption"; BACKEND_FAILURE = "backend"; INTERMITTENT = "intermittent"


class FaultInjector:
    """Host-side fault injection for tests: wraps callables so that chosen calls raise the matching error."""

    def __init__(self, seed: int = 0):
        self.rng, self.rules, self.injected = random.Random(seed), [], 0

    def add(self, kind: FaultKind, probability: float = 1.0, max_count: int | None = None):
        self.rules.append({"kind": kind, "p": probability, "left": max_count})

    def maybe_fail(self):
        for r in self.rules:
            if (r["left"] is None or r["left"] > 0) and self.rng.random() < r["p"]:
                if r["left"] is not None:
                    r["left"] -= 1
                self.injected += 1
                k = r["kind"]
                if k in (FaultKind.NETWORK_FAILURE, FaultKind.INTERMITTENT):
                    raise TorshDistributedError.communication_error(f"injected {k.value} fault")
                if k is FaultKind.TIMEOUT:
                    raise TorshDistributedError.operation_timeout("injected timeout")
                if k is FaultKind.PROCESS_CRASH:
                    raise TorshDistributedError.process_failure("injected process crash")
                if k is FaultKind.MEMORY_FAILURE:
                    raise TorshDistributedError.memory_allocation_failed("injected allocation failure")
                if k is FaultKind.DATA_CORRUPTION:
                    raise TorshDistributedError.serialization_error("injected data corruption")
                raise TorshDistributedError.backend_error("injected backend failure")

    def wrap(self, fn):
        def wrapped(*a, **kw):
            self.maybe_fail()
            return fn(*a, **kw)
        return wrapped



class NativeWatchdog:
    """Native heartbeat thread (``csrc/host/watchdog.cpp``): beats through a store every ``interval_s`` and reports the
    ranks whose counter has not moved for ``timeout_s``.  It keeps beating while Python is blocked in a collective."""

    def __init__(self, store, rank: int, world_size: int, interval_s: float = 1.0, timeout_s: float = 10.0, prefix: str = "hb"):
        import ctypes

        from .. import _native as nv
        self.store, self.rank, self.world, self.prefix = store, rank, world_size, prefix
        lib = nv.host()
        PUB = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p)
        READ = ctypes.CFUNCTYPE(ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p)

        def publish(r, counter, _ctx):
            try:
                store.set(f"{prefix}/{r}", str(counter).encode())
            except Exception:
                pass

        def read(r, _ctx):
            try:
                v = store.get(f"{prefix}/{r}")
                return int(v) if v else -1
            except Exception:
                return -1
        self._pub, self._read = PUB(publish), READ(read)          # keep the callbacks alive
        lib.tsh_watchdog_start.restype = ctypes.c_void_p
        lib.tsh_watchdog_start.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_double, PUB, READ, ctypes.c_void_p]
        lib.tsh_watchdog_failed.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        lib.tsh_watchdog_beats.restype, lib.tsh_watchdog_beats.argtypes = ctypes.c_longlong, [ctypes.c_void_p]
        lib.tsh_watchdog_stop.argtypes = [ctypes.c_void_p]
        self._lib, self._ct = lib, ctypes
        self._h = lib.tsh_watchdog_start(rank, world_size, interval_s, timeout_s, self._pub, self._read, None)
        if not self._h:
            raise ValueError("bad watchdog arguments")

    def failed_ranks(self) -> list[int]:
        buf = (self._ct.c_int * self.world)()
        self._lib.tsh_watchdog_failed(self._h, buf)
        return [r for r in range(self.world) if buf[r]]

    def beats(self) -> int:
        return self._lib.tsh_watchdog_beats(self._h)

    def stop(self) -> None:
        if self._h:
            self._lib.tsh_watchdog_stop(self._h)
            self._h = None

    def __del__(self):
        try:
            self.stop()
        except Exception:
            pass
