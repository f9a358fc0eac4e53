"""TCP connection pool with retry, exponential back-off and per-peer statistics
(``crates/torsh-distributed/src/communication/*.rs``: ``ConnectionPool``, retry / backoff / timeout helpers, used by the
RPC layer, the parameter server and the stores for their control traffic; tensors between GPUs never travel this way)."""
from __future__ import annotations

import socket
import threading
import time
from contextlib import contextmanager
from dataclasses import dataclass, field

from ..core.error import TorshDistributedError


@dataclass
class RetryPolicy:
    """``BackendConfig{max_retries 3, backoff 2.0, timeout 30 s}`` (``crates/torsh-distributed/src/backend.rs:73-278``)."""
    max_retries: int = 3
    initial_delay_s: float = 0.05
    backoff: float = 2.0
    max_delay_s: float = 2.0
    timeout_s: float = 30.0

    def delays(self):
        d = self.initial_delay_s
        for _ in range(self.max_retries):
            yield min(d, self.max_delay_s)
            d *= self.backoff


def retry(fn, policy: RetryPolicy | None = None, retry_on=(OSError, TimeoutError), sleep=time.sleep):
    """Call ``fn()``; on a retryable exception wait (exponential back-off) and try again, up to ``max_retries`` times."""
    policy = policy or RetryPolicy()
    last = None
    for delay in [0.0, *policy.delays()]:
        if delay:
            sleep(delay)
        try:
            return fn()
        except retry_on as e:          # noqa: PERF203
            last = e
    raise TorshDistributedError.communication_error(f"gave up after {policy.max_retries} retries: {last}")


@dataclass
class PeerStats:
    connects: int = 0
    reuses: int = 0
    failures: int = 0
    bytes_sent: int = 0
    bytes_received: int = 0
    latencies_ms: list = field(default_factory=list)


class ConnectionPool:
    """Keeps up to ``max_per_peer`` idle sockets per ``(host, port)``; ``connection()`` lends one and takes it back unless
    the block raised (a broken socket is dropped, not reused). Idle sockets older than ``idle_timeout_s`` are closed."""

    def __init__(self, max_per_peer: int = 4, idle_timeout_s: float = 60.0, policy: RetryPolicy | None = None):
        self.max_per_peer, self.idle_timeout_s, self.policy = max_per_peer, idle_timeout_s, policy or RetryPolicy()
        self._idle: dict[tuple[str, int], list[tuple[socket.socket, float]]] = {}
        self._lock = threading.Lock()
        self.stats: dict[tuple[str, int], PeerStats] = {}

    def _stats(self, peer):
        return self.stats.setdefault(peer, PeerStats())

    def _connect(self, peer):
        t0 = time.perf_counter()
        try:
            s = retry(lambda: socket.create_connection(peer, timeout=self.policy.timeout_s), self.policy)
        except TorshDistributedError:
            self._stats(peer).failures += 1
            raise
        s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        st = self._stats(peer)
        st.connects += 1
        st.latencies_ms.append((time.perf_counter() - t0) * 1e3)
        return s

    def acquire(self, host: str, port: int) -> socket.socket:
        peer = (host, port)
        now = time.monotonic()
        with self._lock:
            idle = self._idle.get(peer, [])
            while idle:
                s, since = idle.pop()
                if now - since <= self.idle_timeout_s:
                    self._stats(peer).reuses += 1
                    return s
                s.close()
        return self._connect(peer)

    def release(self, host: str, port: int, s: socket.socket, broken: bool = False):
        peer = (host, port)
        if broken:
            s.close()
            return
        with self._lock:
            idle = self._idle.setdefault(peer, [])
            if len(idle) < self.max_per_peer:
                idle.append((s, time.monotonic()))
                return
        s.close()

    @contextmanager
    def connection(self, host: str, port: int):
        s = self.acquire(host, port)
        try:
            yield s
        except BaseException:
            self.release(host, port, s, broken=True)
            raise
        self.release(host, port, s)

    def request(self, host: str, port: int, payload: bytes, reply_bytes: int) -> bytes:
        """Send ``payload`` and read exactly ``reply_bytes`` back on a pooled connection."""
        with self.connection(host, port) as s:
            s.sendall(payload)
            buf = bytearray()
            while len(buf) < reply_bytes:
                chunk = s.recv(reply_bytes - len(buf))
                if not chunk:
                    raise ConnectionError("peer closed the connection")
                buf += chunk
            st = self._stats((host, port))
            st.bytes_sent += len(payload)
            st.bytes_received += len(buf)
            return bytes(buf)

    def idle_count(self, host: str, port: int) -> int:
        with self._lock:
            return len(self._idle.get((host, port), []))

    def close(self):
        with self._lock:
            for idle in self._idle.values():
                for s, _ in idle:
                    s.close()
            self._idle.clear()
