"""Rendezvous key-value stores: ``TCPStore`` (native C++ server/client), ``FileStore``, ``MemoryStore``.

Operation set of the reference ``Store`` trait (``crates/torsh-distributed/src/store/store_trait.rs:9-41``):
``set, get, wait, delete, num_keys, contains, set_with_expiry, compare_and_swap, add``. The TCP wire format
(4-byte big-endian length + bincode message, ``store/tcp.rs:38-76``) is implemented in
``csrc/host/tcp_store.cpp``.
"""
from __future__ import annotations

import ctypes
import json
import os
import threading
import time
from pathlib import Path

from .. import _native as nv
from ..core.error import TorshDistributedError

_cfg = False


def _lib():
    global _cfg
    lib = nv.host()
    if not _cfg:
        vp, cp, i, i64, u64 = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64
        lib.tsh_last_error.restype = cp
        lib.tsh_free.argtypes = [vp]
        lib.tsh_store_server_start.restype = vp
        lib.tsh_store_server_start.argtypes = [cp, i, ctypes.POINTER(i)]
        lib.tsh_store_server_stop.argtypes = [vp]
        lib.tsh_store_client_connect.restype = vp
        lib.tsh_store_client_connect.argtypes = [cp, i, i]
        lib.tsh_store_client_close.argtypes = [vp]
        lib.tsh_store_set.argtypes = [vp, cp, cp, u64, i64]
        lib.tsh_store_get.argtypes = [vp, cp, ctypes.POINTER(vp), ctypes.POINTER(u64)]
        lib.tsh_store_wait.argtypes = [vp, ctypes.POINTER(cp), i, i]
        lib.tsh_store_delete.argtypes = [vp, cp]
        lib.tsh_store_num_keys.restype = i64
        lib.tsh_store_num_keys.argtypes = [vp]
        lib.tsh_store_contains.argtypes = [vp, cp]
        lib.tsh_store_cas.argtypes = [vp, cp, cp, u64, i, cp, u64]
        lib.tsh_store_add.argtypes = [vp, cp, i64, ctypes.POINTER(i64)]
        _cfg = True
    return lib


def _err(lib, what):
    return TorshDistributedError.communication_error(f"{what}: {lib.tsh_last_error().decode(errors='replace')}")


class Store:
    """Interface shared by every store."""

    def set(self, key: str, value: bytes, ttl: float | None = None): raise NotImplementedError
    def get(self, key: str) -> bytes | None: raise NotImplementedError
    def wait(self, keys, timeout: float = 30.0): raise NotImplementedError
    def delete(self, key: str): raise NotImplementedError
    def num_keys(self) -> int: raise NotImplementedError
    def contains(self, key: str) -> bool: raise NotImplementedError
    def compare_and_swap(self, key: str, expected: bytes | None, value: bytes) -> bool: raise NotImplementedError
    def add(self, key: str, delta: int) -> int: raise NotImplementedError
    def close(self): pass

    def set_with_expiry(self, key, value, ttl):
        self.set(key, value, ttl)

    def barrier(self, name: str, world_size: int, timeout: float = 60.0):
        """All ``world_size`` participants block until everyone has arrived."""
        n = self.add(f"{name}/count", 1)
        if n == world_size:
            self.set(f"{name}/done", b"1")
        self.wait([f"{name}/done"], timeout)


class TCPStore(Store):
    def __init__(self, host: str = "127.0.0.1", port: int = 29500, is_server: bool = False, timeout: float = 30.0):
        lib = _lib()
        self._lib, self._server, self.host = lib, None, host
        if is_server:
            bound = ctypes.c_int(0)
            self._server = lib.tsh_store_server_start(host.encode(), port, ctypes.byref(bound))
            if not self._server:
                raise _err(lib, "TCPStore server")
            port = bound.value
        self.port = port
        self._client = lib.tsh_store_client_connect(host.encode(), port, int(timeout * 1000))
        if not self._client:
            raise _err(lib, "TCPStore connect")

    def set(self, key, value, ttl=None):
        if self._lib.tsh_store_set(self._client, key.encode(), value, len(value), -1 if ttl is None else int(ttl)) != 0:
            raise _err(self._lib, "set")

    def get(self, key):
        out, n = ctypes.c_void_p(), ctypes.c_uint64()
        rc = self._lib.tsh_store_get(self._client, key.encode(), ctypes.byref(out), ctypes.byref(n))
        if rc < 0:
            raise _err(self._lib, "get")
        if rc == 0:
            return None
        try:
            return ctypes.string_at(out.value, n.value)
        finally:
            self._lib.tsh_free(out)

    def wait(self, keys, timeout: float = 30.0):
        keys = [keys] if isinstance(keys, str) else list(keys)
        arr = (ctypes.c_char_p * len(keys))(*[k.encode() for k in keys])
        if self._lib.tsh_store_wait(self._client, arr, len(keys), max(1, int(timeout * 1000))) != 0:
            raise TorshDistributedError.operation_timeout(f"wait for {keys} timed out after {timeout}s")

    def delete(self, key):
        if self._lib.tsh_store_delete(self._client, key.encode()) != 0:
            raise _err(self._lib, "delete")

    def num_keys(self):
        n = self._lib.tsh_store_num_keys(self._client)
        if n < 0:
            raise _err(self._lib, "num_keys")
        return int(n)

    def contains(self, key):
        rc = self._lib.tsh_store_contains(self._client, key.encode())
        if rc < 0:
            raise _err(self._lib, "contains")
        return rc == 1

    def compare_and_swap(self, key, expected, value):
        rc = self._lib.tsh_store_cas(self._client, key.encode(), expected or b"", len(expected or b""),
                                     0 if expected is None else 1, value, len(value))
        if rc < 0:
            raise _err(self._lib, "compare_and_swap")
        return rc == 1

    def add(self, key, delta):
        out = ctypes.c_int64()
        if self._lib.tsh_store_add(self._client, key.encode(), delta, ctypes.byref(out)) != 0:
            raise _err(self._lib, "add")
        return out.value

    def close(self):
        if self._client:
            self._lib.tsh_store_client_close(self._client)
            self._client = None
        if self._server:
            self._lib.tsh_store_server_stop(self._server)
            self._server = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MemoryStore(Store):
    """In-process store (``crates/torsh-distributed/src/store/memory.rs``)."""

    def __init__(self):
        self._d: dict[str, tuple[bytes, float | None]] = {}
        self._cv = threading.Condition()

    def _alive(self, k):
        v = self._d.get(k)
        if v is None:
            return False
        if v[1] is not None and time.monotonic() >= v[1]:
            del self._d[k]
            return False
        return True

    def set(self, key, value, ttl=None):
        with self._cv:
            self._d[key] = (bytes(value), None if ttl is None else time.monotonic() + ttl)
            self._cv.notify_all()

    def get(self, key):
        with self._cv:
            return self._d[key][0] if self._alive(key) else None

    def wait(self, keys, timeout=30.0):
        keys = [keys] if isinstance(keys, str) else list(keys)
        end = time.monotonic() + timeout
        with self._cv:
            while not all(self._alive(k) for k in keys):
                left = end - time.monotonic()
                if left <= 0:
                    raise TorshDistributedError.operation_timeout(f"wait for {keys} timed out after {timeout}s")
                self._cv.wait(min(left, 0.1))

    def delete(self, key):
        with self._cv:
            self._d.pop(key, None)

    def num_keys(self):
        with self._cv:
            return sum(1 for k in list(self._d) if self._alive(k))

    def contains(self, key):
        with self._cv:
            return self._alive(key)

    def compare_and_swap(self, key, expected, value):
        with self._cv:
            present = self._alive(key)
            ok = (present and self._d[key][0] == expected) if expected is not None else not present
            if ok:
                self._d[key] = (bytes(value), None)
                self._cv.notify_all()
            return ok

    def add(self, key, delta):
        with self._cv:
            cur = int.from_bytes(self._d[key][0], "little", signed=True) if self._alive(key) else 0
            cur += delta
            self._d[key] = (cur.to_bytes(8, "little", signed=True), None)
            self._cv.notify_all()
            return cur


class FileStore(Store):
    """Directory-backed store for ranks sharing a filesystem (``crates/torsh-distributed/src/store/file.rs``).
    One file per key, written atomically by rename; ``add`` / CAS serialise through a lock file."""

    def __init__(self, path):
        self.dir = Path(path)
        self.dir.mkdir(parents=True, exist_ok=True)

    def _p(self, key):
        return self.dir / (key.replace("/", "%2F") + ".kv")

    def _lock(self):
        lock = self.dir / ".lock"
        while True:
            try:
                fd = os.open(lock, os.O_CREAT | os.O_EXCL | os.O_WRONLY)
                os.close(fd)
                return lock
            except FileExistsError:
                time.sleep(0.002)

    def _read(self, key):
        try:
            doc = json.loads(self._p(key).read_text())
        except (FileNotFoundError, json.JSONDecodeError):
            return None
        if doc["exp"] is not None and time.time() >= doc["exp"]:
            return None
        return bytes.fromhex(doc["v"])

    def set(self, key, value, ttl=None):
        tmp = self._p(key).with_suffix(f".tmp{os.getpid()}{threading.get_ident()}")
        tmp.write_text(json.dumps({"v": bytes(value).hex(), "exp": None if ttl is None else time.time() + ttl}))
        os.replace(tmp, self._p(key))

    def get(self, key):
        return self._read(key)

    def wait(self, keys, timeout=30.0):
        keys = [keys] if isinstance(keys, str) else list(keys)
        end = time.monotonic() + timeout
        while not all(self._read(k) is not None for k in keys):
            if time.monotonic() >= end:
                raise TorshDistributedError.operation_timeout(f"wait for {keys} timed out after {timeout}s")
            time.sleep(0.01)

    def delete(self, key):
        self._p(key).unlink(missing_ok=True)

    def num_keys(self):
        return sum(1 for f in self.dir.glob("*.kv") if self._read(f.stem.replace("%2F", "/")) is not None)

    def contains(self, key):
        return self._read(key) is not None

    def compare_and_swap(self, key, expected, value):
        lock = self._lock()
        try:
            cur = self._read(key)
            ok = (cur == expected) if expected is not None else cur is None
            if ok:
                self.set(key, value)
            return ok
        finally:
            os.unlink(lock)

    def add(self, key, delta):
        lock = self._lock()
        try:
            cur = self._read(key)
            n = (int.from_bytes(cur, "little", signed=True) if cur else 0) + delta
            self.set(key, n.to_bytes(8, "little", signed=True))
            return n
        finally:
            os.unlink(lock)


class RedisStore(Store):
    """Store on a Redis server, spoken over a plain socket in RESP2 (``crates/torsh-distributed/src/store/redis.rs:87-586``;
    no client library is needed). Keys get a ``prefix``; ``compare_and_swap`` runs a small Lua script so that it is
    atomic on the server; ``wait`` polls with back-off."""

    _CAS = ("local cur = redis.call('GET', KEYS[1]); "
            "if (ARGV[1] == '0' and cur == false) or (ARGV[1] == '1' and cur == ARGV[2]) then "
            "redis.call('SET', KEYS[1], ARGV[3]); return 1 else return 0 end")

    def __init__(self, host: str = "127.0.0.1", port: int = 6379, prefix: str = "torsh/", timeout: float = 30.0,
                 password: str | None = None, db: int = 0):
        import socket
        self.prefix, self.timeout = prefix, timeout
        self._lock = threading.Lock()
        self._sock = socket.create_connection((host, port), timeout=timeout)
        self._rf = self._sock.makefile("rb")
        if password:
            self._cmd("AUTH", password)
        if db:
            self._cmd("SELECT", str(db))

    # ---- RESP2 ---------------------------------------------------------------------------------------
    @staticmethod
    def _enc(*parts) -> bytes:
        out = [b"*%d\r\n" % len(parts)]
        for p in parts:
            b = p if isinstance(p, (bytes, bytearray)) else str(p).encode()
            out.append(b"$%d\r\n" % len(b) + bytes(b) + b"\r\n")
        return b"".join(out)

    def _read(self):
        line = self._rf.readline()
        if not line:
            raise TorshDistributedError.communication_error("redis: connection closed")
        kind, rest = line[:1], line[1:-2]
        if kind == b"+":
            return rest
        if kind == b"-":
            raise TorshDistributedError.communication_error("redis: " + rest.decode(errors="replace"))
        if kind == b":":
            return int(rest)
        if kind == b"$":
            n = int(rest)
            if n < 0:
                return None
            data = self._rf.read(n + 2)
            return data[:-2]
        if kind == b"*":
            n = int(rest)
            return None if n < 0 else [self._read() for _ in range(n)]
        raise TorshDistributedError.communication_error(f"redis: bad reply type {kind!r}")

    def _cmd(self, *parts):
        with self._lock:
            self._sock.sendall(self._enc(*parts))
            return self._read()

    def _k(self, key: str) -> str:
        return self.prefix + key

    # ---- Store ---------------------------------------------------------------------------------------
    def set(self, key, value, ttl=None):
        if ttl is None:
            self._cmd("SET", self._k(key), value)
        else:
            self._cmd("SET", self._k(key), value, "PX", max(1, int(ttl * 1000)))

    def get(self, key):
        return self._cmd("GET", self._k(key))

    def contains(self, key):
        return self._cmd("EXISTS", self._k(key)) == 1

    def delete(self, key):
        return self._cmd("DEL", self._k(key)) == 1

    def num_keys(self):
        return len(self._cmd("KEYS", self.prefix + "*") or [])

    def add(self, key, delta):
        return int(self._cmd("INCRBY", self._k(key), int(delta)))

    def compare_and_swap(self, key, expected, value):
        return self._cmd("EVAL", self._CAS, 1, self._k(key), "0" if expected is None else "1",
                         b"" if expected is None else expected, value) == 1

    def wait(self, keys, timeout: float = 30.0):
        deadline, delay = time.monotonic() + timeout, 0.001
        keys = [keys] if isinstance(keys, str) else list(keys)
        while True:
            if all(self.contains(k) for k in keys):
                return
            if time.monotonic() >= deadline:
                raise TorshDistributedError.operation_timeout(f"redis wait for {keys} timed out after {timeout}s")
            time.sleep(delay)
            delay = min(delay * 2, 0.05)

    def close(self):
        try:
            self._rf.close()
            self._sock.close()
        except OSError:
            pass


def create_store(kind: str, **kw) -> Store:
    """Factory (``crates/torsh-distributed/src/store/mod.rs:28``): ``tcp``, ``file``, ``memory``, ``redis``."""
    if kind == "redis":
        return RedisStore(**kw)
    if kind == "tcp":
        return TCPStore(**kw)
    if kind == "file":
        return FileStore(**kw)
    if kind == "memory":
        return MemoryStore()
    raise TorshDistributedError.configuration_error(f"unknown store kind {kind!r}")
