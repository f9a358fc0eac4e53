"""Remote procedure calls between workers over TCP (``crates/torsh-distributed/src/rpc.rs:25-787``):
``init_rpc`` / ``shutdown``, ``register_function``, ``rpc_sync`` / ``rpc_async``, ``remote`` → :class:`RRef`,
``delete_rref``.  Workers find each other through a :class:`~torsh_b200.parallel.store.Store` (``rpc/<name>`` →
``host:port``).  Messages are msgpack frames with a 4-byte big-endian length; tensors travel as
``{dtype, shape, raw bytes}`` — no pickling, so a peer can only invoke functions that were registered by name."""
from __future__ import annotations

import socket
import socketserver
import struct
import threading
import uuid
from concurrent.futures import Future, ThreadPoolExecutor

import msgpack
import numpy as np
import torch

_state: dict = {}
_TORCH = {"float32": torch.float32, "float64": torch.float64, "float16": torch.float16, "bfloat16": torch.bfloat16,
          "int64": torch.int64, "int32": torch.int32, "uint8": torch.uint8, "bool": torch.bool}


def _enc(o):
    if isinstance(o, torch.Tensor):
        t = o.detach().cpu().contiguous()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype == torch.bfloat16 else t.numpy().tobytes()
        return {"__t": str(t.dtype).replace("torch.", ""), "s": list(t.shape), "b": raw}
    if isinstance(o, RRef):
        return {"__rref": o.id, "o": o.owner}
    if isinstance(o, (list, tuple)):
        return [_enc(v) for v in o]
    if isinstance(o, dict):
        return {k: _enc(v) for k, v in o.items()}
    return o


def _dec(o):
    if isinstance(o, dict):
        if "__t" in o:
            dt = _TORCH[o["__t"]]
            if dt == torch.bfloat16:
                return torch.frombuffer(bytearray(o["b"]), dtype=torch.uint8).view(torch.bfloat16).reshape(o["s"]).clone()
            return torch.from_numpy(np.frombuffer(o["b"], dtype=str(dt).replace("torch.", "")).copy()).reshape(o["s"])
        if "__rref" in o:
            return RRef(o["__rref"], o["o"])
        return {k: _dec(v) for k, v in o.items()}
    if isinstance(o, list):
        return [_dec(v) for v in o]
    return o


def _send(sock, obj):
    data = msgpack.packb(_enc(obj), use_bin_type=True)
    sock.sendall(struct.pack(">I", len(data)) + data)


def _recv(sock):
    hdr = b""
    while len(hdr) < 4:
        chunk = sock.recv(4 - len(hdr))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        hdr += chunk
    (n,) = struct.unpack(">I", hdr)
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(1 << 20, n - len(buf)))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return _dec(msgpack.unpackb(bytes(buf), raw=False))


class RRef:
    """Handle to a value that lives on worker ``owner``."""

    def __init__(self, rref_id: str, owner: str):
        self.id, self.owner = rref_id, owner

    def to_here(self):
        return rpc_sync(self.owner, "__rref_get", (self.id,))

    def rpc_sync(self, method: str, *args):
        return rpc_sync(self.owner, "__rref_call", (self.id, method, list(args)))

    def is_owner(self) -> bool:
        return _state.get("name") == self.owner


class _Handler(socketserver.BaseRequestHandler):
    def handle(self):
        try:
            while True:
                msg = _recv(self.request)
                try:
                    _send(self.request, {"ok": True, "value": _dispatch(msg["fn"], msg["args"], msg.get("kwargs") or {}, msg.get("keep"))})
                except Exception as e:  # the error travels back to the caller
                    _send(self.request, {"ok": False, "error": f"{type(e).__name__}: {e}"})
        except (ConnectionError, OSError):
            return


def _dispatch(fn: str, args, kwargs, keep):
    if fn == "__rref_get":
        return _state["rrefs"][args[0]]
    if fn == "__rref_call":
        return getattr(_state["rrefs"][args[0]], args[1])(*args[2])
    if fn == "__rref_del":
        return _state["rrefs"].pop(args[0], None) is not None
    if fn not in _state["functions"]:
        raise KeyError(f"function {fn!r} is not registered on worker {_state['name']!r}")
    out = _state["functions"][fn](*args, **kwargs)
    if keep:
        _state["rrefs"][keep] = out
        return None
    return out


class _Server(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True


def init_rpc(name: str, store, rank: int = 0, world_size: int = 1, host: str = "127.0.0.1", num_threads: int = 8) -> None:
    if _state:
        raise RuntimeError("RPC is already initialised")
    srv = _Server((host, 0), _Handler)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    _state.update(name=name, rank=rank, world=world_size, store=store, server=srv, functions={}, rrefs={}, conns={},
                  lock=threading.Lock(), pool=ThreadPoolExecutor(num_threads))
    store.set(f"rpc/{name}", f"{host}:{srv.server_address[1]}".encode())


def register_function(name: str, fn) -> None:
    _state["functions"][name] = fn


def _conn(to: str):
    with _state["lock"]:
        c = _state["conns"].get(to)
        if c is None:
            _state["store"].wait([f"rpc/{to}"])
            addr = _state["store"].get(f"rpc/{to}")
            host, port = addr.decode().rsplit(":", 1)
            c = (socket.create_connection((host, int(port)), timeout=30), threading.Lock())
            _state["conns"][to] = c
        return c


def _call(to: str, fn: str, args, kwargs, keep=None):
    if to == _state["name"]:
        return _dispatch(fn, list(args), kwargs, keep)
    sock, lock = _conn(to)
    with lock:
        _send(sock, {"fn": fn, "args": list(args), "kwargs": kwargs, "keep": keep})
        rep = _recv(sock)
    if not rep["ok"]:
        raise RuntimeError(f"remote error on {to}: {rep['error']}")
    return rep["value"]


def rpc_sync(to: str, fn: str, args=(), kwargs=None):
    return _call(to, fn, args, kwargs or {})


def rpc_async(to: str, fn: str, args=(), kwargs=None) -> Future:
    return _state["pool"].submit(_call, to, fn, args, kwargs or {})


def remote(to: str, fn: str, args=(), kwargs=None) -> RRef:
    """Run ``fn`` on ``to`` and keep the result there; returns a reference to it."""
    rid = uuid.uuid4().hex
    _call(to, fn, args, kwargs or {}, keep=rid)
    return RRef(rid, to)


def delete_rref(ref: RRef) -> bool:
    return bool(_call(ref.owner, "__rref_del", (ref.id,), {}))


def shutdown() -> None:
    if not _state:
        return
    for sock, _ in _state["conns"].values():
        try:
            sock.close()
        except OSError:
            pass
    _state["server"].shutdown()
    _state["server"].server_close()
    _state["pool"].shutdown(wait=False)
    _state.clear()
