"""bincode-2 "standard" configuration (little-endian, varint integers) in Python.

Same rules as ``csrc/host/bincode.h``; used for the model-state and checkpoint containers whose
schemas are nested maps (``crates/torsh-nn/src/serialization.rs``, ``crates/torsh-nn/src/checkpoint.rs``).
"""
from __future__ import annotations

import struct


class Writer:
    def __init__(self):
        self.b = bytearray()

    def u8(self, v): self.b.append(v & 0xFF)

    def varu(self, v: int):
        if v < 251:
            self.b.append(v)
        elif v <= 0xFFFF:
            self.b.append(251); self.b += struct.pack("<H", v)
        elif v <= 0xFFFFFFFF:
            self.b.append(252); self.b += struct.pack("<I", v)
        else:
            self.b.append(253); self.b += struct.pack("<Q", v)

    def vari(self, v: int):
        self.varu((v << 1) ^ (v >> 63) if v >= 0 else ((-v) << 1) - 1)

    def boolean(self, v): self.b.append(1 if v else 0)
    def f32(self, v): self.b += struct.pack("<f", v)
    def f64(self, v): self.b += struct.pack("<d", v)

    def string(self, s: str):
        e = s.encode()
        self.varu(len(e)); self.b += e

    def raw(self, data: bytes): self.b += data

    def option(self, v, fn):
        if v is None:
            self.b.append(0)
        else:
            self.b.append(1); fn(v)

    def seq(self, items, fn):
        self.varu(len(items))
        for it in items:
            fn(it)

    def map(self, d: dict, kfn, vfn):
        self.varu(len(d))
        for k in sorted(d):
            kfn(k); vfn(d[k])

    def bytes(self) -> bytes:
        return bytes(self.b)


class Reader:
    def __init__(self, data: bytes):
        self.d, self.i = memoryview(data), 0

    def _take(self, n):
        if self.i + n > len(self.d):
            raise ValueError("bincode: unexpected end of input")
        v = self.d[self.i:self.i + n]; self.i += n
        return v

    def u8(self): return self._take(1)[0]

    def varu(self) -> int:
        t = self.u8()
        if t < 251: return t
        if t == 251: return struct.unpack("<H", self._take(2))[0]
        if t == 252: return struct.unpack("<I", self._take(4))[0]
        if t == 253: return struct.unpack("<Q", self._take(8))[0]
        raise ValueError("bincode: 128-bit integers are not supported")

    def vari(self) -> int:
        z = self.varu()
        return (z >> 1) ^ -(z & 1)

    def boolean(self) -> bool:
        b = self.u8()
        if b > 1: raise ValueError("bincode: invalid bool")
        return b == 1

    def f32(self): return struct.unpack("<f", self._take(4))[0]
    def f64(self): return struct.unpack("<d", self._take(8))[0]
    def string(self) -> str: return bytes(self._take(self.varu())).decode()
    def raw(self, n) -> bytes: return bytes(self._take(n))
    def option(self, fn): return fn() if self.u8() == 1 else None
    def seq(self, fn): return [fn() for _ in range(self.varu())]
    def map(self, kfn, vfn): return {kfn(): vfn() for _ in range(self.varu())}
    def remaining(self): return len(self.d) - self.i
