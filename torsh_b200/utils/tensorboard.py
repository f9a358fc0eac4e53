"""TensorBoard event-file writer (``crates/torsh-utils/src/tensorboard``, ``crates/torsh-metrics`` writers) without
the tensorboard / protobuf packages: records are ``len | masked_crc32c(len) | payload | masked_crc32c(payload)`` and
the payload is a hand-encoded ``Event`` protobuf (scalars, histograms, text)."""
from __future__ import annotations

import os
import socket
import struct
import time
from pathlib import Path

_CRC_TABLE = []
for _i in range(256):
    _c = _i
    for _ in range(8):
        _c = (_c >> 1) ^ 0x82F63B78 if _c & 1 else _c >> 1
    _CRC_TABLE.append(_c)


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC_TABLE[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _ld(num: int, data: bytes) -> bytes: return _field(num, 2, _varint(len(data)) + data)
def _f64(num: int, v: float) -> bytes: return _field(num, 1, struct.pack("<d", v))
def _f32(num: int, v: float) -> bytes: return _field(num, 5, struct.pack("<f", v))
def _i64(num: int, v: int) -> bytes: return _field(num, 0, _varint(v))


class SummaryWriter:
    def __init__(self, log_dir: str = "runs", filename_suffix: str = ""):
        Path(log_dir).mkdir(parents=True, exist_ok=True)
        name = f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}.{os.getpid()}{filename_suffix}"
        self.path = Path(log_dir) / name
        self._f = open(self.path, "wb")
        self._event(_ld(3, b"brain.Event:2"))

    def _event(self, body: bytes, step: int | None = None):
        ev = _f64(1, time.time()) + (_i64(2, step) if step is not None else b"") + body
        hdr = struct.pack("<Q", len(ev))
        self._f.write(hdr + struct.pack("<I", _masked(hdr)) + ev + struct.pack("<I", _masked(ev)))

    def add_scalar(self, tag: str, value: float, step: int = 0):
        val = _ld(1, tag.encode()) + _f32(2, float(value))
        self._event(_ld(5, _ld(1, val)), step)

    def add_scalars(self, main_tag: str, values: dict, step: int = 0):
        for k, v in values.items():
            self.add_scalar(f"{main_tag}/{k}", v, step)

    def add_histogram(self, tag: str, values, step: int = 0, bins: int = 30):
        import torch
        v = torch.as_tensor(values).detach().float().flatten().cpu()
        lo, hi = v.min().item(), v.max().item()
        hi = hi if hi > lo else lo + 1e-6
        counts = torch.histc(v, bins, lo, hi)
        edges = torch.linspace(lo, hi, bins + 1)[1:]
        packed = lambda xs: b"".join(struct.pack("<d", float(x)) for x in xs)
        histo = (_f64(1, lo) + _f64(2, hi) + _f64(3, float(v.numel())) + _f64(4, v.sum().item()) +
                 _f64(5, (v * v).sum().item()) + _ld(6, packed(edges)) + _ld(7, packed(counts)))
        self._event(_ld(5, _ld(1, _ld(1, tag.encode()) + _ld(5, histo))), step)

    def add_text(self, tag: str, text: str, step: int = 0):
        tensor = _i64(1, 7) + _ld(8, text.encode())                           # DT_STRING, string_val
        meta = _ld(1, _ld(1, b"text"))                                        # plugin_data.plugin_name
        self._event(_ld(5, _ld(1, _ld(1, tag.encode()) + _ld(9, meta) + _ld(8, tensor))), step)

    def flush(self): self._f.flush()
    def close(self): self._f.close()
    def __enter__(self): return self
    def __exit__(self, *a): self.close()


def read_events(path) -> list[tuple[int, str, float]]:
    """Parse scalar events back (step, tag, value): used by tests and ``train monitor``-style tooling."""
    buf, out, off = Path(path).read_bytes(), [], 0

    def fields(b):
        i = 0
        while i < len(b):
            key, n = 0, 0
            while True:
                key |= (b[i] & 0x7F) << n; n += 7; i += 1
                if not b[i - 1] & 0x80:
                    break
            num, wire = key >> 3, key & 7
            if wire == 0:
                v, n = 0, 0
                while True:
                    v |= (b[i] & 0x7F) << n; n += 7; i += 1
                    if not b[i - 1] & 0x80:
                        break
                yield num, v
            elif wire == 1:
                yield num, b[i:i + 8]; i += 8
            elif wire == 5:
                yield num, b[i:i + 4]; i += 4
            else:
                ln, n = 0, 0
                while True:
                    ln |= (b[i] & 0x7F) << n; n += 7; i += 1
                    if not b[i - 1] & 0x80:
                        break
                yield num, b[i:i + ln]; i += ln

    while off < len(buf):
        (ln,) = struct.unpack_from("<Q", buf, off)
        hdr = buf[off:off + 8]
        assert struct.unpack_from("<I", buf, off + 8)[0] == _masked(hdr), "length CRC mismatch"
        ev = buf[off + 12: off + 12 + ln]
        assert struct.unpack_from("<I", buf, off + 12 + ln)[0] == _masked(ev), "payload CRC mismatch"
        off += 16 + ln
        step, summ = 0, None
        for num, v in fields(ev):
            if num == 2: step = v
            if num == 5: summ = v
        if summ is None:
            continue
        for num, val in fields(summ):
            tag, sv = None, None
            for n2, v2 in fields(val):
                if n2 == 1: tag = v2.decode()
                if n2 == 2 and isinstance(v2, bytes) and len(v2) == 4: sv = struct.unpack("<f", v2)[0]
            if sv is not None:
                out.append((step, tag, sv))
    return out
