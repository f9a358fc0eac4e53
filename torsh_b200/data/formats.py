"""Dataset file formats read and written without their home frameworks: TFRecord (length-delimited records with masked
CRC-32C) with a minimal ``tf.train.Example`` codec, the MNIST IDX format, and the CIFAR-10 / CIFAR-100 python batches;
image-folder and CSV-manifest datasets on top of ``vision.io``. Nothing is downloaded: each loader reads a local path
in the layout the dataset is published in. Reference: crates/torsh-data/src/ (tfrecord_integration.rs, vision datasets).
"""
from __future__ import annotations

import gzip
import pickle
import struct
from pathlib import Path

import numpy as np
import torch

# ---- CRC-32C (Castagnoli), table-driven -------------------------------------------------------------------------------
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


def masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


# ---- TFRecord ------------------------------------------------------------------------------------------------------
class TFRecordWriter:
    def __init__(self, path):
        self.f = open(path, "wb")

    def write(self, record: bytes):
        head = struct.pack("<Q", len(record))
        self.f.write(head + struct.pack("<I", masked_crc(head)) + record + struct.pack("<I", masked_crc(record)))

    def close(self):
        self.f.close()

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


def read_tfrecords(path, verify: bool = True):
    """Yields the raw records of a TFRecord file; a length or payload checksum mismatch raises ``ValueError``."""
    with open(path, "rb") as f:
        while True:
            head = f.read(8)
            if not head:
                return
            if len(head) < 8:
                raise ValueError("truncated TFRecord header")
            (n,), (hc,) = struct.unpack("<Q", head), struct.unpack("<I", f.read(4))
            if verify and hc != masked_crc(head):
                raise ValueError("TFRecord length checksum mismatch")
            body = f.read(n)
            (bc,) = struct.unpack("<I", f.read(4))
            if len(body) < n or (verify and bc != masked_crc(body)):
                raise ValueError("TFRecord payload checksum mismatch or truncation")
            yield body


# minimal protobuf wire codec for tf.train.Example { features { feature: map<string, Feature> } }
def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _read_varint(buf: bytes, pos: int):
    shift = val = 0
    while True:
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7


def _ld(field: int, payload: bytes) -> bytes:
    return _varint((field << 3) | 2) + _varint(len(payload)) + payload


def encode_example(features: dict) -> bytes:
    """``features``: name -> bytes / str (BytesList), list of ints (Int64List) or list of floats (FloatList)."""
    entries = b""
    for name, v in features.items():
        if isinstance(v, (bytes, str)):
            v = [v]
        v = list(v.tolist() if hasattr(v, "tolist") else v)
        if v and isinstance(v[0], (bytes, str)):
            inner = _ld(1, b"".join(_ld(1, x.encode() if isinstance(x, str) else x) for x in v))
        elif v and isinstance(v[0], float):
            inner = _ld(2, _ld(1, struct.pack(f"<{len(v)}f", *v)))
        else:
            inner = _ld(3, _ld(1, b"".join(_varint(int(x) & 0xFFFFFFFFFFFFFFFF) for x in v)))
        entries += _ld(1, _ld(1, name.encode()) + _ld(2, inner))
    return _ld(1, entries)


def _fields(buf: bytes):
    pos = 0
    while pos < len(buf):
        key, pos = _read_varint(buf, pos)
        f, wt = key >> 3, key & 7
        if wt == 2:
            n, pos = _read_varint(buf, pos)
            yield f, wt, buf[pos:pos + n]
            pos += n
        elif wt == 0:
            v, pos = _read_varint(buf, pos)
            yield f, wt, v
        elif wt == 5:
            yield f, wt, buf[pos:pos + 4]
            pos += 4
        elif wt == 1:
            yield f, wt, buf[pos:pos + 8]
            pos += 8
        else:
            raise ValueError(f"unsupported protobuf wire type {wt}")


def decode_example(record: bytes) -> dict:
    out = {}
    for f, _, feats in _fields(record):
        if f != 1:
            continue
        for f2, _, entry in _fields(feats):
            if f2 != 1:
                continue
            name, value = None, None
            for f3, _, payload in _fields(entry):
                if f3 == 1:
                    name = payload.decode()
                elif f3 == 2:
                    for kind, _, lst in _fields(payload):
                        if kind == 1:
                            value = [p for f5, _, p in _fields(lst) if f5 == 1]
                        elif kind == 2:
                            vals = []
                            for f5, wt, p in _fields(lst):
                                if f5 == 1 and wt == 2:
                                    vals += list(struct.unpack(f"<{len(p) // 4}f", p))
                                elif f5 == 1 and wt == 5:
                                    vals.append(struct.unpack("<f", p)[0])
                            value = vals
                        elif kind == 3:
                            vals = []
                            for f5, wt, p in _fields(lst):
                                if f5 == 1 and wt == 2:
                                    q = 0
                                    while q < len(p):
                                        v, q = _read_varint(p, q)
                                        vals.append(v - (1 << 64) if v >> 63 else v)
                                elif f5 == 1 and wt == 0:
                                    vals.append(p - (1 << 64) if p >> 63 else p)
                            value = vals
            out[name] = value
    return out


class TFRecordDataset(torch.utils.data.IterableDataset):
    """Iterates decoded examples of one or more TFRecord files; ``transform(example_dict)`` shapes them into tensors."""

    def __init__(self, paths, transform=None, verify: bool = True):
        self.paths = [paths] if isinstance(paths, (str, Path)) else list(paths)
        self.transform, self.verify = transform, verify

    def __iter__(self):
        info = torch.utils.data.get_worker_info()
        paths = self.paths if info is None else self.paths[info.id::info.num_workers]
        for p in paths:
            for rec in read_tfrecords(p, self.verify):
                ex = decode_example(rec)
                yield self.transform(ex) if self.transform else ex


# ---- MNIST IDX -----------------------------------------------------------------------------------------------------
_IDX_TYPES = {0x08: np.uint8, 0x09: np.int8, 0x0B: ">i2", 0x0C: ">i4", 0x0D: ">f4", 0x0E: ">f8"}


def read_idx(path) -> torch.Tensor:
    p = Path(path)
    data = gzip.open(p, "rb").read() if p.suffix == ".gz" else p.read_bytes()
    if data[0] or data[1]:
        raise ValueError("not an IDX file")
    dt, nd = data[2], data[3]
    dims = struct.unpack(f">{nd}I", data[4:4 + 4 * nd])
    arr = np.frombuffer(data, dtype=_IDX_TYPES[dt], offset=4 + 4 * nd).reshape(dims)
    return torch.from_numpy(arr.astype(arr.dtype.newbyteorder("=")).copy())


def write_idx(path, t: torch.Tensor):
    a = t.numpy()
    code = {np.dtype(np.uint8): 0x08, np.dtype(np.int8): 0x09, np.dtype(np.int16): 0x0B, np.dtype(np.int32): 0x0C,
            np.dtype(np.float32): 0x0D, np.dtype(np.float64): 0x0E}[a.dtype]
    Path(path).write_bytes(bytes([0, 0, code, a.ndim]) + struct.pack(f">{a.ndim}I", *a.shape) + a.astype(a.dtype.newbyteorder(">")).tobytes())


class MNIST(torch.utils.data.Dataset):
    """``root/{train,t10k}-images-idx3-ubyte[.gz]`` and ``...-labels-idx1-ubyte[.gz]``."""

    def __init__(self, root, train: bool = True, transform=None):
        stem = "train" if train else "t10k"
        def find(name):
            for suffix in ("", ".gz"):
                p = Path(root) / (name + suffix)
                if p.exists():
                    return p
            raise FileNotFoundError(f"{name} not found under {root} (this library does not download)")
        self.images = read_idx(find(f"{stem}-images-idx3-ubyte"))
        self.labels = read_idx(find(f"{stem}-labels-idx1-ubyte")).long()
        self.transform = transform

    def __len__(self): return self.labels.numel()

    def __getitem__(self, i):
        x = self.images[i].float().div(255)[None]
        return (self.transform(x) if self.transform else x), int(self.labels[i])


class CIFAR(torch.utils.data.Dataset):
    """CIFAR-10 (``data_batch_1..5``, ``test_batch``) or CIFAR-100 (``train``, ``test``) python pickles under ``root``."""

    def __init__(self, root, train: bool = True, hundred: bool = False, transform=None):
        root = Path(root)
        names = (["train"] if train else ["test"]) if hundred else ([f"data_batch_{i}" for i in range(1, 6)] if train else ["test_batch"])
        xs, ys = [], []
        for n in names:
            p = root / n
            if not p.exists():
                if n.startswith("data_batch") and xs:
                    continue
                raise FileNotFoundError(f"{p} not found (this library does not download)")
            with open(p, "rb") as f:
                d = pickle.load(f, encoding="bytes")
            xs.append(np.asarray(d[b"data"], dtype=np.uint8).reshape(-1, 3, 32, 32))
            ys += list(d[b"fine_labels" if hundred else b"labels"])
        self.images, self.labels, self.transform = torch.from_numpy(np.concatenate(xs)), torch.tensor(ys), transform

    def __len__(self): return self.labels.numel()

    def __getitem__(self, i):
        x = self.images[i].float().div(255)
        return (self.transform(x) if self.transform else x), int(self.labels[i])


class ImageFolder(torch.utils.data.Dataset):
    """``root/<class name>/<image file>``; classes are the sorted directory names. Images are read with ``vision.io``."""

    def __init__(self, root, transform=None):
        from ..vision.io import global_io
        self.io, self.transform = global_io(), transform
        self.classes = sorted(d.name for d in Path(root).iterdir() if d.is_dir())
        self.samples = [(p, ci) for ci, c in enumerate(self.classes) for p in sorted((Path(root) / c).iterdir())
                        if p.is_file() and self.io.is_supported_image(p)]

    def __len__(self): return len(self.samples)

    def __getitem__(self, i):
        p, y = self.samples[i]
        x = self.io.load_image(p).float().div(255)
        return (self.transform(x) if self.transform else x), y
