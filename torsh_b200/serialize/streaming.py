"""Chunked multi-tensor files and lazy loading (``crates/torsh-tensor/src/serialize/streaming.rs``,
``lazy_loading.rs``): a stream of named TRSH records followed by a JSON index and an 16-byte trailer
(``index offset u64 | magic "TRSX" | version u32``).  The writer appends records as tensors become available (a
checkpoint larger than host memory can be written tensor by tensor); the reader maps the file and decodes a tensor
only when it is asked for."""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

from .trsh import decode_trsh, encode_trsh

MAGIC = b"TRSX"


class StreamingWriter:
    def __init__(self, path, compression_level: int = 0):
        self.path, self.level = Path(path), compression_level
        self._f = open(self.path, "wb")
        self._index: dict[str, dict] = {}

    def write(self, name: str, tensor: torch.Tensor, metadata: dict | None = None) -> None:
        if name in self._index:
            raise KeyError(f"tensor {name!r} was already written")
        blob = encode_trsh(tensor, self.level, metadata)
        off = self._f.tell()
        self._f.write(blob)
        self._index[name] = {"offset": off, "size": len(blob), "shape": list(tensor.shape), "dtype": str(tensor.dtype).replace("torch.", "")}

    def write_state_dict(self, sd: dict) -> None:
        for k, v in sd.items():
            if isinstance(v, torch.Tensor):
                self.write(k, v)

    def close(self) -> None:
        if self._f.closed:
            return
        off = self._f.tell()
        self._f.write(json.dumps(self._index).encode())
        self._f.write(struct.pack("<Q4sI", off, MAGIC, 1))
        self._f.close()

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


class StreamingReader:
    def __init__(self, path):
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        off, magic, version = struct.unpack("<Q4sI", self._mm[-16:])
        if magic != MAGIC or version != 1:
            raise ValueError("not a streamed tensor file")
        self.index: dict[str, dict] = json.loads(self._mm[off:-16])
        self.loads = 0

    def keys(self): return list(self.index)
    def shape(self, name): return tuple(self.index[name]["shape"])
    def __contains__(self, name): return name in self.index
    def __len__(self): return len(self.index)

    def load(self, name: str) -> torch.Tensor:
        e = self.index[name]
        self.loads += 1
        return decode_trsh(self._mm[e["offset"]: e["offset"] + e["size"]])[0]

    __getitem__ = load

    def __iter__(self):
        for k in self.index:
            yield k, self.load(k)

    def load_into(self, module: torch.nn.Module, strict: bool = True) -> list[str]:
        """Copy matching tensors into ``module`` one at a time (peak extra memory = one tensor)."""
        missing = []
        with torch.no_grad():
            for n, p in list(module.named_parameters()) + list(module.named_buffers()):
                if n in self.index:
                    p.copy_(self.load(n).to(p.dtype))
                else:
                    missing.append(n)
        if strict and missing:
            raise KeyError(f"missing tensors: {missing[:5]}{'...' if len(missing) > 5 else ''}")
        return missing

    def close(self):
        self._mm.close(); self._f.close()

    def __enter__(self): return self
    def __exit__(self, *a): self.close()


class LazyTensor:
    """Handle that decodes on first use (``.get()``), as the reference's lazy loader does for mmapped storage."""

    def __init__(self, reader: StreamingReader, name: str):
        self.reader, self.name, self._t = reader, name, None

    @property
    def shape(self): return self.reader.shape(self.name)

    def get(self) -> torch.Tensor:
        if self._t is None:
            self._t = self.reader.load(self.name)
        return self._t
