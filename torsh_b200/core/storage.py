"""Storage layer of the core: memory formats and their strides, aligned / memory-mapped / shared storages with views,
a registry with memory accounting, and chunking helpers sized for the B200 memory hierarchy.
Reference: crates/torsh-core/src/storage/{memory_format,aligned,mapped,views,registry,memory_info}.rs, chunking.rs.
"""
from __future__ import annotations

import enum
import math
import mmap
import os
import threading
import weakref
from dataclasses import dataclass

import torch


class MemoryFormat(enum.Enum):
    CONTIGUOUS = "contiguous"              # row-major
    CHANNELS_LAST = "channels_last"        # NHWC strides on a 4-D NCHW shape
    CHANNELS_LAST_3D = "channels_last_3d"  # NDHWC strides on a 5-D shape
    STRIDED = "strided"                    # anything else

    def strides(self, shape) -> tuple:
        """Element strides of ``shape`` (given in logical N, C, spatial... order) in this format."""
        shape = tuple(int(s) for s in shape)
        if self is MemoryFormat.CONTIGUOUS or self is MemoryFormat.STRIDED:
            out, acc = [], 1
            for s in reversed(shape):
                out.append(acc)
                acc *= max(s, 1)
            return tuple(reversed(out))
        want = 4 if self is MemoryFormat.CHANNELS_LAST else 5
        if len(shape) != want:
            raise ValueError(f"{self.value} needs a {want}-D shape, got {len(shape)}-D")
        order = [0] + list(range(2, want)) + [1]                     # physical order: N, spatial..., C
        strides, acc = [0] * want, 1
        for d in reversed(order):
            strides[d] = acc
            acc *= max(shape[d], 1)
        return tuple(strides)

    def to_torch(self):
        return {MemoryFormat.CONTIGUOUS: torch.contiguous_format, MemoryFormat.CHANNELS_LAST: torch.channels_last,
                MemoryFormat.CHANNELS_LAST_3D: torch.channels_last_3d}.get(self, torch.preserve_format)

    @staticmethod
    def of(t: torch.Tensor) -> "MemoryFormat":
        if t.is_contiguous():
            return MemoryFormat.CONTIGUOUS
        if t.dim() == 4 and t.is_contiguous(memory_format=torch.channels_last):
            return MemoryFormat.CHANNELS_LAST
        if t.dim() == 5 and t.is_contiguous(memory_format=torch.channels_last_3d):
            return MemoryFormat.CHANNELS_LAST_3D
        return MemoryFormat.STRIDED


@dataclass
class MemoryInfo:
    allocated_bytes: int = 0
    peak_bytes: int = 0
    allocations: int = 0
    live: int = 0


class StorageRegistry:
    """Accounts for the storages created through this module (bytes now, peak, counts per kind)."""

    def __init__(self):
        self._lock = threading.Lock()
        self.info: dict[str, MemoryInfo] = {}

    def _add(self, kind: str, nbytes: int):
        with self._lock:
            i = self.info.setdefault(kind, MemoryInfo())
            i.allocated_bytes += nbytes
            i.peak_bytes = max(i.peak_bytes, i.allocated_bytes)
            i.allocations += 1
            i.live += 1

    def _remove(self, kind: str, nbytes: int):
        with self._lock:
            i = self.info[kind]
            i.allocated_bytes -= nbytes
            i.live -= 1

    def total_bytes(self) -> int:
        return sum(i.allocated_bytes for i in self.info.values())


registry = StorageRegistry()


class Storage:
    """A typed, flat buffer with explicit provenance. ``tensor`` is the 1-D view of all elements; ``view(shape, offset,
    strides)`` gives strided views without copying. Kinds: ``aligned`` (host or device memory whose base address is a
    multiple of ``alignment``), ``mapped`` (a file mapped into memory, shared between processes), ``shared`` (POSIX
    shared memory through torch's ``share_memory_``)."""

    def __init__(self, tensor: torch.Tensor, kind: str, keep=None):
        self.tensor, self.kind, self._keep = tensor, kind, keep
        self.nbytes = tensor.numel() * tensor.element_size()
        registry._add(kind, self.nbytes)
        weakref.finalize(self, registry._remove, kind, self.nbytes)

    # ---- constructors ----
    @classmethod
    def aligned(cls, numel: int, dtype=torch.float32, alignment: int = 256, device="cpu") -> "Storage":
        es = torch.empty((), dtype=dtype).element_size()
        if alignment % es or alignment & (alignment - 1):
            raise ValueError("alignment must be a power of two and a multiple of the element size")
        raw = torch.empty(numel * es + alignment, dtype=torch.uint8, device=device)
        off = (-raw.data_ptr()) % alignment
        t = raw[off:off + numel * es].view(dtype)
        assert t.data_ptr() % alignment == 0
        return cls(t, "aligned", keep=raw)

    @classmethod
    def mapped(cls, path, numel: int, dtype=torch.float32, create: bool = False) -> "Storage":
        es = torch.empty((), dtype=dtype).element_size()
        nbytes = numel * es
        if create or not os.path.exists(path):
            with open(path, "wb") as f:
                f.truncate(nbytes)
        f = open(path, "r+b")
        mm = mmap.mmap(f.fileno(), nbytes)
        t = torch.frombuffer(mm, dtype=dtype, count=numel)
        return cls(t, "mapped", keep=(mm, f))

    @classmethod
    def shared(cls, numel: int, dtype=torch.float32) -> "Storage":
        t = torch.zeros(numel, dtype=dtype)
        t.share_memory_()
        return cls(t, "shared")

    # ---- views ----
    def view(self, shape, offset: int = 0, strides=None, fmt: MemoryFormat = MemoryFormat.CONTIGUOUS) -> torch.Tensor:
        strides = tuple(strides) if strides is not None else fmt.strides(shape)
        span = sum((s - 1) * st for s, st in zip(shape, strides)) + 1 if all(s > 0 for s in shape) else 0
        if offset < 0 or offset + span > self.tensor.numel():
            raise ValueError(f"view of span {span} at offset {offset} exceeds the storage of {self.tensor.numel()} elements")
        # as_strided counts its offset from the start of the underlying allocation, not from this storage's first element
        return torch.as_strided(self.tensor, tuple(shape), strides, self.tensor.storage_offset() + offset)

    def flush(self):
        if self.kind == "mapped":
            self._keep[0].flush()

    def __len__(self):
        return self.tensor.numel()


# ---- chunking ------------------------------------------------------------------------------------------------------
class ChunkingStrategy(enum.Enum):
    COMPUTE_INTENSIVE = "compute"      # few large chunks: one per SM wave
    MEMORY_INTENSIVE = "memory"        # chunks sized to stay inside L2
    CACHE_FRIENDLY = "cache"           # chunks sized to shared memory
    CUSTOM = "custom"


@dataclass
class TensorChunkConfig:
    strategy: ChunkingStrategy = ChunkingStrategy.MEMORY_INTENSIVE
    custom_bytes: int = 0
    l2_bytes: int = 126 << 20          # B200
    smem_bytes: int = 227 << 10
    sms: int = 148
    alignment: int = 256

    def compute_chunk_size(self, numel: int, element_size: int) -> int:
        """Elements per chunk (a multiple of the alignment, at least one alignment unit, at most the tensor)."""
        total = numel * element_size
        if self.strategy is ChunkingStrategy.COMPUTE_INTENSIVE:
            want = math.ceil(total / self.sms)
        elif self.strategy is ChunkingStrategy.MEMORY_INTENSIVE:
            want = self.l2_bytes // 4            # two inputs and an output resident with room to spare
        elif self.strategy is ChunkingStrategy.CACHE_FRIENDLY:
            want = self.smem_bytes // 2
        else:
            want = self.custom_bytes
        want = max(self.alignment, want // self.alignment * self.alignment)
        return max(1, min(numel, want // element_size))

    def chunks(self, numel: int, element_size: int):
        n = self.compute_chunk_size(numel, element_size)
        return [(s, min(s + n, numel)) for s in range(0, numel, n)]


def is_aligned(t: torch.Tensor, alignment: int = 16) -> bool:
    return t.data_ptr() % alignment == 0
