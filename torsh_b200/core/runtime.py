"""Python face of the native device runtime (``csrc/kernels/runtime.cu``, ``csrc/include/tb_pool.h``): device
properties, caching device / pinned / host memory pools, priority stream pool, event pool and the CUDA-graph cache —
the reference's ``CudaDevice`` / ``StreamPool`` / ``EventPool`` / graph cache / memory manager
(``crates/torsh-backend/src/cuda/{device,stream,event_coordination,graph}.rs``, ``src/cuda/memory/*``).

Streams handed out here are plain CUDA streams; :meth:`StreamPool.get` wraps them as ``torch.cuda.ExternalStream`` so
PyTorch ops and this library's kernels can be ordered on them.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _native as nv

_STAT_NAMES = ("allocated_bytes", "reserved_bytes", "peak_allocated_bytes", "peak_reserved_bytes", "alloc_calls",
               "free_calls", "cache_hits", "raw_allocs", "raw_frees", "splits", "merges", "oom_retries", "segments")
PRESSURE = ("low", "moderate", "high", "critical")
HIGH, NORMAL, LOW = 0, 1, 2


def _stats(fn, *args) -> dict:
    buf = (ctypes.c_uint64 * 13)()
    fn(*args, buf)
    return dict(zip(_STAT_NAMES, buf))


def _lib():
    lib = nv.require_cuda()
    if not getattr(lib, "_rt_typed", False):
        vp, u64 = ctypes.c_void_p, ctypes.c_uint64
        lib.tb_rt_malloc.restype, lib.tb_rt_malloc.argtypes = vp, [u64, vp]
        lib.tb_rt_free.argtypes = [vp]
        lib.tb_rt_empty_cache.restype = u64
        lib.tb_rt_set_mem_limit.argtypes = [u64]
        lib.tb_rt_fragmentation.restype = ctypes.c_double
        lib.tb_rt_pinned_alloc.restype, lib.tb_rt_pinned_alloc.argtypes = vp, [u64]
        lib.tb_rt_pinned_free.argtypes = [vp]
        lib.tb_rt_memcpy_async.argtypes = [vp, vp, u64, vp]
        lib.tb_rt_memset_async.argtypes = [vp, ctypes.c_int, u64, vp]
        lib.tb_rt_managed_alloc.restype, lib.tb_rt_managed_alloc.argtypes = vp, [u64]
        lib.tb_rt_managed_free.argtypes = [vp]
        lib.tb_rt_managed_prefetch.argtypes = [vp, u64, ctypes.c_int, vp]
        lib.tb_rt_managed_advise.argtypes = [vp, u64, ctypes.c_int, ctypes.c_int]
        lib.tb_rt_stream_get.restype, lib.tb_rt_stream_get.argtypes = vp, [ctypes.c_int, ctypes.c_int]
        for f in ("tb_rt_stream_priority", "tb_rt_stream_sync", "tb_rt_stream_query"):
            getattr(lib, f).argtypes = [vp]
        lib.tb_rt_event_acquire.restype, lib.tb_rt_event_acquire.argtypes = vp, [ctypes.c_int]
        lib.tb_rt_event_release.argtypes = [vp, ctypes.c_int]
        lib.tb_rt_event_record.argtypes = [vp, vp]
        lib.tb_rt_stream_wait_event.argtypes = [vp, vp]
        lib.tb_rt_event_sync.argtypes = [vp]
        lib.tb_rt_event_query.argtypes = [vp]
        lib.tb_rt_event_elapsed_ms.restype, lib.tb_rt_event_elapsed_ms.argtypes = ctypes.c_float, [vp, vp]
        lib.tb_rt_graph_begin.argtypes = [vp]
        lib.tb_rt_graph_end.argtypes = [vp, u64]
        lib.tb_rt_graph_has.argtypes = [u64]
        lib.tb_rt_graph_launch.argtypes = [u64, vp]
        lib.tb_rt_graph_node_count.argtypes = [u64]
        lib.tb_rt_graph_set_capacity.argtypes = [u64]
        lib.tb_rt_occupancy.argtypes = [ctypes.c_int, ctypes.c_int, u64, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        lib._rt_typed = True
    nv.stream_ptr()  # binds the library to torch's current device
    return lib


@dataclass
class DeviceInfo:
    name: str
    sm_count: int
    smem_per_block_optin: int
    smem_per_sm: int
    l2_bytes: int
    total_memory: int
    free_memory: int
    capability: tuple[int, int]
    sm_clock_khz: int
    mem_clock_khz: int
    bus_width_bits: int
    max_threads_per_sm: int
    regs_per_sm: int
    cluster_launch: bool
    warp_size: int
    tmem_columns: int

    @property
    def peak_hbm_gbs(self) -> float:
        """Nominal DRAM bandwidth from clock x bus width x 2 (double data rate)."""
        return self.mem_clock_khz * 1e3 * self.bus_width_bits / 8 * 2 / 1e9


def device_info(device: int | None = None) -> DeviceInfo:
    lib = _lib()
    out, name = (ctypes.c_uint64 * 16)(), ctypes.create_string_buffer(64)
    nv.check(lib.tb_rt_device_info(torch.cuda.current_device() if device is None else device, out, name), "device_info")
    v = list(out)
    return DeviceInfo(name.value.decode(), v[0], v[1], v[2], v[3], v[4], v[5], (v[6], v[7]), v[8], v[9], v[10], v[11],
                      v[12], bool(v[13]), v[14], v[15])


def occupancy(threads: int, regs_per_thread: int, smem_bytes: int) -> tuple[int, str]:
    lib = _lib()
    n, lim = ctypes.c_int(), ctypes.c_int()
    nv.check(lib.tb_rt_occupancy(threads, regs_per_thread, smem_bytes, ctypes.byref(n), ctypes.byref(lim)), "occupancy")
    return n.value, ("threads", "registers", "shared memory", "CTA slots")[lim.value]


# ------------------------------------------------------------------------------------------------ memory
class DeviceBuffer:
    """A block from the device pool; ``tensor()`` views it as a torch tensor (no copy, no ownership transfer)."""

    def __init__(self, nbytes: int, stream: torch.cuda.Stream | None = None):
        lib = _lib()
        self.nbytes = nbytes
        self.ptr = lib.tb_rt_malloc(nbytes, nv.stream_ptr(stream))
        if not self.ptr:
            raise torch.cuda.OutOfMemoryError(lib.tb_last_error().decode())

    def tensor(self, shape, dtype=torch.uint8) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        if n * torch.empty((), dtype=dtype).element_size() > self.nbytes:
            raise ValueError("view larger than the buffer")

        class _Holder:  # __cuda_array_interface__ provider keeps `self` alive through the tensor
            pass
        h = _Holder()
        h.owner = self
        typestr = {torch.uint8: "|u1", torch.float32: "<f4", torch.float16: "<f2", torch.int32: "<i4", torch.int64: "<i8"}
        if dtype == torch.bfloat16:
            h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2", "data": (self.ptr, False), "version": 2}
            return torch.as_tensor(h, device="cuda").view(torch.bfloat16)
        h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr[dtype], "data": (self.ptr, False), "version": 2}
        return torch.as_tensor(h, device="cuda")

    def free(self):
        if self.ptr:
            nv.check(_lib().tb_rt_free(self.ptr), "tb_rt_free")
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DeviceMemoryPool:
    """Statistics and controls of the current device's caching pool."""

    @staticmethod
    def stats() -> dict: return _stats(_lib().tb_rt_mem_stats)
    @staticmethod
    def empty_cache() -> int: return _lib().tb_rt_empty_cache()
    @staticmethod
    def set_limit(nbytes: int) -> None: _lib().tb_rt_set_mem_limit(nbytes)
    @staticmethod
    def reset_peak() -> None: _lib().tb_rt_reset_peak()
    @staticmethod
    def pressure() -> str: return PRESSURE[_lib().tb_rt_mem_pressure()]
    @staticmethod
    def fragmentation() -> float: return _lib().tb_rt_fragmentation()
    @staticmethod
    def alloc(nbytes: int, stream=None) -> DeviceBuffer: return DeviceBuffer(nbytes, stream)


def use_as_torch_allocator() -> None:
    """Route PyTorch's CUDA allocations through this pool (must run before the first CUDA allocation)."""
    from .. import _build
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_build.LIBDIR / "libtorsh_b200_cuda.so"), "tb_torch_alloc", "tb_torch_free")
    torch.cuda.memory.change_current_allocator(alloc)


class PinnedBuffer:
    def __init__(self, nbytes: int):
        lib = _lib()
        self.nbytes, self.ptr = nbytes, lib.tb_rt_pinned_alloc(nbytes)
        if not self.ptr:
            raise MemoryError(f"pinned pool: cannot allocate {nbytes} bytes")

    def tensor(self, shape, dtype=torch.uint8) -> torch.Tensor:
        ct = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)
        t = torch.frombuffer(ct, dtype=torch.uint8).view(dtype).reshape(shape) if dtype != torch.uint8 else \
            torch.frombuffer(ct, dtype=torch.uint8).reshape(shape)
        t._pinned_owner = self
        return t

    def copy_to_device_async(self, dst: torch.Tensor, stream=None) -> None:
        nv.check(_lib().tb_rt_memcpy_async(dst.data_ptr(), self.ptr, min(self.nbytes, dst.numel() * dst.element_size()),
                                           nv.stream_ptr(stream)), "memcpy_async")

    def free(self):
        if self.ptr:
            _lib().tb_rt_pinned_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    @staticmethod
    def stats() -> dict: return _stats(_lib().tb_rt_pinned_stats)


class UnifiedBuffer:
    """Managed memory (``crates/torsh-backend/src/cuda/unified_buffer.rs``, ``backend.rs:464-629``): one allocation that
    the host and the device address through the same pointer. ``host_view`` is a CPU tensor over it; ``prefetch`` moves
    the pages ahead of use and ``advise`` sets read-mostly / preferred-location / accessed-by hints. Device kernels take
    ``ptr`` (or a tensor made by a kernel-side wrapper); synchronise before reading on the other side."""

    READ_MOSTLY, PREFERRED_LOCATION, ACCESSED_BY = 0, 1, 2

    def __init__(self, nbytes: int):
        self.nbytes, self.ptr = nbytes, _lib().tb_rt_managed_alloc(nbytes)
        if not self.ptr:
            raise MemoryError(f"managed memory: cannot allocate {nbytes} bytes")

    def host_view(self, shape, dtype=torch.uint8) -> torch.Tensor:
        ct = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)
        t = torch.frombuffer(ct, dtype=torch.uint8)
        t = (t.view(dtype) if dtype != torch.uint8 else t).reshape(shape)
        t._managed_owner = self
        return t

    def prefetch(self, device: int | None = None, stream=None) -> None:
        """``device=None``: the current GPU; ``device=-1``: back to the host."""
        dev = torch.cuda.current_device() if device is None else device
        nv.check(_lib().tb_rt_managed_prefetch(self.ptr, self.nbytes, dev, nv.stream_ptr(stream)), "managed_prefetch")

    def advise(self, advice: int, device: int | None = None) -> None:
        dev = torch.cuda.current_device() if device is None else device
        nv.check(_lib().tb_rt_managed_advise(self.ptr, self.nbytes, advice, dev), "managed_advise")

    def copy_to(self, dst: torch.Tensor, stream=None) -> None:
        nv.check(_lib().tb_rt_memcpy_async(dst.data_ptr(), self.ptr, min(self.nbytes, dst.numel() * dst.element_size()),
                                           nv.stream_ptr(stream)), "memcpy_async")

    def free(self):
        if self.ptr:
            _lib().tb_rt_managed_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class HostPool:
    """The same pool over plain host memory (``libtorsh_b200_host.so``): works without a GPU."""

    def __init__(self, raw_budget: int = 0, limit: int = 0):
        self.lib = nv.host()
        vp, u64 = ctypes.c_void_p, ctypes.c_uint64
        self.lib.tsh_pool_create.restype, self.lib.tsh_pool_create.argtypes = vp, [u64, u64]
        self.lib.tsh_pool_alloc.restype, self.lib.tsh_pool_alloc.argtypes = vp, [vp, u64, u64]
        self.lib.tsh_pool_free.argtypes = [vp, vp]
        self.lib.tsh_pool_destroy.argtypes = [vp]
        self.lib.tsh_pool_release_cached.restype, self.lib.tsh_pool_release_cached.argtypes = u64, [vp]
        self.lib.tsh_pool_round_size.restype, self.lib.tsh_pool_round_size.argtypes = u64, [u64]
        self.lib.tsh_pool_size_of.restype, self.lib.tsh_pool_size_of.argtypes = u64, [vp, vp]
        self.lib.tsh_pool_stats.argtypes = [vp, ctypes.POINTER(ctypes.c_uint64 * 13)]
        self.lib.tsh_pool_pressure.argtypes = [vp, u64]
        self.lib.tsh_pool_fragmentation.restype, self.lib.tsh_pool_fragmentation.argtypes = ctypes.c_double, [vp]
        self.h = self.lib.tsh_pool_create(raw_budget, limit)

    def alloc(self, nbytes: int, stream: int = 0) -> int | None: return self.lib.tsh_pool_alloc(self.h, nbytes, stream)
    def free(self, p: int) -> bool: return self.lib.tsh_pool_free(self.h, p) == 0
    def release_cached(self) -> int: return self.lib.tsh_pool_release_cached(self.h)
    def round_size(self, n: int) -> int: return self.lib.tsh_pool_round_size(n)
    def size_of(self, p: int) -> int: return self.lib.tsh_pool_size_of(self.h, p)
    def pressure(self, capacity: int) -> str: return PRESSURE[self.lib.tsh_pool_pressure(self.h, capacity)]
    def fragmentation(self) -> float: return self.lib.tsh_pool_fragmentation(self.h)

    def stats(self) -> dict:
        buf = (ctypes.c_uint64 * 13)()
        self.lib.tsh_pool_stats(self.h, ctypes.byref(buf))
        return dict(zip(_STAT_NAMES, buf))

    def close(self):
        if self.h:
            self.lib.tsh_pool_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------------------------ streams / events
class StreamPool:
    """Round-robin pools of non-blocking streams in three priority classes (HIGH for communication, NORMAL, LOW for
    prefetch / copies)."""

    def __init__(self, size_per_class: int = 4):
        self.size = size_per_class

    def get_raw(self, cls: int = NORMAL) -> int:
        s = _lib().tb_rt_stream_get(cls, self.size)
        if not s:
            raise nv.NativeError("could not create a stream")
        return s

    def get(self, cls: int = NORMAL) -> torch.cuda.Stream:
        return torch.cuda.ExternalStream(self.get_raw(cls))

    @staticmethod
    def priority(stream) -> int:
        return _lib().tb_rt_stream_priority(ctypes.c_void_p(stream if isinstance(stream, int) else stream.cuda_stream))

    @staticmethod
    def count(cls: int) -> int: return _lib().tb_rt_stream_count(cls)


class Event:
    """Pooled CUDA event."""

    def __init__(self, timing: bool = False):
        self.timing = timing
        self.h = _lib().tb_rt_event_acquire(int(timing))
        if not self.h:
            raise nv.NativeError("could not create an event")

    def record(self, stream=None):
        nv.check(_lib().tb_rt_event_record(self.h, nv.stream_ptr(stream)), "event_record"); return self
    def wait(self, stream=None): nv.check(_lib().tb_rt_stream_wait_event(nv.stream_ptr(stream), self.h), "stream_wait_event")
    def synchronize(self): nv.check(_lib().tb_rt_event_sync(self.h), "event_sync")
    def query(self) -> bool: return _lib().tb_rt_event_query(self.h) == 1
    def elapsed_ms(self, end: "Event") -> float: return _lib().tb_rt_event_elapsed_ms(self.h, end.h)

    def release(self):
        if self.h:
            _lib().tb_rt_event_release(self.h, int(self.timing))
            self.h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    @staticmethod
    def pool_stats() -> dict:
        buf = (ctypes.c_uint64 * 2)()
        _lib().tb_rt_event_stats(buf)
        return {"created": buf[0], "reused": buf[1]}


# ------------------------------------------------------------------------------------------------ graphs
class GraphCache:
    """Instantiated CUDA graphs keyed by an integer (callers hash shape / phase into it); least recently launched
    entries are evicted beyond the capacity."""

    def __init__(self, capacity: int | None = None):
        if capacity:
            _lib().tb_rt_graph_set_capacity(capacity)

    @staticmethod
    def key(*parts) -> int:
        return hash(parts) & 0xFFFFFFFFFFFFFFFF

    def has(self, key: int) -> bool: return bool(_lib().tb_rt_graph_has(key))

    def capture(self, key: int, fn, stream: torch.cuda.Stream | None = None) -> None:
        """Run ``fn()`` under capture on ``stream`` (default: a pooled stream) and store the instantiated graph.
        ``fn`` must launch only this library's kernels or capture-safe work, and allocate nothing."""
        lib = _lib()
        stream = stream or StreamPool().get(NORMAL)
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            nv.check(lib.tb_rt_graph_begin(nv.stream_ptr(stream)), "graph_begin")
            try:
                fn()
            finally:
                rc = lib.tb_rt_graph_end(nv.stream_ptr(stream), key)
            nv.check(rc, "graph_end")
        torch.cuda.current_stream().wait_stream(stream)

    def launch(self, key: int, stream=None) -> None:
        nv.check(_lib().tb_rt_graph_launch(key, nv.stream_ptr(stream)), "graph_launch")

    def node_count(self, key: int) -> int: return _lib().tb_rt_graph_node_count(key)
    def clear(self) -> None: _lib().tb_rt_graph_clear()

    def stats(self) -> dict:
        buf = (ctypes.c_uint64 * 4)()
        _lib().tb_rt_graph_stats(buf)
        return dict(zip(("entries", "hits", "misses", "evictions"), buf))
