"""Symmetric (peer-mapped) device memory and the per-communicator state the fused kernels need.

A :class:`SymmetricBuffer` is the same allocation on every rank of a process group, mapped into every
rank's address space: ``peer_ptrs[r]`` is rank ``r``'s copy as seen from this GPU, ``multicast_ptr``
(when the NVSwitch supports NVLS) is one address whose stores reach every copy and whose
``multimem.ld_reduce`` loads return the sum over all copies. Two allocators provide it: PyTorch's
symmetric-memory allocator (the default) and this package's own C++ heap over the CUDA virtual-memory API
(``TORSH_SYMM_BACKEND=native``: ``cuMemCreate`` blocks exchanged as file descriptors over Unix sockets, every
peer mapped with ``cuMemMap``, one multicast object per block; ``csrc/kernels/symm_heap.cu``). Everything
that touches the memory is this package's own kernels. The reference models this layer as ``MultiGpuContext`` with
``cudaMemcpyPeerAsync`` copies and a host-staged ring (``crates/torsh-backend/src/cuda/multi_gpu.rs:225-560``).

:class:`CommContext` adds what one stream of collectives needs: a symmetric flag array
(``[64][8]`` uint32, one slot per CTA) and a device-side epoch counter that every launch reads and a
one-thread kernel bumps afterwards, so captured CUDA graphs can replay collectives without
host-side bookkeeping. Collectives that may run concurrently need separate contexts.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

MAX_RANKS = 8
GUARD_BYTES = 256
CANARY_BYTE = 0xA5
FLAG_SLOTS = 320   # one cross-rank barrier slot per CTA of a collective kernel (COMM_MAX_BLOCKS in the CUDA source)


class _DevicePointer:
    """Lets torch wrap raw device memory without copying (CUDA array interface, bytes)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _tensor_at(ptr: int, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    return torch.as_tensor(_DevicePointer(ptr, nbytes), device=device).view(dtype)


class NativeSymmetricHeap:
    """One heap of the C++ symmetric allocator per process group (`tb_symm_*`). The group's first rank picks the job
    string; a barrier makes sure every rank's rendezvous socket is bound before the first allocation."""

    _heaps: dict = {}

    @classmethod
    def get(cls, group) -> "NativeSymmetricHeap":
        key = group.group_name if hasattr(group, "group_name") else id(group)
        if key not in cls._heaps:
            cls._heaps[key] = cls(group)
        return cls._heaps[key]

    def __init__(self, group):
        import uuid
        from .. import _native as nv
        self.group, self.rank, self.world = group, dist.get_rank(group), dist.get_world_size(group)
        job = [uuid.uuid4().hex[:16] if self.rank == 0 else None]
        dist.broadcast_object_list(job, src=dist.get_global_rank(group, 0), group=group)
        lib = nv.cuda()
        nv.stream_ptr()                      # binds the library to this process's device
        lib.tb_symm_init.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.tb_symm_alloc.argtypes = [ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                      ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
                                      ctypes.POINTER(ctypes.c_size_t)]
        lib.tb_symm_free.argtypes = [ctypes.c_void_p]
        self.lib = lib
        self.index = lib.tb_symm_init(job[0].encode(), self.rank, self.world, torch.cuda.current_device())
        if self.index < 0:
            raise RuntimeError(f"symmetric heap: {nv.cuda().tb_last_error().decode(errors='replace')}")
        dist.barrier(group)

    def alloc(self, nbytes: int, multicast: bool = True):
        """Collective. Returns (handle, [peer pointers], multicast pointer or 0, mapped bytes)."""
        from .. import _native as nv
        nv.stream_ptr()
        handle, mc, mapped = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_size_t()
        peers = (ctypes.c_void_p * MAX_RANKS)()
        rc = self.lib.tb_symm_alloc(self.index, nbytes, 1 if multicast else 0, ctypes.byref(handle), peers,
                                    ctypes.byref(mc), ctypes.byref(mapped))
        if rc != 0:
            raise RuntimeError(f"symmetric heap: {nv.cuda().tb_last_error().decode(errors='replace')}")
        return handle, [int(peers[q] or 0) for q in range(self.world)], int(mc.value or 0), int(mapped.value)

    def free(self, handle):
        self.lib.tb_symm_free(handle)


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group=None, zero: bool = True):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > MAX_RANKS:
            raise ValueError(f"symmetric buffers support up to {MAX_RANKS} ranks (one NVSwitch domain)")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.native = os.environ.get("TORSH_SYMM_BACKEND", "torch") == "native"
        if self.native:
            self._init_native(numel, dtype, dev)
            return
        import torch.distributed._symmetric_memory as symm_mem
        try:
            import warnings
            with warnings.catch_warnings():          # newer torch enables every group by itself and says so
                warnings.simplefilter("ignore")
                symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        # TORSH_SYMM_CANARIES=1 puts 256 guard bytes with a fixed pattern in front of and behind the payload of every
        # symmetric buffer; check_canaries() tells whether a kernel of this or another rank wrote outside its range
        self.guard_bytes = GUARD_BYTES if os.environ.get("TORSH_SYMM_CANARIES", "0") == "1" else 0
        es = torch.empty((), dtype=dtype).element_size()
        g = self.guard_bytes // es
        self._raw = symm_mem.empty(numel + 2 * g, dtype=dtype, device=dev)
        self.tensor = self._raw[g:g + numel]
        if zero:
            self.tensor.zero_()
        if g:
            self._raw.view(torch.uint8)[:self.guard_bytes].fill_(CANARY_BYTE)
            self._raw.view(torch.uint8)[self.guard_bytes + numel * es:].fill_(CANARY_BYTE)
        self.handle = symm_mem.rendezvous(self._raw, self.group)
        self.peer_ptrs = [int(p) + self.guard_bytes for p in self.handle.buffer_ptrs]
        try:
            mc = int(self.handle.multicast_ptr or 0)
            self.multicast_ptr = mc + self.guard_bytes if mc else 0
        except Exception:
            self.multicast_ptr = 0
        self._ptr_array = (ctypes.c_void_p * MAX_RANKS)(*(self.peer_ptrs + [0] * (MAX_RANKS - self.world)))
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def _init_native(self, numel: int, dtype: torch.dtype, dev: torch.device):
        """Block from the C++ heap: zero-filled by the allocator, every peer mapped, one multicast address."""
        self.guard_bytes = GUARD_BYTES if os.environ.get("TORSH_SYMM_CANARIES", "0") == "1" else 0
        es = torch.empty((), dtype=dtype).element_size()
        g = self.guard_bytes // es
        heap = NativeSymmetricHeap.get(self.group)
        self._heap = heap
        self._block, peers, mc, _ = heap.alloc((numel + 2 * g) * es)
        self.handle = None
        self._peer_base = peers
        self._raw = _tensor_at(peers[self.rank], numel + 2 * g, dtype, dev)
        self.tensor = self._raw[g:g + numel]
        if g:
            self._raw.view(torch.uint8)[:self.guard_bytes].fill_(CANARY_BYTE)
            self._raw.view(torch.uint8)[self.guard_bytes + numel * es:].fill_(CANARY_BYTE)
        self.peer_ptrs = [p + self.guard_bytes for p in peers]
        self.multicast_ptr = mc + self.guard_bytes if mc else 0
        self._ptr_array = (ctypes.c_void_p * MAX_RANKS)(*(self.peer_ptrs + [0] * (MAX_RANKS - self.world)))
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def release(self):
        """Collective: unmaps and releases a block of the native heap (no-op for the torch allocator, whose blocks go
        with their tensors)."""
        if getattr(self, "native", False) and self._block is not None:
            self.tensor = self._raw = None
            self._heap.free(self._block)
            self._block = None

    def check_canaries(self) -> bool:
        """True when the guard bytes around the payload are intact (always True when canaries are off)."""
        if not self.guard_bytes:
            return True
        raw = self._raw.view(torch.uint8)
        es = self._raw.element_size()
        front = raw[:self.guard_bytes]
        back = raw[self.guard_bytes + self.tensor.numel() * es:]
        return bool((front == CANARY_BYTE).all().item()) and bool((back == CANARY_BYTE).all().item())

    def peer_tensor(self, rank: int) -> torch.Tensor:
        """Rank ``rank``'s copy of the payload as a tensor of this process (peer-mapped memory): usable as the source or
        destination of copies and as a kernel operand, not by library kernels."""
        if rank == self.rank:
            return self.tensor
        g = self.guard_bytes // self._raw.element_size()
        if self.native:
            return _tensor_at(self._peer_base[rank], self._raw.numel(), self._raw.dtype, self._raw.device)[g:g + self.tensor.numel()]
        full = self.handle.get_buffer(rank, (self._raw.numel(),), self._raw.dtype, 0)
        return full[g:g + self.tensor.numel()]

    @property
    def ptr_array(self):
        """``void* [8]`` for the launchers."""
        return self._ptr_array

    def mc(self, use_nvls: bool = True) -> ctypes.c_void_p:
        return ctypes.c_void_p(self.multicast_ptr if use_nvls else 0)

    @property
    def has_multicast(self) -> bool:
        return self.multicast_ptr != 0


class CommContext:
    """Flags + epoch counter for one ordered stream of fused collectives."""

    def __init__(self, group=None):
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.flags = SymmetricBuffer(FLAG_SLOTS * MAX_RANKS, torch.int32, self.group, zero=True)
        # barrier values start at 2: a zero-initialised flag never satisfies the first wait
        self.epoch = torch.ones(1, dtype=torch.int32, device=self.flags.tensor.device)
        torch.cuda.synchronize()
        dist.barrier(self.group)
