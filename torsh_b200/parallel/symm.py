"""Symmetric (peer-mapped) device memory and the per-communicator state the fused kernels need.

A :class:`SymmetricBuffer` is the same allocation on every rank of a process group, mapped into every
rank's address space: ``peer_ptrs[r]`` is rank ``r``'s copy as seen from this GPU, ``multicast_ptr``
(when the NVSwitch supports NVLS) is one address whose stores reach every copy and whose
``multimem.ld_reduce`` loads return the sum over all copies. Allocation and handle exchange use
PyTorch's symmetric-memory allocator (the framework layer); everything that touches the memory is
this package's own kernels. The reference models this layer as ``MultiGpuContext`` with
``cudaMemcpyPeerAsync`` copies and a host-staged ring (``crates/torsh-backend/src/cuda/multi_gpu.rs:225-560``).

:class:`CommContext` adds what one stream of collectives needs: a symmetric flag array
(``[64][8]`` uint32, one slot per CTA) and a device-side epoch counter that every launch reads and a
one-thread kernel bumps afterwards, so captured CUDA graphs can replay collectives without
host-side bookkeeping. Collectives that may run concurrently need separate contexts.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

MAX_RANKS = 8
FLAG_SLOTS = 320   # one cross-rank barrier slot per CTA of a collective kernel (COMM_MAX_BLOCKS in the CUDA source)


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group=None, zero: bool = True):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > MAX_RANKS:
            raise ValueError(f"symmetric buffers support up to {MAX_RANKS} ranks (one NVSwitch domain)")
        dev = torch.device("cuda", torch.cuda.current_device())
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=dev)
        if zero:
            self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr or 0)
        except Exception:
            self.multicast_ptr = 0
        self._ptr_array = (ctypes.c_void_p * MAX_RANKS)(*(self.peer_ptrs + [0] * (MAX_RANKS - self.world)))
        torch.cuda.synchronize()
        dist.barrier(self.group)

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
