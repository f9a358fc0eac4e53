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
import os

import torch
import torch.distributed as dist

MAX_RANKS = 8
GUARD_BYTES = 256
CANARY_BYTE = 0xA5
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
