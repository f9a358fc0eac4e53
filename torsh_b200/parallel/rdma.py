"""One-sided memory access API (``crates/torsh-distributed/src/rdma_support.rs:27-700``, where it is simulated): memory
regions registered under remote keys, endpoints and connections, READ / WRITE / SEND / compare-and-swap / fetch-and-add
work requests with completions, a registered-buffer pool and a tensor scheduler that splits transfers into work requests.

On one NVSwitch box the device-side equivalent of RDMA is peer-mapped symmetric memory (``parallel.symm``): the fused
kernels load and store a peer's buffer directly. This module is the host-side model of the same verbs; its fabric is a
process-local registry (ranks as threads) or any object with the same ``lookup`` method, which is what the tests drive."""
from __future__ import annotations

import enum
import itertools
import threading
import time
from dataclasses import dataclass, field

import torch


class RdmaOperation(enum.Enum):
    READ = "read"; WRITE = "write"; SEND = "send"; RECV = "recv"; ATOMIC_CAS = "cas"; ATOMIC_FAA = "faa"


class CompletionStatus(enum.Enum):
    SUCCESS = "success"; REMOTE_ACCESS_ERROR = "remote_access_error"; LOCAL_LENGTH_ERROR = "local_length_error"
    INVALID_KEY = "invalid_key"; NOT_CONNECTED = "not_connected"


class ConnectionState(enum.Enum):
    INIT = "init"; CONNECTED = "connected"; ERROR = "error"; CLOSED = "closed"


@dataclass
class MemoryAccess:
    local_write: bool = True
    remote_read: bool = True
    remote_write: bool = True
    remote_atomic: bool = True


@dataclass
class MemoryRegion:
    """A registered 1-D tensor; ``rkey`` names it to remote peers."""
    tensor: torch.Tensor
    rkey: int
    access: MemoryAccess = field(default_factory=MemoryAccess)

    @property
    def length(self) -> int:
        return self.tensor.numel()


@dataclass
class WorkRequest:
    wr_id: int
    op: RdmaOperation
    local: torch.Tensor | None
    remote_rank: int
    rkey: int
    remote_offset: int = 0
    compare: int = 0
    value: int = 0


@dataclass
class WorkCompletion:
    wr_id: int
    status: CompletionStatus
    op: RdmaOperation
    nbytes: int = 0
    result: int | None = None          # the old value for atomics


@dataclass
class RdmaStatistics:
    reads: int = 0
    writes: int = 0
    atomics: int = 0
    bytes_read: int = 0
    bytes_written: int = 0
    errors: int = 0


class LoopbackFabric:
    """Process-local fabric: every endpoint registers here; ``lookup(rank, rkey)`` finds a peer's region."""

    def __init__(self):
        self._regions: dict[tuple[int, int], MemoryRegion] = {}
        self.lock = threading.Lock()

    def publish(self, rank: int, region: MemoryRegion):
        with self.lock:
            self._regions[(rank, region.rkey)] = region

    def withdraw(self, rank: int, rkey: int):
        with self.lock:
            self._regions.pop((rank, rkey), None)

    def lookup(self, rank: int, rkey: int) -> MemoryRegion | None:
        with self.lock:
            return self._regions.get((rank, rkey))


class RdmaMemoryPool:
    """Pre-registered buffers in size classes (``RdmaMemoryPool``): registration is the expensive step, so buffers are
    registered once and handed out."""

    def __init__(self, endpoint: "RdmaEndpoint", sizes=(1 << 12, 1 << 16, 1 << 20), per_class: int = 4, dtype=torch.uint8):
        self.ep, self.dtype = endpoint, dtype
        self.free: dict[int, list[MemoryRegion]] = {s: [endpoint.register(torch.zeros(s, dtype=dtype)) for _ in range(per_class)] for s in sizes}
        self.stats = {"hits": 0, "misses": 0}

    def acquire(self, numel: int) -> MemoryRegion:
        for s in sorted(self.free):
            if s >= numel and self.free[s]:
                self.stats["hits"] += 1
                return self.free[s].pop()
        self.stats["misses"] += 1
        return self.ep.register(torch.zeros(numel, dtype=self.dtype))

    def release(self, region: MemoryRegion):
        self.free.setdefault(region.length, []).append(region)


class RdmaEndpoint:
    """One rank's side: registers regions, posts work requests against connected peers, polls completions."""

    _keys = itertools.count(1)

    def __init__(self, rank: int, fabric: LoopbackFabric):
        self.rank, self.fabric = rank, fabric
        self.regions: dict[int, MemoryRegion] = {}
        self.connections: dict[int, ConnectionState] = {}
        self.completions: list[WorkCompletion] = []
        self.stats = RdmaStatistics()
        self._wr = itertools.count(1)

    def register(self, tensor: torch.Tensor, access: MemoryAccess | None = None) -> MemoryRegion:
        assert tensor.dim() == 1 and tensor.is_contiguous(), "register 1-D contiguous tensors"
        mr = MemoryRegion(tensor, next(RdmaEndpoint._keys), access or MemoryAccess())
        self.regions[mr.rkey] = mr
        self.fabric.publish(self.rank, mr)
        return mr

    def deregister(self, mr: MemoryRegion):
        self.regions.pop(mr.rkey, None)
        self.fabric.withdraw(self.rank, mr.rkey)

    def connect(self, peer: int):
        self.connections[peer] = ConnectionState.CONNECTED

    def disconnect(self, peer: int):
        self.connections[peer] = ConnectionState.CLOSED

    def _fail(self, wr: WorkRequest, status: CompletionStatus) -> WorkCompletion:
        self.stats.errors += 1
        wc = WorkCompletion(wr.wr_id, status, wr.op)
        self.completions.append(wc)
        return wc

    def post(self, op: RdmaOperation, peer: int, rkey: int, local: torch.Tensor | None = None, remote_offset: int = 0,
             compare: int = 0, value: int = 0) -> WorkCompletion:
        wr = WorkRequest(next(self._wr), op, local, peer, rkey, remote_offset, compare, value)
        if self.connections.get(peer) is not ConnectionState.CONNECTED:
            return self._fail(wr, CompletionStatus.NOT_CONNECTED)
        mr = self.fabric.lookup(peer, rkey)
        if mr is None:
            return self._fail(wr, CompletionStatus.INVALID_KEY)
        a = mr.access
        if op is RdmaOperation.READ:
            if not a.remote_read:
                return self._fail(wr, CompletionStatus.REMOTE_ACCESS_ERROR)
            if remote_offset + local.numel() > mr.length:
                return self._fail(wr, CompletionStatus.LOCAL_LENGTH_ERROR)
            local.copy_(mr.tensor[remote_offset:remote_offset + local.numel()])
            self.stats.reads += 1
            self.stats.bytes_read += local.numel() * local.element_size()
            wc = WorkCompletion(wr.wr_id, CompletionStatus.SUCCESS, op, local.numel() * local.element_size())
        elif op is RdmaOperation.WRITE:
            if not a.remote_write:
                return self._fail(wr, CompletionStatus.REMOTE_ACCESS_ERROR)
            if remote_offset + local.numel() > mr.length:
                return self._fail(wr, CompletionStatus.LOCAL_LENGTH_ERROR)
            with self.fabric.lock:
                mr.tensor[remote_offset:remote_offset + local.numel()].copy_(local)
            self.stats.writes += 1
            self.stats.bytes_written += local.numel() * local.element_size()
            wc = WorkCompletion(wr.wr_id, CompletionStatus.SUCCESS, op, local.numel() * local.element_size())
        elif op in (RdmaOperation.ATOMIC_CAS, RdmaOperation.ATOMIC_FAA):
            if not a.remote_atomic:
                return self._fail(wr, CompletionStatus.REMOTE_ACCESS_ERROR)
            with self.fabric.lock:
                old = int(mr.tensor[remote_offset])
                if op is RdmaOperation.ATOMIC_FAA:
                    mr.tensor[remote_offset] = old + value
                elif old == compare:
                    mr.tensor[remote_offset] = value
            self.stats.atomics += 1
            wc = WorkCompletion(wr.wr_id, CompletionStatus.SUCCESS, op, mr.tensor.element_size(), result=old)
        else:
            return self._fail(wr, CompletionStatus.REMOTE_ACCESS_ERROR)
        self.completions.append(wc)
        return wc

    def poll(self, max_entries: int = 16) -> list[WorkCompletion]:
        out, self.completions = self.completions[:max_entries], self.completions[max_entries:]
        return out


class RdmaTensorScheduler:
    """Splits a tensor transfer into work requests of at most ``max_wr_elems`` elements (``RdmaTensorScheduler``)."""

    def __init__(self, endpoint: RdmaEndpoint, max_wr_elems: int = 1 << 20):
        self.ep, self.max = endpoint, max_wr_elems

    def _run(self, op, peer, rkey, flat, remote_offset):
        done = []
        for off in range(0, flat.numel(), self.max):
            done.append(self.ep.post(op, peer, rkey, flat[off:off + self.max], remote_offset + off))
            if done[-1].status is not CompletionStatus.SUCCESS:
                break
        return done

    def write_tensor(self, t: torch.Tensor, peer: int, rkey: int, remote_offset: int = 0) -> list[WorkCompletion]:
        return self._run(RdmaOperation.WRITE, peer, rkey, t.contiguous().reshape(-1), remote_offset)

    def read_tensor(self, out: torch.Tensor, peer: int, rkey: int, remote_offset: int = 0) -> list[WorkCompletion]:
        assert out.is_contiguous()
        return self._run(RdmaOperation.READ, peer, rkey, out.reshape(-1), remote_offset)
