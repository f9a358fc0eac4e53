"""Process-group API with the reference's names over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

``init_process_group(backend, rank, world_size, master_addr, master_port)`` has the reference signature
(``crates/torsh-distributed/src/lib.rs:540-548``) but performs a real rendezvous; the reference stores
address and port and builds a ``MockBackend`` for every backend type
(``crates/torsh-distributed/src/process_group.rs:17-122``). Environment variables ``RANK/WORLD_SIZE/
LOCAL_RANK/MASTER_ADDR/MASTER_PORT`` and their ``TORSH_``-prefixed forms are honoured.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from enum import Enum

import torch
import torch.distributed as dist

from ..core.error import TorshDistributedError


class BackendType(Enum):
    NCCL = "nccl"; GLOO = "gloo"; MPI = "mpi"; CUSTOM = "custom"


@dataclass
class BackendConfig:
    """``crates/torsh-distributed/src/backend.rs:73-278``: timeout 30 s, 3 retries, backoff 2.0."""
    timeout_s: float = 30.0
    enable_compression: bool = False
    max_retries: int = 3
    retry_backoff: float = 2.0


def _env(name: str, default=None):
    return os.environ.get(name, os.environ.get("TORSH_" + name, default))


class ProcessGroup:
    """Handle with ``rank`` / ``world_size`` / address, wrapping a ``torch.distributed`` group."""

    def __init__(self, group, backend: BackendType, master_addr: str, master_port: int):
        self.group, self.backend, self.master_addr, self.master_port = group, backend, master_addr, master_port

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.group)

    def barrier(self, timeout_s: float | None = None):
        if timeout_s is None:
            dist.barrier(self.group)
            return
        w = dist.barrier(self.group, async_op=True)
        if not w.wait(datetime.timedelta(seconds=timeout_s)):
            raise TorshDistributedError.operation_timeout(f"barrier timed out after {timeout_s}s")

    def new_subgroup(self, ranks: list[int]) -> "ProcessGroup":
        return ProcessGroup(dist.new_group(ranks), self.backend, self.master_addr, self.master_port)


_default: ProcessGroup | None = None


def init_process_group(backend: str | BackendType | None = None, rank: int | None = None, world_size: int | None = None,
                       master_addr: str | None = None, master_port: int | None = None,
                       config: BackendConfig | None = None) -> ProcessGroup:
    global _default
    cfg = config or BackendConfig()
    if backend is None:
        backend = BackendType.NCCL if torch.cuda.is_available() else BackendType.GLOO
    backend = BackendType(backend) if not isinstance(backend, BackendType) else backend
    if backend in (BackendType.MPI, BackendType.CUSTOM):
        raise TorshDistributedError.feature_not_available(f"backend {backend.value} is not built (nccl and gloo are)")
    rank = int(_env("RANK", 0)) if rank is None else rank
    world_size = int(_env("WORLD_SIZE", 1)) if world_size is None else world_size
    master_addr = master_addr or _env("MASTER_ADDR", "127.0.0.1")
    master_port = int(master_port or _env("MASTER_PORT", 29500))
    if not 0 <= rank < world_size:
        raise TorshDistributedError.rank_out_of_bounds(f"rank {rank} not in [0, {world_size})")
    if not dist.is_initialized():
        kw = {}
        if backend is BackendType.NCCL:
            local = int(_env("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1)))
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend.value, init_method=f"tcp://{master_addr}:{master_port}", rank=rank,
                                world_size=world_size, timeout=datetime.timedelta(seconds=max(cfg.timeout_s, 1.0)), **kw)
    _default = ProcessGroup(dist.group.WORLD, backend, master_addr, master_port)
    return _default


def destroy_process_group():
    global _default
    if dist.is_initialized():
        dist.destroy_process_group()
    _default = None


def is_initialized() -> bool:
    return dist.is_initialized()


def is_available() -> bool:
    return dist.is_available()


def get_rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def get_world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def default_group() -> ProcessGroup:
    if _default is None:
        raise TorshDistributedError.backend_not_initialized("call init_process_group() first")
    return _default
