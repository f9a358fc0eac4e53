"""``DeviceType`` and device-string parsing (``crates/torsh-core/src/device/types.rs:39-67,212``).

Only CPU and CUDA exist in this build; Metal / WebGPU variants parse (so configuration files written
for the reference load) but raise when used.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum

import torch

from .error import TorshError


class DeviceType(Enum):
    CPU = "cpu"
    CUDA = "cuda"
    METAL = "metal"
    WGPU = "wgpu"


@dataclass(frozen=True)
class Device:
    kind: DeviceType
    index: int = 0

    def __str__(self) -> str:
        return "cpu" if self.kind is DeviceType.CPU else f"{self.kind.value}:{self.index}"

    def torch(self) -> torch.device:
        if self.kind is DeviceType.CPU:
            return torch.device("cpu")
        if self.kind is DeviceType.CUDA:
            return torch.device("cuda", self.index)
        raise TorshError.device_error(f"{self} is not available in this build (CUDA sm_100a and CPU only)")

    def is_cuda(self) -> bool:
        return self.kind is DeviceType.CUDA


def parse_device(spec) -> Device:
    """``"cpu"``, ``"cuda"``, ``"cuda:3"``, ``"metal:0"``, ``"wgpu:0"`` → :class:`Device`."""
    if isinstance(spec, Device):
        return spec
    if isinstance(spec, torch.device):
        return Device(DeviceType(spec.type), spec.index or 0)
    s = str(spec).strip().lower()
    name, _, idx = s.partition(":")
    try:
        kind = DeviceType(name)
    except ValueError as e:
        raise TorshError.invalid_argument(f"unknown device {spec!r}") from e
    if idx and not idx.isdigit():
        raise TorshError.invalid_argument(f"bad device index in {spec!r}")
    return Device(kind, int(idx) if idx else 0)


def device_count() -> int:
    return torch.cuda.device_count()
