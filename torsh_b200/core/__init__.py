"""Core vocabulary: dtypes, devices, shapes, errors, runtime configuration, distributed metadata."""
from .device import Device, DeviceType, device_count, parse_device
from .dtype import DType, from_torch_dtype, to_torch_dtype
from .error import TorshDistributedError, TorshError
from .runtime_config import RuntimeConfig
from .shape import Shape

__all__ = ["DType", "Device", "DeviceType", "Shape", "TorshError", "TorshDistributedError", "RuntimeConfig",
           "device_count", "parse_device", "from_torch_dtype", "to_torch_dtype"]
