"""Shared helpers for the op wrappers: dtype codes, alignment checks, ctypes signatures."""
from __future__ import annotations

import ctypes

import torch

from .. import _native as nv

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
_sigs_done: set[str] = set()


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"kernel supports bf16 / fp32, got {t.dtype}")


def kernel_ok(*tensors: torch.Tensor) -> bool:
    """True when every tensor is a CUDA bf16/fp32 tensor (the kernels' domain)."""
    return all(t is None or (t.is_cuda and t.dtype in (torch.bfloat16, torch.float32)) for t in tensors)


def aligned(t: torch.Tensor) -> torch.Tensor:
    """Contiguous and 16-byte aligned (copies only when needed)."""
    if not t.is_contiguous():
        t = t.contiguous()
    if t.data_ptr() % 16:
        t = t.clone()
    return t


def fn(name: str, argtypes):
    """Fetch a launcher from the CUDA library and set its signature once."""
    lib = nv.require_cuda()
    f = getattr(lib, name)
    if name not in _sigs_done:
        f.restype = ctypes.c_int
        f.argtypes = argtypes
        _sigs_done.add(name)
    return f


_KERNELS_PER_CALL = {"tb_flash_attn_bwd": 3, "tb_lamb_multi": 2, "tb_bn_fwd": 3, "tb_bn_bwd": 3}


def call(name: str, argtypes, *args):
    nv.check(fn(name, argtypes)(*args), name)
    nv.launch_count += _KERNELS_PER_CALL.get(name, 1)
