"""ctypes bridge to the two in-tree native libraries.

``cuda()`` returns ``libtorsh_b200_cuda.so`` (sm_100a kernels), ``host()`` returns
``libtorsh_b200_host.so`` (C++ runtime). On a machine with a GPU a missing CUDA library is an
error, never a silent fallback: every op that has a kernel calls :func:`require_cuda` first.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent / "lib"
_lock = threading.Lock()
_cuda_lib = None
_host_lib = None
_status = {}
launch_count = 0  # kernels of this library launched so far (incremented by the op wrappers)

c_void_p, c_int, c_float, c_long, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_int64, ctypes.c_size_t


class NativeError(RuntimeError):
    """A native launcher refused its arguments or a CUDA call failed."""


class KernelTimeout(RuntimeError):
    """A bounded device-side wait ran out; the kernel set its status word and returned."""


class KernelCheckFailed(RuntimeError):
    """A device-side check (``TORSH_KERNEL_CHECKS=1``) found an index outside its range; the kernel skipped the access,
    recorded the code in the status word and carried on."""


def _load(name: str, build_fn: str):
    path = _LIBDIR / name
    if not path.exists() and os.environ.get("TORSH_B200_NO_AUTOBUILD") != "1":
        from . import _build
        getattr(_build, build_fn)()
    if not path.exists():
        raise NativeError(f"{path} is missing: run `python -m torsh_b200._build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL)


def cuda():
    """The CUDA kernel library (loaded on first use)."""
    global _cuda_lib
    if _cuda_lib is None:
        with _lock:
            if _cuda_lib is None:
                lib = _load("libtorsh_b200_cuda.so", "build_cuda")
                lib.tb_last_error.restype = ctypes.c_char_p
                _cuda_lib = lib
    return _cuda_lib


def host():
    """The host runtime library (loaded on first use)."""
    global _host_lib
    if _host_lib is None:
        with _lock:
            if _host_lib is None:
                _host_lib = _load("libtorsh_b200_host.so", "build_host")
    return _host_lib


def cuda_available() -> bool:
    return torch.cuda.is_available()


def require_cuda():
    if not torch.cuda.is_available():
        raise NativeError("this op needs a CUDA device")
    return cuda()


def check(rc: int, what: str = "") -> None:
    """Raise when a launcher returned a non-zero code."""
    if rc != 0:
        msg = cuda().tb_last_error().decode(errors="replace")
        raise NativeError(f"{what} failed (rc={rc}): {msg}")


_bound_device = -1


def stream_ptr(stream: torch.cuda.Stream | None = None) -> c_void_p:
    """Raw handle of the launch stream. Also tells the native library which device is current
    (its statically linked CUDA runtime keeps its own per-thread device)."""
    global _bound_device
    d = torch.cuda.current_device()
    if d != _bound_device:
        cuda().tb_set_device(d)
        _bound_device = d
    s = stream if stream is not None else torch.cuda.current_stream()
    return c_void_p(s.cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 status word that kernels with bounded waits write on timeout."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _status.get(key)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = st
        from .core.runtime_config import RuntimeConfig
        if RuntimeConfig.global_().kernel_checks:
            enable_kernel_checks(True, key)
    return st


def enable_kernel_checks(on: bool = True, device: int | None = None) -> None:
    """Switches the device-side index checks on or off: kernels that index memory with values read from tensors (token
    ids, class targets, expert slots, graph edges) then record code 108 in the status word when an index is out of range
    (they skip or clamp such an index either way). Default from ``TORSH_KERNEL_CHECKS``; the reference's counterpart is
    its debug-only validation layer (``crates/torsh-core/src/debug_validation.rs``)."""
    key = torch.cuda.current_device() if device is None else device
    lib = cuda()
    lib.tb_set_kernel_checks.restype = ctypes.c_int
    lib.tb_set_kernel_checks.argtypes = [ctypes.c_void_p]
    with torch.cuda.device(key):
        stream_ptr()
        word = status_word(key).data_ptr() if on else None
        check(lib.tb_set_kernel_checks(word), "tb_set_kernel_checks")


_STATUS_NAMES = {
    101: "MMA warp waited for a TMA stage that never landed",
    102: "TMA producer waited for a stage that was never released",
    103: "epilogue waited for an accumulator that never completed",
    104: "MMA warp waited for an accumulator that was never drained",
    105: "a flag owned by a peer GPU never arrived",
    106: "a device-side wait ran out",
    107: "bad kernel argument detected on the device",
    108: "an index read from a tensor was outside its range (device-side check)",
}


def check_status(device=None, reset: bool = True) -> None:
    """Synchronise and raise :class:`KernelTimeout` if any kernel recorded an error."""
    st = status_word(device)
    code = int(st[0].item())
    if code != 0:
        if reset:
            st.zero_()
            try:   # a kernel that gave up may have left its tile-scheduler counters non-zero
                f = cuda().tb_gemm_reset_scheduler
                f.restype, f.argtypes = ctypes.c_int, [ctypes.c_void_p]
                f(stream_ptr())
            except Exception:
                pass
        exc = KernelCheckFailed if code in (107, 108) else KernelTimeout
        raise exc(f"device status {code}: {_STATUS_NAMES.get(code, 'unknown')}")
