"""Tensor files: TRSH binary (``.trsh`` / ``.bin``), JSON, NumPy ``.npy``.

The TRSH codec is native (``csrc/host/trsh_codec.cpp``): header, bincode metadata, CRC-32 and zstd.
Format source: ``crates/torsh-tensor/src/serialize/binary.rs`` and ``serialize/common.rs:315-383``;
extension mapping as in ``serialize/core.rs:408-433``.
"""
from __future__ import annotations

import ctypes
import json
import time
from pathlib import Path

import numpy as np
import torch

from .. import _native as nv
from ..core.dtype import DType, from_torch_dtype, to_torch_dtype
from ..core.error import TorshError

TORSH_VERSION = "0.1.3"
_RUST_TO_DTYPE = {"f32": torch.float32, "f64": torch.float64, "i8": torch.int8, "i16": torch.int16, "i32": torch.int32,
                  "i64": torch.int64, "u8": torch.uint8, "bool": torch.bool, "half::binary16::f16": torch.float16,
                  "half::bfloat::bf16": torch.bfloat16, "f16": torch.float16, "bf16": torch.bfloat16,
                  "u32": torch.uint32, "u64": torch.uint64}
_cfg = False


def _lib():
    global _cfg
    lib = nv.host()
    if not _cfg:
        lib.tsh_last_error.restype = ctypes.c_char_p
        lib.tsh_crc32.restype = ctypes.c_uint32
        lib.tsh_crc32.argtypes = [ctypes.c_void_p, ctypes.c_uint64]
        lib.tsh_free.argtypes = [ctypes.c_void_p]
        lib.tsh_trsh_encode.restype = ctypes.c_int
        lib.tsh_trsh_encode.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                        ctypes.c_int, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_uint64,
                                        ctypes.POINTER(ctypes.c_char_p), ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64,
                                        ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64)]
        lib.tsh_trsh_decode.restype = ctypes.c_int
        lib.tsh_trsh_decode.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64)]
        _cfg = True
    return lib


def crc32(data: bytes) -> int:
    """CRC-32 (poly 0xEDB88320, init 0xFFFFFFFF, final NOT) as used by the TRSH header."""
    return _lib().tsh_crc32(data, len(data))


def encode_trsh(t: torch.Tensor, compression_level: int = 0, metadata: dict | None = None,
                timestamp: int | None = None) -> bytes:
    lib = _lib()
    src = t.detach().cpu().contiguous()
    dt = from_torch_dtype(src.dtype)
    flat = src.reshape(-1)   # a zero-dim tensor cannot be re-viewed as bytes
    raw = flat.view(torch.uint8).numpy().tobytes() if src.dtype != torch.bool else flat.to(torch.uint8).numpy().tobytes()
    dims = (ctypes.c_int64 * max(src.dim(), 1))(*src.shape)
    kv = []
    for k, v in sorted((metadata or {}).items()):
        kv += [str(k).encode(), str(v).encode()]
    arr = (ctypes.c_char_p * max(len(kv), 1))(*kv)
    dev_kind, dev_idx = (1, t.device.index or 0) if t.is_cuda else (0, 0)
    out, n = ctypes.c_void_p(), ctypes.c_uint64()
    rc = lib.tsh_trsh_encode(dims, src.dim(), dev_kind, dev_idx, int(t.requires_grad), dt.rust_name.encode(),
                             TORSH_VERSION.encode(), int(time.time()) if timestamp is None else timestamp, arr,
                             len(kv) // 2, raw, len(raw), compression_level, ctypes.byref(out), ctypes.byref(n))
    if rc != 0:
        raise TorshError.serialization(lib.tsh_last_error().decode())
    try:
        return ctypes.string_at(out.value, n.value)
    finally:
        lib.tsh_free(out)


def decode_trsh(buf: bytes) -> tuple[torch.Tensor, dict]:
    lib = _lib()
    mj, data, n = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_uint64()
    rc = lib.tsh_trsh_decode(buf, len(buf), ctypes.byref(mj), ctypes.byref(data), ctypes.byref(n))
    if rc != 0:
        raise TorshError.serialization(lib.tsh_last_error().decode())
    try:
        meta = json.loads(ctypes.string_at(mj.value).decode())
        raw = ctypes.string_at(data.value, n.value)
    finally:
        lib.tsh_free(mj)
        lib.tsh_free(data)
    dtype = _RUST_TO_DTYPE.get(meta["dtype_name"])
    if dtype is None:
        raise TorshError.serialization(f"unknown element type {meta['dtype_name']!r}")
    if dtype == torch.bool:
        t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(torch.bool)
    else:
        t = torch.frombuffer(bytearray(raw), dtype=dtype)
    t = t.reshape(meta["shape"]).clone()
    t.requires_grad_(bool(meta["requires_grad"]) and t.is_floating_point())
    return t, meta


def _format_of(path: Path) -> str:
    ext = path.suffix.lower()
    return {".trsh": "binary", ".bin": "binary", ".torsh": "binary", ".json": "json", ".npy": "numpy", ".parquet": "parquet",
            ".arrow": "arrow", ".feather": "arrow", ".h5": "hdf5", ".hdf5": "hdf5"}.get(ext, "binary")


def save_tensor(t: torch.Tensor, path, compression_level: int = 0, metadata: dict | None = None) -> None:
    """``Tensor::save(path, opts)``: the format follows the file extension."""
    path = Path(path)
    fmt = _format_of(path)
    if fmt in ("parquet", "arrow", "hdf5"):
        from . import data_science as ds
        {"parquet": ds.save_parquet, "arrow": ds.save_arrow, "hdf5": ds.save_hdf5}[fmt]({"tensor": t}, str(path))
    elif fmt == "binary":
        path.write_bytes(encode_trsh(t, compression_level, metadata))
    elif fmt == "json":
        src = t.detach().cpu()
        doc = {"metadata": {"shape": list(src.shape), "device": "cpu", "requires_grad": bool(t.requires_grad),
                            "dtype_name": from_torch_dtype(src.dtype).rust_name, "version": TORSH_VERSION,
                            "timestamp": int(time.time()), "custom_metadata": metadata or {}, "format": "Json",
                            "data_size": src.numel() * src.element_size(), "compressed": False, "checksum": None},
               "data": src.reshape(-1).tolist()}
        path.write_text(json.dumps(doc, indent=2 if compression_level == 0 else None))
    else:
        np.save(path, t.detach().cpu().float().numpy() if t.dtype == torch.bfloat16 else t.detach().cpu().numpy())


def load_tensor(path) -> torch.Tensor:
    path = Path(path)
    fmt = _format_of(path)
    if fmt in ("parquet", "arrow", "hdf5"):
        from . import data_science as ds
        return {"parquet": ds.load_parquet, "arrow": ds.load_arrow, "hdf5": ds.load_hdf5}[fmt](str(path))["tensor"]
    if fmt == "binary":
        return decode_trsh(path.read_bytes())[0]
    if fmt == "json":
        doc = json.loads(path.read_text())
        m = doc["metadata"]
        t = torch.tensor(doc["data"], dtype=_RUST_TO_DTYPE.get(m["dtype_name"], torch.float32)).reshape(m["shape"])
        return t.requires_grad_(bool(m.get("requires_grad")) and t.is_floating_point())
    return torch.from_numpy(np.load(path))
