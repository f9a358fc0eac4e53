"""``DType``: the 17 element types of the reference (``crates/torsh-core/src/dtype/core.rs:16-51``)."""
from __future__ import annotations

from enum import Enum

import torch


class DType(Enum):
    U8 = "u8"; I8 = "i8"; I16 = "i16"; I32 = "i32"; I64 = "i64"; U16 = "u16"; U32 = "u32"; U64 = "u64"
    F16 = "f16"; BF16 = "bf16"; F32 = "f32"; F64 = "f64"; BOOL = "bool"; C64 = "c64"; C128 = "c128"
    QINT8 = "qint8"; QUINT8 = "quint8"; QINT32 = "qint32"

    @property
    def size_bytes(self) -> int:
        return _SIZES[self]

    def is_float(self) -> bool:
        return self in (DType.F16, DType.BF16, DType.F32, DType.F64)

    def is_complex(self) -> bool:
        return self in (DType.C64, DType.C128)

    def is_int(self) -> bool:
        return self in (DType.U8, DType.I8, DType.I16, DType.I32, DType.I64, DType.U16, DType.U32, DType.U64)

    def is_quantized(self) -> bool:
        return self in (DType.QINT8, DType.QUINT8, DType.QINT32)

    @property
    def rust_name(self) -> str:
        """Element type name as written into TRSH metadata (Rust ``type_name``)."""
        return _RUST.get(self, self.value)


_SIZES = {DType.U8: 1, DType.I8: 1, DType.I16: 2, DType.I32: 4, DType.I64: 8, DType.U16: 2, DType.U32: 4, DType.U64: 8, DType.F16: 2,
          DType.BF16: 2, DType.F32: 4, DType.F64: 8, DType.BOOL: 1, DType.C64: 8, DType.C128: 16, DType.QINT8: 1,
          DType.QUINT8: 1, DType.QINT32: 4}
_RUST = {DType.F16: "half::binary16::f16", DType.BF16: "half::bfloat::bf16", DType.C64: "num_complex::Complex<f32>",
         DType.C128: "num_complex::Complex<f64>"}
_TO_TORCH = {DType.U8: torch.uint8, DType.I8: torch.int8, DType.I16: torch.int16, DType.I32: torch.int32,
             DType.I64: torch.int64, DType.U16: torch.uint16, DType.U32: torch.uint32, DType.U64: torch.uint64, DType.F16: torch.float16,
             DType.BF16: torch.bfloat16, DType.F32: torch.float32, DType.F64: torch.float64, DType.BOOL: torch.bool,
             DType.C64: torch.complex64, DType.C128: torch.complex128, DType.QINT8: torch.qint8,
             DType.QUINT8: torch.quint8, DType.QINT32: torch.qint32}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def to_torch_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        return d
    if isinstance(d, str):
        d = DType(d)
    return _TO_TORCH[d]


def from_torch_dtype(d: torch.dtype) -> DType:
    return _FROM_TORCH[d]
