"""Runtime dtype table.

Mirrors the reference's ``DTypeId`` set and block-size arithmetic
(crates/incin-core/src/tensor/dtype.rs:83-101,131-194): plain scalar dtypes plus the block-quantised
``Q8_0`` (32 values share one f16 scale: 34 bytes per block).
"""
from __future__ import annotations

import enum

import torch

Q8_0_BLOCK = 32
Q8_0_BLOCK_BYTES = 34


class DTypeId(enum.Enum):
    U8 = "u8"
    U32 = "u32"
    I64 = "i64"
    BF16 = "bf16"
    F16 = "f16"
    F32 = "f32"
    F64 = "f64"
    Q8_0 = "q8_0"

    @property
    def is_float(self) -> bool:
        return self in (DTypeId.BF16, DTypeId.F16, DTypeId.F32, DTypeId.F64)

    @property
    def is_int(self) -> bool:
        return self in (DTypeId.U8, DTypeId.U32, DTypeId.I64)

    @property
    def is_quantized(self) -> bool:
        return self is DTypeId.Q8_0

    @property
    def safetensors_name(self) -> str:
        return {"u8": "U8", "u32": "U32", "i64": "I64", "bf16": "BF16", "f16": "F16", "f32": "F32",
                "f64": "F64"}[self.value]


_ELEM_BYTES = {DTypeId.U8: 1, DTypeId.U32: 4, DTypeId.I64: 8, DTypeId.BF16: 2, DTypeId.F16: 2, DTypeId.F32: 4,
               DTypeId.F64: 8}
_TO_TORCH = {DTypeId.U8: torch.uint8, DTypeId.U32: torch.uint32, DTypeId.I64: torch.int64, DTypeId.BF16: torch.bfloat16,
             DTypeId.F16: torch.float16, DTypeId.F32: torch.float32, DTypeId.F64: torch.float64}
_FROM_TORCH = {v: k for k, v in _TO_TORCH.items()}


def size_bytes(dtype: DTypeId, numel: int) -> int:
    """Storage bytes of ``numel`` logical elements; Q8_0 rounds up to whole 32-element blocks."""
    if numel < 0:
        raise ValueError("negative element count")
    if dtype is DTypeId.Q8_0:
        return (numel + Q8_0_BLOCK - 1) // Q8_0_BLOCK * Q8_0_BLOCK_BYTES
    return _ELEM_BYTES[dtype] * numel


def to_torch(dtype: DTypeId) -> torch.dtype:
    if dtype is DTypeId.Q8_0:
        raise TypeError("Q8_0 is a block format, not a torch scalar dtype (see incin_b200.ops.quant)")
    return _TO_TORCH[dtype]


def from_torch(dtype: torch.dtype) -> DTypeId:
    try:
        return _FROM_TORCH[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} has no incin DTypeId") from None
