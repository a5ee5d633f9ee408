"""Element types, torch-like promotion and FP8 / half host conversions.

Eleven dtypes; ``promote`` follows PyTorch except that U8 + I8 gives I32 (there is no I16) and FP8 never
promotes implicitly.  FP8 E4M3fn (max 448, no infinity) and E5M2 (max 57344) encode with
round-to-nearest-even and saturation.  ``Fp8DelayedScaling`` keeps an amax history and derives
``scale = fp8_max / max(history) / 2**margin``.
Parity: include/nexus/core/dtype.hpp:32-168, include/nexus/core/half.hpp of the reference."""
from __future__ import annotations

import enum
from collections import deque
from typing import Deque

import numpy as np
import torch


class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    BF16 = 2
    F64 = 3
    I32 = 4
    I64 = 5
    I8 = 6
    U8 = 7
    Bool = 8
    F8E4M3 = 9
    F8E5M2 = 10


ALL_DTYPES = tuple(DType)
_SIZE = {DType.F64: 8, DType.I64: 8, DType.F32: 4, DType.I32: 4, DType.F16: 2, DType.BF16: 2, DType.I8: 1,
         DType.U8: 1, DType.Bool: 1, DType.F8E4M3: 1, DType.F8E5M2: 1}
_NAMES = {DType.F32: "f32", DType.F16: "f16", DType.BF16: "bf16", DType.F64: "f64", DType.I32: "i32",
          DType.I64: "i64", DType.I8: "i8", DType.U8: "u8", DType.Bool: "bool", DType.F8E4M3: "f8e4m3",
          DType.F8E5M2: "f8e5m2"}
_TORCH = {DType.F32: torch.float32, DType.F16: torch.float16, DType.BF16: torch.bfloat16, DType.F64: torch.float64,
          DType.I32: torch.int32, DType.I64: torch.int64, DType.I8: torch.int8, DType.U8: torch.uint8,
          DType.Bool: torch.bool, DType.F8E4M3: torch.float8_e4m3fn, DType.F8E5M2: torch.float8_e5m2}
_FROM_TORCH = {v: k for k, v in _TORCH.items()}


class TensorError(RuntimeError):
    pass


def size_of(d: DType) -> int:
    return _SIZE[DType(d)]


def to_string(d: DType) -> str:
    return _NAMES[DType(d)]


def parse_dtype(name: str) -> DType:
    for k, v in _NAMES.items():
        if v == name.lower():
            return k
    raise TensorError(f"unknown dtype {name!r}")


def is_float8(d: DType) -> bool:
    return d in (DType.F8E4M3, DType.F8E5M2)


def is_floating(d: DType) -> bool:
    return d in (DType.F16, DType.BF16, DType.F32, DType.F64) or is_float8(d)


def is_integral(d: DType) -> bool:
    return d in (DType.U8, DType.I8, DType.I32, DType.I64)


def to_torch(d: DType) -> torch.dtype:
    return _TORCH[DType(d)]


def from_torch(t: torch.dtype) -> DType:
    return _FROM_TORCH[t]


def _core():
    from .. import _native
    return _native


def promote(a: DType, b: DType) -> DType:
    """Result dtype of a binary op: torch-like, except U8 + I8 -> I32 (PyTorch gives int16) and FP8 never promotes
    implicitly.  The table lives in the native host module (`csrc/host/lowp.cpp`)."""
    a, b = DType(a), DType(b)
    try:
        return DType(_core().dtype_promote(int(a), int(b)))
    except ValueError:
        raise TensorError(f"{to_string(a)} and {to_string(b)} do not promote implicitly; convert FP8 explicitly") from None


# ------------------------------------------------------------------------------------- host conversions
# Bit-level round-to-nearest-even conversions in the native host module; arrays of any shape.
def float_to_bf16_bits(x) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16); NaN stays NaN."""
    return _core().f32_to_bf16_bits(np.asarray(x, dtype=np.float32))


def bf16_bits_to_float(b) -> np.ndarray:
    return _core().bf16_bits_to_f32(np.asarray(b, dtype=np.uint16))


def float_to_half_bits(x) -> np.ndarray:
    return _core().f32_to_f16_bits(np.asarray(x, dtype=np.float32))


def half_bits_to_float(b) -> np.ndarray:
    return _core().f16_bits_to_f32(np.asarray(b, dtype=np.uint16))


FP8_MAX = {DType.F8E4M3: 448.0, DType.F8E5M2: 57344.0}


def fp8_decode(codes, fmt: DType) -> np.ndarray:
    """FP8 bit patterns -> float32.  E4M3fn: only S.1111.111 is NaN, no infinity; E5M2: IEEE-like."""
    return _core().fp8_bits_to_f32(np.asarray(codes, dtype=np.uint8), DType(fmt) == DType.F8E5M2)


def fp8_encode(x, fmt: DType) -> np.ndarray:
    """float32 -> FP8 bit patterns, RNE, saturating to +-max (NaN -> the format's NaN code)."""
    return _core().f32_to_fp8_bits(np.asarray(x, dtype=np.float32), DType(fmt) == DType.F8E5M2)


class Fp8DelayedScaling:
    """Delayed scaling recipe: the scale used at step t comes from the amax history of earlier steps."""

    def __init__(self, fmt: DType = DType.F8E4M3, history: int = 16, margin: int = 0):
        self.fmt, self.margin = DType(fmt), margin
        self.hist: Deque[float] = deque(maxlen=history)
        self.scale = 1.0

    def update(self, amax: float) -> float:
        """Records this step's amax; returns the scale to use from now on."""
        self.hist.append(float(amax))
        m = max(self.hist)
        if m > 0 and np.isfinite(m):
            self.scale = FP8_MAX[self.fmt] / m / (2.0 ** self.margin)
        return self.scale

    def scale_inv(self) -> float:
        return 1.0 / self.scale
