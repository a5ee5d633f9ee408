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
_FLOAT_RANK = {DType.F16: 1, DType.BF16: 1, DType.F32: 2, DType.F64: 3}
_INT_RANK = {DType.U8: 1, DType.I8: 1, DType.I32: 2, DType.I64: 3}


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
    return d in _FLOAT_RANK or is_float8(d)


def is_integral(d: DType) -> bool:
    return d in _INT_RANK


def to_torch(d: DType) -> torch.dtype:
    return _TORCH[DType(d)]


def from_torch(t: torch.dtype) -> DType:
    return _FROM_TORCH[t]


def promote(a: DType, b: DType) -> DType:
    a, b = DType(a), DType(b)
    if a == b:
        return a
    if is_float8(a) or is_float8(b):
        raise TensorError(f"{to_string(a)} and {to_string(b)} do not promote implicitly; convert FP8 explicitly")
    if a == DType.Bool:
        return b
    if b == DType.Bool:
        return a
    fa, fb = a in _FLOAT_RANK, b in _FLOAT_RANK
    if fa != fb:
        return a if fa else b
    if fa:
        ra, rb = _FLOAT_RANK[a], _FLOAT_RANK[b]
        if ra == rb:
            return DType.F32            # F16 + BF16
        return a if ra > rb else b
    if {a, b} == {DType.U8, DType.I8}:
        return DType.I32                # documented deviation: PyTorch gives int16
    return a if _INT_RANK[a] >= _INT_RANK[b] else b


# ------------------------------------------------------------------------------------- host conversions
def float_to_bf16_bits(x) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16); NaN stays NaN."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)
    return np.where(nan, np.uint16(0x7FC0), r)


def bf16_bits_to_float(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def float_to_half_bits(x) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def half_bits_to_float(b) -> np.ndarray:
    return np.asarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


FP8_MAX = {DType.F8E4M3: 448.0, DType.F8E5M2: 57344.0}


def _fp8_table(fmt: DType) -> np.ndarray:
    """Decode table of all 256 bit patterns."""
    out = np.zeros(256, dtype=np.float32)
    e_bits, m_bits, bias = (4, 3, 7) if fmt == DType.F8E4M3 else (5, 2, 15)
    for code in range(256):
        s = -1.0 if code & 0x80 else 1.0
        e = (code >> m_bits) & ((1 << e_bits) - 1)
        m = code & ((1 << m_bits) - 1)
        if fmt == DType.F8E4M3:
            if e == 15 and m == 7:
                out[code] = np.nan           # E4M3fn: only S.1111.111 is NaN, no infinity
                continue
        elif e == 31:
            out[code] = s * np.inf if m == 0 else np.nan
            continue
        if e == 0:
            out[code] = s * m * 2.0 ** (1 - bias - m_bits)
        else:
            out[code] = s * (1 + m / (1 << m_bits)) * 2.0 ** (e - bias)
    return out


_FP8_DECODE = {DType.F8E4M3: _fp8_table(DType.F8E4M3), DType.F8E5M2: _fp8_table(DType.F8E5M2)}


def fp8_decode(codes, fmt: DType) -> np.ndarray:
    return _FP8_DECODE[DType(fmt)][np.asarray(codes, dtype=np.uint8)]


def fp8_encode(x, fmt: DType) -> np.ndarray:
    """float32 -> FP8 bit patterns, RNE, saturating to +-max (NaN -> NaN code)."""
    fmt = DType(fmt)
    x = np.asarray(x, dtype=np.float32)
    table = _FP8_DECODE[fmt]
    pos_codes = np.array([c for c in range(128) if np.isfinite(table[c])], dtype=np.uint8)
    vals = table[pos_codes]                     # ascending
    a = np.minimum(np.abs(x), FP8_MAX[fmt])
    hi = np.clip(np.searchsorted(vals, a, side="left"), 0, len(vals) - 1)
    lo = np.clip(hi - 1, 0, len(vals) - 1)
    dlo, dhi = np.abs(a - vals[lo]), np.abs(vals[hi] - a)
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((pos_codes[hi] & 1) == 0))   # ties -> even mantissa
    code = np.where(pick_hi, pos_codes[hi], pos_codes[lo]).astype(np.uint8)
    code = np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)
    nan_code = 0x7F if fmt == DType.F8E4M3 else 0x7E
    return np.where(np.isnan(x), np.uint8(nan_code), code)


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
