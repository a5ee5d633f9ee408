"""DLPack exchange (zero-copy) for FP32 tensors on CPU, CUDA and pinned host memory.
Parity: include/nexus/interop/dlpack.hpp of the reference (DLPack v0.8, F32 only)."""
from __future__ import annotations

import torch
from torch.utils import dlpack as _dl

K_CPU, K_CUDA, K_CUDA_HOST = 1, 2, 3


def device_type(t: torch.Tensor) -> int:
    if t.is_cuda:
        return K_CUDA
    return K_CUDA_HOST if t.is_pinned() else K_CPU


def to_dlpack(t: torch.Tensor):
    if t.dtype != torch.float32:
        raise TypeError("DLPack export supports FP32 tensors")
    return _dl.to_dlpack(t)


def from_dlpack(capsule_or_obj) -> torch.Tensor:
    t = _dl.from_dlpack(capsule_or_obj)
    if t.dtype != torch.float32:
        raise TypeError("DLPack import supports FP32 tensors")
    return t
