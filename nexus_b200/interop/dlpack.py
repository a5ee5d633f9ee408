"""DLPack v0.8 exchange (zero copy) for FP32 tensors on CPU, CUDA and pinned host memory.

The capsules are made and read by the native host module (`csrc/host/dlpack.cpp`): export wraps the tensor's buffer and
holds the tensor until the consumer's deleter runs; import validates the capsule, marks it consumed and returns the
geometry plus a keeper that runs the producer's deleter when the imported view dies.  Any DLPack consumer (torch, numpy,
cupy, jax) can take an exported capsule, and any producer's capsule or `__dlpack__` object can be imported.
Parity: include/nexus/interop/dlpack.hpp of the reference (DLPack v0.8, F32 only)."""
from __future__ import annotations

import numpy as np
import torch

from .. import _native

K_CPU, K_CUDA, K_CUDA_HOST = 1, 2, 3


def _as_torch(t) -> torch.Tensor:
    if isinstance(t, torch.Tensor):
        return t
    if hasattr(t, "torch") and callable(t.torch):       # nexus_b200.core.Tensor
        return t.torch()
    raise TypeError(f"DLPack export takes a torch.Tensor or a framework Tensor, got {type(t).__name__}")


def device_type(t) -> int:
    t = _as_torch(t)
    if t.is_cuda:
        return K_CUDA
    return K_CUDA_HOST if t.is_pinned() else K_CPU


def to_dlpack(t):
    """A "dltensor" capsule that shares ``t``'s memory.  ``t`` stays alive until the consumer releases the capsule."""
    tt = _as_torch(t)
    if tt.dtype != torch.float32:
        raise TypeError("DLPack export supports FP32 tensors")
    if tt.requires_grad:
        tt = tt.detach()
    strides = [] if tt.is_contiguous() else list(tt.stride())
    return _native.dlpack_export(tt.data_ptr(), list(tt.shape), strides, 32, device_type(tt),
                                 tt.device.index or 0 if tt.is_cuda else 0, tt)


class _Span:
    """Flat FP32 window over imported memory, in the array-interface form for its device; owns the keeper."""

    def __init__(self, info):
        self.keeper = info["keeper"]
        desc = {"shape": (int(info["span"]),), "typestr": "<f4", "data": (int(info["ptr"]), False), "strides": None}
        if info["device_type"] == K_CUDA:
            self.__cuda_array_interface__ = {**desc, "version": 2}
        else:
            self.__array_interface__ = {**desc, "version": 3}


def from_dlpack(obj, as_tensor: bool = False):
    """Zero-copy import of a DLPack capsule, or of any object with ``__dlpack__``.  Returns a torch tensor that views
    the producer's memory (``as_tensor=True``: the framework's Tensor over it); the producer's deleter runs when the
    last view goes away."""
    capsule = obj.__dlpack__() if hasattr(obj, "__dlpack__") and not isinstance(obj, type) else obj
    info = _native.dlpack_import(capsule)
    shape, strides = list(info["shape"]), list(info["strides"])
    if info["span"] == 0:
        dev = torch.device("cuda", info["device_id"]) if info["device_type"] == K_CUDA else torch.device("cpu")
        info["keeper"].release()
        out = torch.empty(shape, dtype=torch.float32, device=dev)
    else:
        span = _Span(info)
        if info["device_type"] == K_CUDA:
            flat = torch.as_tensor(span, device=torch.device("cuda", info["device_id"]))
        else:
            flat = torch.from_numpy(np.asarray(span))
        out = torch.as_strided(flat, shape, strides)
    if as_tensor:
        from ..core.tensor import Tensor
        return Tensor.from_torch(out)
    return out
