"""Autocast policy table: thread-local, per device kind.  Each op class maps to one cast policy:
``Lower`` (run in the autocast dtype on tensor cores), ``Fp32``, ``Promote`` (widest input) or ``Keep``.
Parity: include/nexus/amp/autocast.hpp:37-150 of the reference."""
from __future__ import annotations

import enum
import threading

from ..core.device import DeviceKind
from ..core.dtype import DType, TensorError, promote


class OpClass(enum.IntEnum):
    Matmul = 0
    Linear = 1
    Bmm = 2
    Conv = 3
    Attention = 4
    Softmax = 5
    LogSoftmax = 6
    CrossEntropy = 7
    LayerNorm = 8
    RmsNorm = 9
    Exp = 10
    Log = 11
    Pow = 12
    Sum = 13
    Mean = 14
    Norm = 15
    Add = 16
    Cat = 17
    Where = 18
    Reshape = 19
    Embedding = 20
    Dropout = 21


class CastPolicy(enum.IntEnum):
    Lower = 0
    Fp32 = 1
    Promote = 2
    Keep = 3


_LOWER = {OpClass.Matmul, OpClass.Linear, OpClass.Bmm, OpClass.Conv, OpClass.Attention}
_FP32 = {OpClass.Softmax, OpClass.LogSoftmax, OpClass.CrossEntropy, OpClass.LayerNorm, OpClass.RmsNorm, OpClass.Exp,
         OpClass.Log, OpClass.Pow, OpClass.Sum, OpClass.Mean, OpClass.Norm}
_PROMOTE = {OpClass.Add, OpClass.Cat, OpClass.Where}


def policy_for(op: OpClass) -> CastPolicy:
    if op in _LOWER:
        return CastPolicy.Lower
    if op in _FP32:
        return CastPolicy.Fp32
    if op in _PROMOTE:
        return CastPolicy.Promote
    return CastPolicy.Keep


_tls = threading.local()


def _states():
    if not hasattr(_tls, "states"):
        _tls.states = {k: (False, DType.BF16) for k in DeviceKind}
    return _tls.states


def autocast_state(kind: DeviceKind = DeviceKind.Cuda):
    return _states()[kind]


class AutocastGuard:
    def __init__(self, kind: DeviceKind = DeviceKind.Cuda, dtype: DType = DType.BF16, enabled: bool = True):
        if enabled and dtype not in (DType.BF16, DType.F16):
            raise TensorError("the autocast dtype must be BF16 or F16")
        self.kind, self.new = kind, (enabled, dtype)

    def __enter__(self):
        self.prev = _states()[self.kind]
        _states()[self.kind] = self.new
        return self

    def __exit__(self, *a):
        _states()[self.kind] = self.prev
        return False


def cast_dtype(op: OpClass, inputs, kind: DeviceKind = DeviceKind.Cuda) -> DType:
    """dtype the op runs in, given its input dtypes and the thread's autocast state."""
    enabled, low = _states()[kind]
    widest = inputs[0]
    for d in inputs[1:]:
        widest = promote(widest, d)
    if not enabled:
        return widest
    pol = policy_for(op)
    if pol == CastPolicy.Lower:
        return low if widest in (DType.F32, DType.BF16, DType.F16) else widest
    if pol == CastPolicy.Fp32:
        return DType.F32 if widest in (DType.BF16, DType.F16, DType.F32) else widest
    if pol == CastPolicy.Promote:
        return widest
    return inputs[0]
