"""Storage / Tensor with explicit strides over shared byte storage, and the flat op dispatcher.

``Tensor`` = storage + dtype + shape + int64 strides + offset.  Views (`view_as`, `reshape`, `narrow`,
`slice`, `transpose`, `permute`, `expand`, `squeeze`, `unsqueeze`, `select`, `shallow`) share storage and
its version counter; ``copy()`` (the copy constructor of the reference) is a deep copy.  The dispatcher
is a flat table ``(Op, DType, space) -> function``; a missing combination raises, it never falls back.
Storage is a torch tensor of bytes so that host, pinned-host and device memory behave alike.
Parity: include/nexus/core/tensor.hpp:43-212, include/nexus/core/tensor_ops.hpp:33-121 of the reference."""
from __future__ import annotations

import enum
import math
from typing import Callable, Dict, Optional, Sequence, Tuple

import torch

from .device import DeviceRef, MemorySpace, Shape
from .dtype import DType, TensorError, from_torch, is_float8, promote, size_of, to_torch


class Storage:
    def __init__(self, nbytes: int, space: MemorySpace = MemorySpace.Host, device: DeviceRef = DeviceRef.cpu()):
        self.space, self.device, self.version = space, device, 0
        dev = device.torch_device() if space == MemorySpace.Device else "cpu"
        self.data = torch.zeros(max(int(nbytes), 0), dtype=torch.uint8, device=dev)
        if space == MemorySpace.PinnedHost and torch.cuda.is_available():
            self.data = self.data.pin_memory()

    @staticmethod
    def wrap(t: torch.Tensor) -> "Storage":
        s = Storage.__new__(Storage)
        s.data = t.contiguous().view(-1).view(torch.uint8)
        s.version = 0
        s.space = MemorySpace.Device if t.is_cuda else (MemorySpace.PinnedHost if t.is_pinned() else MemorySpace.Host)
        s.device = DeviceRef.cuda(t.device.index or 0) if t.is_cuda else DeviceRef.cpu()
        return s

    def nbytes(self) -> int:
        return self.data.numel()

    def bump(self) -> None:
        self.version += 1


class Tensor:
    def __init__(self, shape: Sequence[int] = (), dtype: DType = DType.F32, space: MemorySpace = MemorySpace.Host,
                 device: DeviceRef = DeviceRef.cpu(), *, _storage=None, _strides=None, _offset=0):
        self.shape = shape if isinstance(shape, Shape) else Shape(shape)
        self.dtype = DType(dtype)
        self.strides: Tuple[int, ...] = tuple(_strides) if _strides is not None else self.shape.contiguous_strides()
        self.offset = int(_offset)
        self.storage = _storage if _storage is not None else Storage(self.shape.numel() * size_of(dtype), space, device)

    # ---------------------------------------------------------------- construction / conversion
    @staticmethod
    def from_torch(t: torch.Tensor) -> "Tensor":
        st = Storage.wrap(t)
        return Tensor(t.shape, from_torch(t.dtype), _storage=st)

    def torch(self) -> torch.Tensor:
        """Zero-copy strided torch view of this tensor."""
        base = self.storage.data.view(to_torch(self.dtype))
        return torch.as_strided(base, self.shape.dims, self.strides, self.offset)

    def numel(self) -> int:
        return self.shape.numel()

    def space(self) -> MemorySpace:
        return self.storage.space

    def device(self) -> DeviceRef:
        return self.storage.device

    def version(self) -> int:
        return self.storage.version

    def is_contiguous(self) -> bool:
        return self.strides == self.shape.contiguous_strides()

    def _view(self, shape, strides, offset=None) -> "Tensor":
        return Tensor(shape, self.dtype, _storage=self.storage, _strides=strides,
                      _offset=self.offset if offset is None else offset)

    # ---------------------------------------------------------------- zero-copy views
    def shallow(self) -> "Tensor":
        return self._view(self.shape.dims, self.strides)

    def view_as(self, shape: Sequence[int]) -> "Tensor":
        return self.reshape(shape)

    def reshape(self, shape: Sequence[int]) -> "Tensor":
        dims = list(shape)
        if dims.count(-1) == 1:
            known = math.prod(d for d in dims if d != -1)
            dims[dims.index(-1)] = self.numel() // max(known, 1)
        if math.prod(dims) != self.numel():
            raise TensorError(f"reshape: {self.shape} -> {dims} changes the element count")
        if not self.is_contiguous():
            raise TensorError("reshape of a non-contiguous tensor needs contiguous() first")
        return self._view(dims, Shape(dims).contiguous_strides())

    def narrow(self, dim: int, start: int, length: int) -> "Tensor":
        if start < 0 or length < 0 or start + length > self.shape[dim]:
            raise TensorError("narrow: range outside the dimension")
        dims = list(self.shape.dims)
        dims[dim] = length
        return self._view(dims, self.strides, self.offset + start * self.strides[dim])

    def slice(self, dim: int, start: int, stop: int, step: int = 1) -> "Tensor":
        if step <= 0:
            raise TensorError("slice: step must be positive")
        start, stop = max(0, start), min(stop, self.shape[dim])
        dims, st = list(self.shape.dims), list(self.strides)
        dims[dim] = max(0, -(-(stop - start) // step))
        st[dim] *= step
        return self._view(dims, st, self.offset + start * self.strides[dim])

    def transpose(self, a: int, b: int) -> "Tensor":
        dims, st = list(self.shape.dims), list(self.strides)
        dims[a], dims[b], st[a], st[b] = dims[b], dims[a], st[b], st[a]
        return self._view(dims, st)

    def permute(self, order: Sequence[int]) -> "Tensor":
        if sorted(order) != list(range(self.shape.rank())):
            raise TensorError("permute: not a permutation")
        return self._view([self.shape[i] for i in order], [self.strides[i] for i in order])

    def expand(self, shape: Sequence[int]) -> "Tensor":
        if len(shape) != self.shape.rank():
            raise TensorError("expand: rank mismatch")
        st = list(self.strides)
        for i, (have, want) in enumerate(zip(self.shape.dims, shape)):
            if have != want:
                if have != 1:
                    raise TensorError("expand: only size-1 dimensions expand")
                st[i] = 0
        return self._view(shape, st)

    def squeeze(self, dim: int) -> "Tensor":
        if self.shape[dim] != 1:
            raise TensorError("squeeze: dimension is not 1")
        dims, st = list(self.shape.dims), list(self.strides)
        del dims[dim], st[dim]
        return self._view(dims, st)

    def unsqueeze(self, dim: int) -> "Tensor":
        dims, st = list(self.shape.dims), list(self.strides)
        dims.insert(dim, 1)
        st.insert(dim, st[dim] * self.shape[dim] if dim < len(st) else 1)
        return self._view(dims, st)

    def select(self, dim: int, index: int) -> "Tensor":
        return self.narrow(dim, index, 1).squeeze(dim)

    # ---------------------------------------------------------------- copies
    def copy(self) -> "Tensor":
        """Deep copy (what the copy constructor of the reference does)."""
        return Tensor.from_torch(self.torch().clone())

    def contiguous(self) -> "Tensor":
        return self if self.is_contiguous() and self.offset == 0 else Tensor.from_torch(self.torch().contiguous())

    def to(self, target) -> "Tensor":
        if isinstance(target, DType):
            if target == self.dtype:
                return self
            return Tensor.from_torch(self.torch().to(to_torch(target)))
        if isinstance(target, MemorySpace):
            t = self.torch()
            if target == MemorySpace.Device:
                return Tensor.from_torch(t.cuda())
            t = t.cpu()
            return Tensor.from_torch(t.pin_memory() if target == MemorySpace.PinnedHost and torch.cuda.is_available() else t)
        raise TensorError("to(): expected a DType or a MemorySpace")

    def copy_from(self, src: "Tensor") -> "Tensor":
        if src.shape != self.shape:
            raise TensorError("copy_from: shape mismatch")
        self.torch().copy_(src.torch())
        self.storage.bump()
        return self

    def fill(self, value) -> "Tensor":
        dispatch(Op.Fill, self.dtype, self.space())(self, value)
        return self


# -------------------------------------------------------------------------------------------- dispatcher
class Op(enum.IntEnum):
    Copy = 0
    Fill = 1
    Add = 2
    Mul = 3
    Matmul = 4
    Sum = 5
    Sub = 6
    Div = 7
    Unary = 8
    UnaryGrad = 9
    RowSoftmax = 10
    RowSoftmaxGrad = 11
    CrossEntropy = 12
    CrossEntropyGrad = 13
    ReduceRows = 14
    GatherRows = 15
    EmbeddingGrad = 16
    SqNorm = 17
    AdamW = 18


UNARY_FNS = ("relu", "gelu", "silu", "sigmoid", "tanh", "exp", "log", "neg", "sqrt", "abs", "square")
_TABLE: Dict[Tuple[Op, DType, int], Callable] = {}


def register(op: Op, dtype: DType, space: MemorySpace, fn: Callable) -> None:
    _TABLE[(op, DType(dtype), 0 if space != MemorySpace.Device else 1)] = fn


def dispatch(op: Op, dtype: DType, space: MemorySpace) -> Callable:
    fn = _TABLE.get((op, DType(dtype), 0 if space != MemorySpace.Device else 1))
    if fn is None:
        where = "device" if space == MemorySpace.Device else "host"
        raise TensorError(f"no kernel registered for {op.name} on {DType(dtype).name} ({where})")
    return fn


def _binary(fn):
    def run(a: Tensor, b: Tensor) -> Tensor:
        out_dt = promote(a.dtype, b.dtype)
        return Tensor.from_torch(fn(a.torch().to(to_torch(out_dt)), b.torch().to(to_torch(out_dt))))
    return run


_UNARY = {"relu": torch.relu, "gelu": lambda x: torch.nn.functional.gelu(x), "silu": torch.nn.functional.silu,
          "sigmoid": torch.sigmoid, "tanh": torch.tanh, "exp": torch.exp, "log": torch.log, "neg": torch.neg,
          "sqrt": torch.sqrt, "abs": torch.abs, "square": torch.square}


def _unary(x: Tensor, fn: str) -> Tensor:
    if fn not in _UNARY:
        raise TensorError(f"unknown unary function {fn!r}")
    return Tensor.from_torch(_UNARY[fn](x.torch()))


def _unary_grad(x: Tensor, grad: Tensor, fn: str) -> Tensor:
    xt = x.torch().detach().float().requires_grad_(True)
    _UNARY[fn](xt).backward(grad.torch().float())
    return Tensor.from_torch(xt.grad.to(to_torch(x.dtype)))


def _adamw(p: Tensor, g: Tensor, m: Tensor, v: Tensor, *, lr, beta1, beta2, eps, weight_decay, step, clip=1.0):
    pt, gt, mt, vt = p.torch(), g.torch().float() * clip, m.torch(), v.torch()
    pf = pt.float()
    pf.mul_(1 - lr * weight_decay)
    mt.mul_(beta1).add_(gt, alpha=1 - beta1)
    vt.mul_(beta2).addcmul_(gt, gt, value=1 - beta2)
    i1, i2 = 1.0 / (1 - beta1 ** step), 1.0 / (1 - beta2 ** step)
    pf.sub_(lr * (mt * i1) / ((vt * i2).sqrt() + eps))
    pt.copy_(pf)
    p.storage.bump()


def _register_defaults() -> None:
    floats = (DType.F32, DType.F64, DType.BF16, DType.F16)
    ints = (DType.I32, DType.I64, DType.I8, DType.U8, DType.Bool)
    for space in (MemorySpace.Host, MemorySpace.Device):
        for dt in floats + ints + (DType.F8E4M3, DType.F8E5M2):
            register(Op.Copy, dt, space, lambda dst, src: dst.copy_from(src))
            if not is_float8(dt):
                register(Op.Fill, dt, space, lambda t, v: (t.torch().fill_(v), t.storage.bump()))
        for dt in floats + (DType.I32, DType.I64):
            register(Op.Add, dt, space, _binary(torch.add))
            register(Op.Sub, dt, space, _binary(torch.sub))
            register(Op.Mul, dt, space, _binary(torch.mul))
            register(Op.Sum, dt, space, lambda x, dim=None: Tensor.from_torch(
                x.torch().sum() if dim is None else x.torch().sum(dim)))
        for dt in floats:
            register(Op.Div, dt, space, _binary(torch.div))
            register(Op.Matmul, dt, space, _binary(torch.matmul))
            register(Op.Unary, dt, space, _unary)
            register(Op.UnaryGrad, dt, space, _unary_grad)
            register(Op.RowSoftmax, dt, space, lambda x: Tensor.from_torch(torch.softmax(x.torch().float(), -1).to(x.torch().dtype)))
            register(Op.RowSoftmaxGrad, dt, space, lambda y, dy: Tensor.from_torch(
                (y.torch().float() * (dy.torch().float() - (y.torch().float() * dy.torch().float()).sum(-1, keepdim=True))).to(y.torch().dtype)))
            register(Op.CrossEntropy, dt, space, lambda lg, tgt: Tensor.from_torch(
                torch.nn.functional.cross_entropy(lg.torch().float(), tgt.torch().long(), reduction="none")))
            register(Op.CrossEntropyGrad, dt, space, lambda lg, tgt, scale=1.0: Tensor.from_torch(
                ((torch.softmax(lg.torch().float(), -1) - torch.nn.functional.one_hot(tgt.torch().long(), lg.shape[-1])) * scale).to(lg.torch().dtype)))
            register(Op.ReduceRows, dt, space, lambda x: Tensor.from_torch(x.torch().float().sum(0).to(x.torch().dtype)))
            register(Op.GatherRows, dt, space, lambda x, idx: Tensor.from_torch(x.torch()[idx.torch().long()]))
            register(Op.EmbeddingGrad, dt, space, lambda dy, idx, rows: Tensor.from_torch(
                torch.zeros(rows, dy.shape[-1], dtype=torch.float32, device=dy.torch().device).index_add_(
                    0, idx.torch().long().view(-1), dy.torch().float().view(-1, dy.shape[-1]))))
            register(Op.SqNorm, dt, space, lambda x: float((x.torch().double() ** 2).sum()))
            register(Op.AdamW, dt, space, _adamw)


_register_defaults()


def add(a: Tensor, b: Tensor) -> Tensor:
    return dispatch(Op.Add, promote(a.dtype, b.dtype), a.space())(a, b)


def mul(a: Tensor, b: Tensor) -> Tensor:
    return dispatch(Op.Mul, promote(a.dtype, b.dtype), a.space())(a, b)


def matmul(a: Tensor, b: Tensor) -> Tensor:
    return dispatch(Op.Matmul, promote(a.dtype, b.dtype), a.space())(a, b)


def unary(x: Tensor, fn: str) -> Tensor:
    return dispatch(Op.Unary, x.dtype, x.space())(x, fn)
