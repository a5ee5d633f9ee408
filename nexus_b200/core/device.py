"""Device references, memory spaces, shapes, execution policy and the global seed.
Parity: include/nexus/core/device.hpp:29-197, shape.hpp:24-125, config.hpp:15-47 of the reference."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Iterable, Tuple

from .dtype import TensorError


class DeviceKind(enum.IntEnum):
    Cpu = 0
    Cuda = 1
    Rocm = 2
    Tpu = 3
    Npu = 4
    Vulkan = 5
    DirectMl = 6
    Metal = 7


class MemorySpace(enum.IntEnum):
    Host = 0
    PinnedHost = 1
    Device = 2


_KIND_NAMES = {"cpu": DeviceKind.Cpu, "cuda": DeviceKind.Cuda, "rocm": DeviceKind.Rocm, "tpu": DeviceKind.Tpu,
               "npu": DeviceKind.Npu, "vulkan": DeviceKind.Vulkan, "directml": DeviceKind.DirectMl,
               "metal": DeviceKind.Metal}


@dataclass(frozen=True)
class DeviceRef:
    kind: DeviceKind = DeviceKind.Cpu
    index: int = -1

    @staticmethod
    def cpu() -> "DeviceRef":
        return DeviceRef(DeviceKind.Cpu, -1)

    @staticmethod
    def cuda(i: int = 0) -> "DeviceRef":
        return DeviceRef(DeviceKind.Cuda, i)

    @staticmethod
    def hybrid() -> "DeviceRef":
        return DeviceRef(DeviceKind.Cpu, -2)

    def is_hybrid(self) -> bool:
        return self.kind == DeviceKind.Cpu and self.index == -2

    def is_cpu(self) -> bool:
        return self.kind == DeviceKind.Cpu and not self.is_hybrid()

    def is_unified(self) -> bool:
        return self.kind in (DeviceKind.Cpu, DeviceKind.Metal)

    @staticmethod
    def parse(spec: str) -> "DeviceRef":
        s = spec.strip().lower()
        name, _, idx = s.partition(":")
        if name == "hybrid":
            if idx:
                raise TensorError("the hybrid device takes no index")
            return DeviceRef.hybrid()
        if name not in _KIND_NAMES:
            raise TensorError(f"unknown device {spec!r}")
        kind = _KIND_NAMES[name]
        if not idx:
            return DeviceRef(kind, -1 if kind == DeviceKind.Cpu else 0)
        if not idx.isdigit():
            raise TensorError(f"bad device index in {spec!r}")
        if kind == DeviceKind.Cpu:
            raise TensorError("the cpu device takes no index")
        return DeviceRef(kind, int(idx))

    def __str__(self) -> str:
        if self.is_hybrid():
            return "hybrid"
        name = [k for k, v in _KIND_NAMES.items() if v == self.kind][0]
        return name if self.kind == DeviceKind.Cpu else f"{name}:{self.index}"

    def torch_device(self) -> str:
        if self.kind == DeviceKind.Cuda:
            return f"cuda:{self.index}"
        if self.kind == DeviceKind.Cpu:
            return "cpu"
        raise TensorError(f"{self} has no tensor runtime in this build")


class Shape:
    """Rank <= 8, overflow-checked element count."""
    MAX_RANK = 8

    def __init__(self, dims: Iterable[int] = ()):
        self.dims: Tuple[int, ...] = tuple(int(d) for d in dims)
        if len(self.dims) > self.MAX_RANK:
            raise TensorError(f"rank {len(self.dims)} exceeds the maximum of {self.MAX_RANK}")
        if any(d < 0 for d in self.dims):
            raise TensorError("negative dimension")

    def rank(self) -> int:
        return len(self.dims)

    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
            if n > (1 << 63) - 1:
                raise TensorError("element count overflows 64 bits")
        return n

    def __getitem__(self, i):
        return self.dims[i]

    def __len__(self):
        return len(self.dims)

    def __eq__(self, other):
        return tuple(other.dims if isinstance(other, Shape) else other) == self.dims

    def __hash__(self):
        return hash(self.dims)

    def __repr__(self):
        return f"Shape{list(self.dims)}"

    def contiguous_strides(self) -> Tuple[int, ...]:
        s, out = 1, []
        for d in reversed(self.dims):
            out.append(s)
            s *= max(d, 1)
        return tuple(reversed(out))


@dataclass(frozen=True)
class ExecutionPolicy:
    device: DeviceRef = DeviceRef.cpu()
    gpus: Tuple[int, ...] = ()

    @staticmethod
    def cpu() -> "ExecutionPolicy":
        return ExecutionPolicy(DeviceRef.cpu())

    @staticmethod
    def cuda(i: int = 0) -> "ExecutionPolicy":
        return ExecutionPolicy(DeviceRef.cuda(i), (i,))

    @staticmethod
    def hybrid_cpu_multi_gpu(gpus: Iterable[int]) -> "ExecutionPolicy":
        return ExecutionPolicy(DeviceRef.hybrid(), tuple(gpus))


_GLOBAL_SEED = [0x5EED]


def global_seed() -> int:
    return _GLOBAL_SEED[0]


def set_global_seed(seed: int) -> None:
    import torch
    _GLOBAL_SEED[0] = int(seed)
    torch.manual_seed(int(seed))
