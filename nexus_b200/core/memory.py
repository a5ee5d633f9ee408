"""Memory gate: one registry for aligned host, pinned host and device allocations with counters,
synchronous / asynchronous byte copies (peer copies included), RAII streams, events and device
buffers, and host-memory registration (pinning in place).
Parity: include/nexus/core/memory.hpp:35-110, include/nexus/cuda/runtime.hpp of the reference."""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .device import DeviceRef, MemorySpace
from .dtype import TensorError


@dataclass
class AllocationCounters:
    allocations: Dict[str, int] = field(default_factory=lambda: {"host": 0, "pinned": 0, "device": 0})
    live_bytes: Dict[str, int] = field(default_factory=lambda: {"host": 0, "pinned": 0, "device": 0})
    peak_bytes: Dict[str, int] = field(default_factory=lambda: {"host": 0, "pinned": 0, "device": 0})
    copies: int = 0
    copied_bytes: int = 0


_KEY = {MemorySpace.Host: "host", MemorySpace.PinnedHost: "pinned", MemorySpace.Device: "device"}


class MemoryGate:
    def __init__(self):
        self._lock = threading.Lock()
        self._live: Dict[int, tuple] = {}
        self.counters = AllocationCounters()

    def alloc(self, nbytes: int, space: MemorySpace = MemorySpace.Host, device: DeviceRef = DeviceRef.cpu(),
              alignment: int = 64) -> torch.Tensor:
        """uint8 tensor of ``nbytes`` whose address is a multiple of ``alignment``."""
        if alignment & (alignment - 1):
            raise TensorError("alignment must be a power of two")
        if space == MemorySpace.Device:
            raw = torch.empty(nbytes + alignment, dtype=torch.uint8, device=device.torch_device())
        else:
            raw = torch.empty(nbytes + alignment, dtype=torch.uint8)
            if space == MemorySpace.PinnedHost:
                if not torch.cuda.is_available():
                    raise TensorError("pinned host memory needs a CUDA runtime")
                raw = raw.pin_memory()
        shift = (-raw.data_ptr()) % alignment
        buf = raw[shift: shift + nbytes]
        key = _KEY[space]
        with self._lock:
            self._live[buf.data_ptr()] = (raw, key, nbytes)
            c = self.counters
            c.allocations[key] += 1
            c.live_bytes[key] += nbytes
            c.peak_bytes[key] = max(c.peak_bytes[key], c.live_bytes[key])
        return buf

    def free(self, buf: torch.Tensor) -> None:
        with self._lock:
            rec = self._live.pop(buf.data_ptr(), None)
            if rec is None:
                raise TensorError("free of memory this gate did not allocate")
            self.counters.live_bytes[rec[1]] -= rec[2]

    def copy_bytes(self, dst: torch.Tensor, src: torch.Tensor, nbytes: Optional[int] = None, *, non_blocking=False,
                   stream: Optional["Stream"] = None) -> None:
        """dst[:n] = src[:n] across any pair of spaces / devices (peer copies go GPU to GPU directly)."""
        n = min(dst.numel(), src.numel()) if nbytes is None else nbytes
        if n > dst.numel() or n > src.numel():
            raise TensorError("copy_bytes: range exceeds a buffer")
        ctx = torch.cuda.stream(stream.raw) if stream is not None else _null()
        with ctx:
            dst.view(torch.uint8).view(-1)[:n].copy_(src.view(torch.uint8).view(-1)[:n], non_blocking=non_blocking)
        with self._lock:
            self.counters.copies += 1
            self.counters.copied_bytes += n

    def copy_bytes_async(self, dst, src, nbytes=None, stream=None) -> None:
        self.copy_bytes(dst, src, nbytes, non_blocking=True, stream=stream)

    def register_host_memory(self, t: torch.Tensor) -> bool:
        """Page-locks existing host memory in place (no copy).  False when there is no CUDA runtime."""
        if not torch.cuda.is_available() or t.is_cuda:
            return False
        rc = torch.cuda.cudart().cudaHostRegister(t.data_ptr(), t.numel() * t.element_size(), 0)
        return int(rc) == 0

    def unregister_host_memory(self, t: torch.Tensor) -> None:
        if torch.cuda.is_available() and not t.is_cuda:
            torch.cuda.cudart().cudaHostUnregister(t.data_ptr())


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_GATE = MemoryGate()


def gate() -> MemoryGate:
    return _GATE


# ------------------------------------------------------------------------------- runtime wrappers
class Stream:
    """Owning CUDA stream."""

    def __init__(self, device: Optional[int] = None, priority: int = 0):
        self.raw = torch.cuda.Stream(device=device, priority=priority)

    def synchronize(self) -> None:
        self.raw.synchronize()

    def wait_event(self, ev: "Event") -> None:
        self.raw.wait_event(ev.raw)

    def handle(self) -> int:
        return self.raw.cuda_stream

    def __enter__(self):
        self._ctx = torch.cuda.stream(self.raw)
        self._ctx.__enter__()
        return self

    def __exit__(self, *a):
        return self._ctx.__exit__(*a)


class Event:
    def __init__(self, timing: bool = False):
        self.raw = torch.cuda.Event(enable_timing=timing)

    def record(self, stream: Optional[Stream] = None) -> None:
        self.raw.record(stream.raw if stream is not None else None)

    def synchronize(self) -> None:
        self.raw.synchronize()

    def query(self) -> bool:
        return self.raw.query()

    def elapsed_ms(self, end: "Event") -> float:
        return self.raw.elapsed_time(end.raw)


class DeviceBuffer:
    """Owning device allocation of ``nbytes`` (released with the object)."""

    def __init__(self, nbytes: int, device: int = 0):
        self.tensor = gate().alloc(nbytes, MemorySpace.Device, DeviceRef.cuda(device), alignment=256)

    def ptr(self) -> int:
        return self.tensor.data_ptr()

    def nbytes(self) -> int:
        return self.tensor.numel()

    def __del__(self):
        try:
            gate().free(self.tensor)
        except Exception:
            pass


def current_device() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else -1


def cuda_check(rc: int, what: str = "CUDA call") -> None:
    if int(rc) != 0:
        raise RuntimeError(f"{what} failed with CUDA error {int(rc)}")
