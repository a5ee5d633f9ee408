"""Host + device mirror of one FP32 tensor with an explicit state machine
(``Synced`` / ``HostAhead`` / ``DeviceAhead``), its own copy stream and event ordering against the
compute stream.  On a unified device (CPU) both sides are the same buffer and every sync is free.
Parity: include/nexus/core/mirrored_tensor.hpp, src/core/mirrored_tensor.cpp of the reference."""
from __future__ import annotations

import enum
from typing import Optional, Sequence

import torch

from .device import DeviceRef, Shape


class MirrorState(enum.IntEnum):
    Synced = 0
    HostAhead = 1
    DeviceAhead = 2


class MirroredTensor:
    def __init__(self, shape: Sequence[int], device: DeviceRef = DeviceRef.cuda(0), pinned: bool = True):
        self.shape = Shape(shape)
        self.device = device
        self.unified = device.is_unified()
        self.host = torch.zeros(self.shape.dims, dtype=torch.float32)
        self._pinned = False
        if not self.unified and pinned:
            self.pin_host()
        self._dev: Optional[torch.Tensor] = None
        self.state = MirrorState.Synced
        self._stream = None
        self._event = None
        self._pending = False
        self.device_stream = None
        self.bytes_to_device = 0
        self.bytes_to_host = 0

    @staticmethod
    def wrap_host(host: torch.Tensor, device: DeviceRef) -> "MirroredTensor":
        m = MirroredTensor(host.shape, device, pinned=False)
        m.host = host
        m.state = MirrorState.HostAhead if not m.unified else MirrorState.Synced
        return m

    # ------------------------------------------------------------------ accessors
    def numel(self) -> int:
        return self.shape.numel()

    def nbytes(self) -> int:
        return self.numel() * 4

    def host_pinned(self) -> bool:
        return self._pinned

    def device_allocated(self) -> bool:
        return self.unified or self._dev is not None

    def device_data(self) -> torch.Tensor:
        if self.unified:
            return self.host
        if self._dev is None:
            self._dev = torch.empty(self.shape.dims, dtype=torch.float32, device=self.device.torch_device())
        return self._dev

    def pin_host(self) -> bool:
        if self._pinned or not torch.cuda.is_available():
            return self._pinned
        self.host = self.host.pin_memory()
        self._pinned = True
        return True

    # ------------------------------------------------------------------ state machine
    def modify_host(self) -> None:
        """Declares a host write.  A device-ahead mirror must be brought back first."""
        if self.state == MirrorState.DeviceAhead:
            raise RuntimeError("modify_host on a device-ahead mirror: call sync_host() first")
        if not self.unified:
            self.state = MirrorState.HostAhead

    def modify_device(self) -> None:
        if self.state == MirrorState.HostAhead:
            raise RuntimeError("modify_device on a host-ahead mirror: call sync_device() first")
        if not self.unified:
            self.device_data()
            self.state = MirrorState.DeviceAhead

    def needs_sync_device(self) -> bool:
        return self.state == MirrorState.HostAhead

    def needs_sync_host(self) -> bool:
        return self.state == MirrorState.DeviceAhead

    def copy_pending(self) -> bool:
        return self._pending

    def _copy_stream(self):
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=self.device.torch_device())
            self._event = torch.cuda.Event()
        return self._stream

    def sync_device(self, blocking: bool = True) -> None:
        """Host -> device when the host is ahead.  Non-blocking: the copy runs on the mirror's own
        stream and the compute stream is made to wait on its event."""
        if self.unified or self.state != MirrorState.HostAhead:
            return
        dev = self.device_data()
        s = self._copy_stream()
        with torch.cuda.stream(s):
            dev.copy_(self.host, non_blocking=self._pinned)
            self._event.record(s)
        compute = self.device_stream or torch.cuda.current_stream(dev.device)
        compute.wait_event(self._event)
        self._pending = not blocking
        if blocking:
            self._event.synchronize()
        self.bytes_to_device += self.nbytes()
        self.state = MirrorState.Synced

    def sync_host(self) -> None:
        if self.unified or self.state != MirrorState.DeviceAhead:
            return
        dev = self.device_data()
        s = self._copy_stream()
        compute = self.device_stream or torch.cuda.current_stream(dev.device)
        s.wait_stream(compute)
        with torch.cuda.stream(s):
            self.host.copy_(dev, non_blocking=self._pinned)
        s.synchronize()
        self.bytes_to_host += self.nbytes()
        self.state = MirrorState.Synced

    def synchronize(self) -> None:
        if self._pending and self._event is not None:
            self._event.synchronize()
        self._pending = False

    def swap(self, other: "MirroredTensor") -> None:
        self.__dict__, other.__dict__ = other.__dict__, self.__dict__
