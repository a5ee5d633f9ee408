"""Backend abstraction: a ``Driver`` interface (memory, streams/events and the FP32 op set), a CPU
reference driver, the CUDA driver on the sm_100a kernels, stub drivers that report why they are
unavailable (HIP, Vulkan, Metal, DirectML, PJRT), and a ``Registry`` that selects by the
``NEXUS_BACKEND`` environment variable.  Operations take FP32 torch tensors living on the driver's
device.  A driver that lacks an op falls back to the CPU reference under an explicit policy
(``Error`` / ``WarnOnce`` / ``WarnAlways``) with statistics; nothing falls back silently.

Parity: include/nexus/backend/backend.hpp:27-236, src/backend/registry.cpp:113-958 of the reference."""
from __future__ import annotations

import ctypes as C
import enum
import math
import os
import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch


class Kind(enum.IntEnum):
    Cpu = 0
    Cuda = 1
    Hip = 2
    Vulkan = 3
    Metal = 4
    DirectMl = 5
    Pjrt = 6


class Operation(enum.IntEnum):
    Add = 0
    Sub = 1
    Mul = 2
    Div = 3
    Neg = 4
    Exp = 5
    Log = 6
    Sqrt = 7
    Rsqrt = 8
    Tanh = 9
    Sigmoid = 10
    Silu = 11
    Relu = 12
    Scale = 13
    Axpy = 14
    MatMul = 15
    ReduceSum = 16
    Fill = 17
    Softmax = 18
    RmsNorm = 19
    LayerNorm = 20
    Rope = 21
    SwiGlu = 22
    Attention = 23
    QuantMatMulQ8 = 24
    QuantMatMulQ4 = 25
    AdamW = 26


ELEMENTWISE = tuple(Operation(i) for i in range(15))
_KIND_NAMES = {"cpu": Kind.Cpu, "cuda": Kind.Cuda, "hip": Kind.Hip, "rocm": Kind.Hip, "vulkan": Kind.Vulkan,
               "metal": Kind.Metal, "directml": Kind.DirectMl, "dml": Kind.DirectMl, "pjrt": Kind.Pjrt}


def parse_kind(text: str) -> Kind:
    k = _KIND_NAMES.get(text.strip().lower())
    if k is None:
        raise ValueError(f"unknown backend {text!r}")
    return k


@dataclass
class DeviceInfo:
    device: str = "cpu"
    name: str = ""
    vendor: str = ""
    api_version: str = ""
    driver_version: str = ""
    memory_bytes: int = 0
    subgroup_size: int = 0
    unified_memory: bool = False


@dataclass
class AllocatorStats:
    allocations: int = 0
    cache_hits: int = 0
    live_blocks: int = 0
    current_bytes: int = 0
    reserved_bytes: int = 0


class FallbackPolicy(enum.IntEnum):
    Error = 0
    WarnOnce = 1
    WarnAlways = 2


@dataclass
class FallbackStats:
    calls: int = 0
    elements: int = 0


_policy = [FallbackPolicy.Error]
_fallbacks: Dict[Tuple[Kind, Operation], FallbackStats] = {}
_warned = set()


def set_fallback_policy(p: FallbackPolicy) -> None:
    _policy[0] = FallbackPolicy(p)


def fallback_policy() -> FallbackPolicy:
    return _policy[0]


def fallback_stats(kind: Kind, op: Operation) -> FallbackStats:
    return _fallbacks.get((kind, op), FallbackStats())


def reset_fallback_stats() -> None:
    _fallbacks.clear()
    _warned.clear()


def require_cpu_fallback(driver: "Driver", op: Operation, elements: int) -> None:
    """Called by a driver before it computes ``op`` on the host instead of its device."""
    if _policy[0] == FallbackPolicy.Error:
        raise RuntimeError(f"backend {driver.name()} has no {op.name} kernel and the fallback policy is Error")
    st = _fallbacks.setdefault((driver.kind(), op), FallbackStats())
    st.calls += 1
    st.elements += int(elements)
    key = (driver.kind(), op)
    if _policy[0] == FallbackPolicy.WarnAlways or key not in _warned:
        _warned.add(key)
        warnings.warn(f"{driver.name()}: {op.name} runs on the CPU reference ({elements} elements)", RuntimeWarning)


# ---------------------------------------------------------------------------------------------- interface
class Driver:
    """Base class: every op has a reference implementation here (torch on the tensor's own device in
    FP32 / FP64 where the reference accumulates in FP64), so a concrete driver overrides what it has."""

    def kind(self) -> Kind:
        raise NotImplementedError

    def name(self) -> str:
        raise NotImplementedError

    def version(self) -> str:
        return "1"

    def devices(self) -> List[DeviceInfo]:
        return []

    def unavailable_reason(self) -> str:
        return ""

    def supports(self, op: Operation) -> bool:
        return False

    def available(self) -> bool:
        return len(self.devices()) > 0

    # memory / ordering ---------------------------------------------------------------------------
    def torch_device(self, index: int = 0) -> torch.device:
        return torch.device("cpu")

    def allocate(self, index: int, nbytes: int) -> torch.Tensor:
        self._stats.allocations += 1
        self._stats.live_blocks += 1
        self._stats.current_bytes += nbytes
        self._stats.reserved_bytes = max(self._stats.reserved_bytes, self._stats.current_bytes)
        return torch.empty(nbytes, dtype=torch.uint8, device=self.torch_device(index))

    def deallocate(self, index: int, buf: torch.Tensor) -> None:
        self._stats.live_blocks -= 1
        self._stats.current_bytes -= buf.numel()

    def copy(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        dst.view(-1).copy_(src.view(-1))

    def synchronize(self, index: int = 0) -> None:
        pass

    def allocator_stats(self, index: int = 0) -> AllocatorStats:
        return self._stats

    def create_stream(self, index: int = 0):
        return None

    def synchronize_stream(self, index: int, stream) -> None:
        pass

    def create_event(self, index: int = 0):
        return None

    def record_event(self, index: int, event, stream) -> None:
        pass

    def stream_wait_event(self, index: int, stream, event) -> None:
        pass

    def __init__(self):
        self._stats = AllocatorStats()

    # reference ops -------------------------------------------------------------------------------
    def fill(self, dst: torch.Tensor, value: float) -> None:
        dst.fill_(value)

    def elementwise(self, op: Operation, a, b, out, scalar: float = 0.0) -> None:
        f = {Operation.Add: lambda: a + b, Operation.Sub: lambda: a - b, Operation.Mul: lambda: a * b,
             Operation.Div: lambda: a / b, Operation.Neg: lambda: -a, Operation.Exp: lambda: a.exp(),
             Operation.Log: lambda: a.log(), Operation.Sqrt: lambda: a.sqrt(), Operation.Rsqrt: lambda: a.rsqrt(),
             Operation.Tanh: lambda: a.tanh(), Operation.Sigmoid: lambda: a.sigmoid(),
             Operation.Silu: lambda: a * a.sigmoid(), Operation.Relu: lambda: a.clamp_min(0),
             Operation.Scale: lambda: a * scalar, Operation.Axpy: lambda: a * scalar + b}[Operation(op)]
        out.copy_(f())

    def matmul(self, a, b, c, *, a_trans=False, b_trans=False, alpha=1.0, beta=0.0) -> None:
        """c = alpha * op(a) @ op(b) + beta * c with b_trans meaning b is stored [n, k]."""
        aa = a.t() if a_trans else a
        bb = b.t() if b_trans else b
        r = alpha * (aa.double() @ bb.double()).float()
        c.copy_(r if beta == 0.0 else r + beta * c)

    def reduce_sum(self, x, out) -> None:
        out.copy_(x.double().sum().float())

    def softmax(self, x, out) -> None:
        out.copy_(torch.softmax(x.float(), -1))

    def rms_norm(self, x, weight, out, eps=1e-5) -> None:
        r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_(x * r * (weight if weight is not None else 1.0))

    def layer_norm(self, x, weight, bias, out, eps=1e-5) -> None:
        out.copy_(torch.nn.functional.layer_norm(x, x.shape[-1:], weight, bias, eps))

    def rope(self, x, out, pos_offset=0, theta=10000.0) -> None:
        """x: [bh, T, 2*half] with interleaved pairs."""
        bh, T, d = x.shape
        half = d // 2
        t = torch.arange(T, device=x.device, dtype=torch.float32) + pos_offset
        inv = theta ** (-(torch.arange(half, device=x.device, dtype=torch.float32) * 2) / (2 * half))
        ang = t[:, None] * inv[None, :]
        c, s = ang.cos(), ang.sin()
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c

    def swiglu(self, x, out) -> None:
        h = x.shape[-1] // 2
        out.copy_(torch.nn.functional.silu(x[..., :h]) * x[..., h:])

    def attention(self, q, k, v, out, causal=True) -> None:
        """[bh, T, D] FP32, scale 1/sqrt(D)."""
        T, D = q.shape[1], q.shape[2]
        s = (q.double() @ k.double().transpose(1, 2)) / math.sqrt(D)
        if causal:
            s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        out.copy_((s.softmax(-1) @ v.double()).float())

    @staticmethod
    def _dequant(wq: torch.Tensor, scales: torch.Tensor, k: int, group: int, bits: int) -> torch.Tensor:
        raw = wq.contiguous().view(torch.uint8)
        n = scales.shape[0]
        if bits == 8:
            q = raw.view(torch.int8).view(n, k).float()
        else:
            b = raw.view(n, k // 2)
            q = torch.stack([(b & 15).float() - 8, (b >> 4).float() - 8], -1).view(n, k)
        return (q.view(n, k // group, group) * scales[:, :, None]).view(n, k)

    def quant_matmul_q8(self, a, wq, scales, c, group=32) -> None:
        c.copy_(a @ self._dequant(wq, scales, a.shape[1], group, 8).t())

    def quant_matmul_q4(self, a, wq, scales, c, group=32) -> None:
        c.copy_(a @ self._dequant(wq, scales, a.shape[1], group, 4).t())

    def adamw_step(self, p, g, m, v, lr, beta1, beta2, eps, weight_decay, step) -> None:
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        p.sub_(lr * ((m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * p))


class CpuDriver(Driver):
    def kind(self):
        return Kind.Cpu

    def name(self):
        return "cpu"

    def devices(self):
        import platform
        return [DeviceInfo("cpu", platform.processor() or "cpu", "host", unified_memory=True)]

    def supports(self, op):
        return True


class CudaDriver(Driver):
    """FP32 op set on the sm_100a kernel library."""

    def __init__(self):
        super().__init__()
        self._devices: Optional[List[DeviceInfo]] = None
        self._why = ""

    def kind(self):
        return Kind.Cuda

    def name(self):
        return "cuda-sm100a"

    def devices(self):
        if self._devices is None:
            self._devices = []
            from ..ops import _cuda as K
            if not torch.cuda.is_available():
                self._why = "no CUDA device is visible"
            elif not K.available():
                self._why = "the sm_100a kernel library has not been built"
            else:
                for i in range(torch.cuda.device_count()):
                    p = torch.cuda.get_device_properties(i)
                    self._devices.append(DeviceInfo(f"cuda:{i}", p.name, "NVIDIA", f"sm_{p.major}{p.minor}",
                                                    torch.version.cuda or "", p.total_memory, 32, False))
        return self._devices

    def unavailable_reason(self):
        self.devices()
        return self._why

    def supports(self, op):
        return True

    def torch_device(self, index=0):
        return torch.device("cuda", index)

    def synchronize(self, index=0):
        torch.cuda.synchronize(index)

    def create_stream(self, index=0):
        return torch.cuda.Stream(device=index)

    def synchronize_stream(self, index, stream):
        stream.synchronize()

    def create_event(self, index=0):
        return torch.cuda.Event()

    def record_event(self, index, event, stream):
        event.record(stream)

    def stream_wait_event(self, index, stream, event):
        stream.wait_event(event)

    # kernels ------------------------------------------------------------------------------------
    @staticmethod
    def _k():
        from ..ops import _cuda as K
        return K

    def fill(self, dst, value):
        K = self._k()
        K._check(K.lib().nx_fill(K._p(dst), C.c_int(K._DT[dst.dtype]), C.c_int64(dst.numel()), C.c_float(value),
                                 K._stream()), "nx_fill")

    def elementwise(self, op, a, b, out, scalar=0.0):
        K = self._k()
        K._check(K.lib().nx_bk_elementwise(K._p(a), K._p(b), K._p(out), C.c_int64(a.numel()), C.c_float(scalar),
                                           C.c_int(int(op)), K._stream()), "nx_bk_elementwise")

    def matmul(self, a, b, c, *, a_trans=False, b_trans=False, alpha=1.0, beta=0.0):
        K = self._k()
        m, n = c.shape
        k = a.shape[0] if a_trans else a.shape[1]
        K._check(K.lib().nx_bk_matmul_f32(K._p(a), K._p(b), K._p(c), C.c_int(m), C.c_int(n), C.c_int(k),
                                          C.c_int(a.stride(0)), C.c_int(b.stride(0)), C.c_int(c.stride(0)),
                                          C.c_int(int(a_trans)), C.c_int(int(b_trans)), C.c_float(alpha),
                                          C.c_float(beta), K._stream()), "nx_bk_matmul_f32")

    def reduce_sum(self, x, out):
        K = self._k()
        L = K.lib()
        L.nx_bk_reduce_partials.restype = C.c_int64
        n = x.numel()
        parts = K.scratch(int(L.nx_bk_reduce_partials(C.c_int64(n))) * 8, "bk_reduce", x.device)
        K._check(L.nx_bk_reduce_sum(K._p(x), C.c_int64(n), K._p(parts), K._p(out), K._stream()), "nx_bk_reduce_sum")

    def _rows(self, x, gamma, beta, out, op, eps):
        K = self._k()
        rows, cols = x.numel() // x.shape[-1], x.shape[-1]
        K._check(K.lib().nx_bk_norm_softmax(K._p(x), K._p(gamma), K._p(beta), K._p(out), C.c_int(rows), C.c_int(cols),
                                            C.c_int(op), C.c_float(eps), K._stream()), "nx_bk_norm_softmax")

    def softmax(self, x, out):
        self._rows(x, None, None, out, 0, 0.0)

    def rms_norm(self, x, weight, out, eps=1e-5):
        self._rows(x, weight, None, out, 1, eps)

    def layer_norm(self, x, weight, bias, out, eps=1e-5):
        self._rows(x, weight, bias, out, 2, eps)

    def rope(self, x, out, pos_offset=0, theta=10000.0):
        K = self._k()
        bh, T, d = x.shape
        K._check(K.lib().nx_bk_rope_pairs(K._p(x), K._p(out), C.c_int(bh), C.c_int(T), C.c_int(d // 2),
                                          C.c_int(pos_offset), C.c_float(theta), K._stream()), "nx_bk_rope_pairs")

    def swiglu(self, x, out):
        K = self._k()
        rows, h2 = x.numel() // x.shape[-1], x.shape[-1]
        K._check(K.lib().nx_bk_swiglu_f32(K._p(x), K._p(out), C.c_int(rows), C.c_int(h2 // 2), K._stream()),
                 "nx_bk_swiglu_f32")

    def attention(self, q, k, v, out, causal=True):
        K = self._k()
        bh, T, D = q.shape
        K._check(K.lib().nx_bk_attention_f32(K._p(q), K._p(k), K._p(v), K._p(out), C.c_int(bh), C.c_int(T), C.c_int(D),
                                             C.c_float(1.0 / math.sqrt(D)), C.c_int(int(causal)), K._stream()),
                 "nx_bk_attention_f32")

    def _qmm(self, a, wq, scales, c, group, bits):
        K = self._k()
        m, k = a.shape
        K._check(K.lib().nx_bk_quant_matmul(K._p(a), K._p(wq), K._p(scales), K._p(c), C.c_int(m), C.c_int(c.shape[1]),
                                            C.c_int(k), C.c_int(group), C.c_int(bits), K._stream()),
                 "nx_bk_quant_matmul")

    def quant_matmul_q8(self, a, wq, scales, c, group=32):
        self._qmm(a, wq, scales, c, group, 8)

    def quant_matmul_q4(self, a, wq, scales, c, group=32):
        self._qmm(a, wq, scales, c, group, 4)

    def adamw_step(self, p, g, m, v, lr, beta1, beta2, eps, weight_decay, step):
        K = self._k()
        K._check(K.lib().nx_bk_adamw_step(K._p(p), K._p(g), K._p(m), K._p(v), C.c_int64(p.numel()), C.c_float(lr),
                                          C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(weight_decay),
                                          C.c_float(1 - beta1 ** step), C.c_float(1 - beta2 ** step), K._stream()),
                 "nx_bk_adamw_step")


class UnavailableDriver(Driver):
    """A backend whose runtime cannot be brought up on this machine; says why."""

    def __init__(self, kind: Kind, name: str, reason: str):
        super().__init__()
        self._kind, self._name, self._reason = kind, name, reason

    def kind(self):
        return self._kind

    def name(self):
        return self._name

    def unavailable_reason(self):
        return self._reason


class Registry:
    _instance: Optional["Registry"] = None

    def __init__(self):
        from .hip import HipDriver
        from .pjrt import PjrtDriver
        self._drivers: List[Driver] = [
            CpuDriver(), CudaDriver(), HipDriver(), PjrtDriver(),
            UnavailableDriver(Kind.Vulkan, "vulkan", "no Vulkan loader on this machine; the shader math runs as "
                                                     "CUDA kernels in the cuda driver"),
            UnavailableDriver(Kind.Metal, "metal", "Metal exists on Apple platforms only"),
            UnavailableDriver(Kind.DirectMl, "directml", "DirectML exists on Windows only"),
        ]

    @classmethod
    def instance(cls) -> "Registry":
        if cls._instance is None:
            cls._instance = Registry()
        return cls._instance

    def add(self, driver: Driver) -> None:
        self._drivers = [d for d in self._drivers if d.kind() != driver.kind()] + [driver]

    def all(self) -> List[Driver]:
        return list(self._drivers)

    def find(self, kind: Kind) -> Optional[Driver]:
        for d in self._drivers:
            if d.kind() == kind:
                return d
        return None

    def require(self, kind: Kind) -> Driver:
        d = self.find(kind)
        if d is None or not d.available():
            why = d.unavailable_reason() if d is not None else "not registered"
            raise RuntimeError(f"backend {Kind(kind).name} is unavailable: {why}")
        return d

    def select(self, op: Operation = Operation.MatMul) -> Driver:
        """``NEXUS_BACKEND`` names the driver; otherwise the first available of cuda, hip, cpu that has ``op``."""
        env = os.environ.get("NEXUS_BACKEND", "").strip()
        if env:
            return self.require(parse_kind(env))
        for kind in (Kind.Cuda, Kind.Hip, Kind.Cpu):
            d = self.find(kind)
            if d is not None and d.available() and d.supports(op):
                return d
        raise RuntimeError("no backend is available")
