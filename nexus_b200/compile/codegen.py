"""Code generation for ``Fused`` element-wise clusters with a run-time compile step and a disk cache keyed
by the source hash: CUDA C++ compiled by NVRTC for sm_100a and launched through the driver API, or plain
C++ compiled by the host compiler into a shared object (CPU).
Parity: include/nexus/compile/codegen.hpp:20-66, src/compile/codegen.cpp, src/cuda/nvrtc_jit.cpp of the
reference (which emits AVX2 source for cl.exe and CUDA source for NVRTC)."""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile
from typing import Dict, List, Tuple

import torch

_EXPR = {"Add": "({0} + {1})", "Sub": "({0} - {1})", "Mul": "({0} * {1})", "Relu": "fmaxf({0}, 0.0f)",
         "Tanh": "tanhf({0})", "Sigmoid": "(1.0f / (1.0f + expf(-{0})))", "Silu": "({0} / (1.0f + expf(-{0})))",
         "Gelu": "(0.5f * {0} * (1.0f + tanhf(0.7978845608028654f * ({0} + 0.044715f * {0} * {0} * {0}))))",
         "Cast": "{0}"}


def cache_dir() -> str:
    d = os.environ.get("NEXUS_JIT_CACHE", os.path.join(tempfile.gettempdir(), "nexus_b200_jit"))
    os.makedirs(d, exist_ok=True)
    return d


def cluster_source(body, n_inputs: int, n_outputs: int, cuda: bool, out_steps: List[int]) -> str:
    """body: [(op, attrs, [("in", i) | ("tmp", j)])]; out_steps: which step each output takes."""
    args = ", ".join([f"const float* __restrict__ in{i}" for i in range(n_inputs)] +
                     [f"float* __restrict__ out{i}" for i in range(n_outputs)] + ["long long n"])
    lines = []
    for j, (op, attrs, srcs) in enumerate(body):
        names = [f"in{i}[i]" if kind == "in" else f"t{i}" for kind, i in srcs]
        if op == "Scale":
            expr = f"({names[0]} * {float(attrs['factor'])!r}f)"
        else:
            expr = _EXPR[op].format(*names)
        lines.append(f"    const float t{j} = {expr};")
    for o, step in enumerate(out_steps):
        lines.append(f"    out{o}[i] = t{step};")
    inner = "\n".join(lines)
    if cuda:
        return (f'extern "C" __global__ void fused({args}) {{\n'
                "  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {\n"
                f"{inner}\n  }}\n}}\n")
    return f'#include <math.h>\nextern "C" void fused({args}) {{\n  for (long long i = 0; i < n; ++i) {{\n{inner}\n  }}\n}}\n'


def compile_cuda(src: str, arch: str = "sm_100a") -> bytes:
    """NVRTC -> CUBIN (cached on disk by the hash of source + architecture)."""
    key = hashlib.sha256((arch + "\n" + src).encode()).hexdigest()
    path = os.path.join(cache_dir(), key + ".cubin")
    if os.path.exists(path):
        with open(path, "rb") as f:
            return f.read()
    from cuda.bindings import nvrtc
    err, prog = nvrtc.nvrtcCreateProgram(src.encode(), b"fused.cu", 0, [], [])
    opts = [f"--gpu-architecture={arch}".encode(), b"--std=c++17"]
    (err,) = nvrtc.nvrtcCompileProgram(prog, len(opts), opts)
    if int(err) != 0:
        _, n = nvrtc.nvrtcGetProgramLogSize(prog)
        log = b" " * n
        nvrtc.nvrtcGetProgramLog(prog, log)
        raise RuntimeError("NVRTC failed:\n" + log.decode(errors="replace"))
    _, n = nvrtc.nvrtcGetCUBINSize(prog)
    cubin = b" " * n
    nvrtc.nvrtcGetCUBIN(prog, cubin)
    nvrtc.nvrtcDestroyProgram(prog)
    tmp = path + f".{os.getpid()}.tmp"
    with open(tmp, "wb") as f:
        f.write(cubin)
    os.replace(tmp, path)
    return cubin


def compile_cpu(src: str) -> str:
    key = hashlib.sha256(("cpu\n" + src).encode()).hexdigest()
    so = os.path.join(cache_dir(), key + ".so")
    if not os.path.exists(so):
        cpp = os.path.join(cache_dir(), key + ".cpp")
        with open(cpp, "w") as f:
            f.write(src)
        tmp = so + f".{os.getpid()}.tmp"
        subprocess.run(["g++", "-O3", "-march=native", "-ffast-math", "-shared", "-fPIC", cpp, "-o", tmp], check=True)
        os.replace(tmp, so)
    return so


class FusedKernel:
    """Callable for one cluster; compiled on first use for the device of its inputs."""

    def __init__(self, body, n_inputs: int, out_steps: List[int]):
        self.body, self.n_in, self.out_steps = body, n_inputs, out_steps
        self._cpu = None
        self._cuda: Dict[int, Tuple[object, object]] = {}

    def source(self, cuda: bool) -> str:
        return cluster_source(self.body, self.n_in, len(self.out_steps), cuda, self.out_steps)

    def __call__(self, *inputs: torch.Tensor) -> List[torch.Tensor]:
        shape = inputs[0].shape
        xs = [t.expand(shape).contiguous().float() for t in inputs]
        outs = [torch.empty(shape, dtype=torch.float32, device=xs[0].device) for _ in self.out_steps]
        n = xs[0].numel()
        if xs[0].is_cuda:
            from cuda.bindings import driver
            dev = xs[0].device.index or 0
            if dev not in self._cuda:
                cubin = compile_cuda(self.source(True))
                err, mod = driver.cuModuleLoadData(cubin)
                if int(err) != 0:
                    raise RuntimeError(f"cuModuleLoadData failed: {err}")
                err, fn = driver.cuModuleGetFunction(mod, b"fused")
                self._cuda[dev] = (mod, fn)
            fn = self._cuda[dev][1]
            vals = tuple(t.data_ptr() for t in xs + outs) + (n,)
            types = tuple([ctypes.c_void_p] * (len(xs) + len(outs)) + [ctypes.c_longlong])
            blocks = max(1, min((n + 255) // 256, 148 * 8))
            (err,) = driver.cuLaunchKernel(fn, blocks, 1, 1, 256, 1, 1, 0, torch.cuda.current_stream().cuda_stream,
                                           (vals, types), 0)
            if int(err) != 0:
                raise RuntimeError(f"cuLaunchKernel failed: {err}")
        else:
            if self._cpu is None:
                self._cpu = ctypes.CDLL(compile_cpu(self.source(False))).fused
            self._cpu(*[ctypes.c_void_p(t.data_ptr()) for t in xs + outs], ctypes.c_longlong(n))
        return outs
