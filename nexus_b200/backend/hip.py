"""HIP driver shell and the CUDA -> HIP source translation table.

The driver looks for the ROCm runtime libraries and reports why it is unavailable when they are
missing (always the case on an NVIDIA machine).  ``hipify_source`` rewrites CUDA runtime / cuBLASLt /
NVRTC / NCCL identifiers to their HIP / hipBLASLt / hiprtc / RCCL names on identifier boundaries.
Parity: src/backend/hip.cpp:38-80,199-255, include/nexus/backend/hip_compat.hpp of the reference."""
from __future__ import annotations

import ctypes.util
import re

from .driver import Driver, Kind

_PREFIX_RULES = (("cudaStream", "hipStream"), ("cudaEvent", "hipEvent"), ("cudaMemcpy", "hipMemcpy"),
                 ("cudaMemset", "hipMemset"), ("cudaMalloc", "hipMalloc"), ("cudaFree", "hipFree"),
                 ("cudaHost", "hipHost"), ("cudaDevice", "hipDevice"), ("cudaGetDevice", "hipGetDevice"),
                 ("cudaSetDevice", "hipSetDevice"), ("cudaGetLastError", "hipGetLastError"),
                 ("cudaGetErrorString", "hipGetErrorString"), ("cudaError", "hipError"),
                 ("cudaSuccess", "hipSuccess"), ("cudaLaunch", "hipLaunch"), ("cudaFunc", "hipFunc"),
                 ("cudaGraph", "hipGraph"), ("cudaOccupancy", "hipOccupancy"), ("cublasLt", "hipblasLt"),
                 ("CUBLASLT_", "HIPBLASLT_"), ("cublas", "hipblas"), ("CUBLAS_", "HIPBLAS_"), ("nvrtc", "hiprtc"),
                 ("NVRTC_", "HIPRTC_"), ("curand", "hiprand"), ("CURAND_", "HIPRAND_"))
_EXACT = {"cuda_runtime.h": "hip/hip_runtime.h", "cuda_runtime_api.h": "hip/hip_runtime_api.h",
          "cuda_fp16.h": "hip/hip_fp16.h", "cuda_bf16.h": "hip/hip_bf16.h", "cublasLt.h": "hipblaslt/hipblaslt.h",
          "nvrtc.h": "hip/hiprtc.h", "nccl.h": "rccl/rccl.h", "__nv_bfloat16": "hip_bfloat16",
          "__nv_bfloat162": "hip_bfloat162", "CUdeviceptr": "hipDeviceptr_t", "CUstream": "hipStream_t",
          "CUmodule": "hipModule_t", "CUfunction": "hipFunction_t", "cuModuleLoadData": "hipModuleLoadData",
          "cuModuleGetFunction": "hipModuleGetFunction", "cuLaunchKernel": "hipModuleLaunchKernel",
          "__shfl_xor_sync": "__shfl_xor", "__shfl_down_sync": "__shfl_down", "__shfl_sync": "__shfl",
          "__syncwarp": "__builtin_amdgcn_wave_barrier"}
# NCCL and RCCL share their API names: only the header and the library differ.
_IDENT = re.compile(r"[A-Za-z_][A-Za-z0-9_\.]*")


def hipify_source(src: str) -> str:
    """Identifier-wise translation; `mask` arguments of the *_sync shuffles are dropped."""
    def repl(m):
        w = m.group(0)
        if w in _EXACT:
            return _EXACT[w]
        for a, b in _PREFIX_RULES:
            if w.startswith(a):
                return b + w[len(a):]
        return w
    out = _IDENT.sub(repl, src)
    # __shfl_xor_sync(mask, v, o) -> __shfl_xor(v, o)
    out = re.sub(r"(__shfl(?:_xor|_down)?)\(\s*[^,()]+,\s*", r"\1(", out)
    return out


class HipDriver(Driver):
    LIBS = ("amdhip64", "hiprtc", "hipblaslt")

    def kind(self):
        return Kind.Hip

    def name(self):
        return "hip"

    def unavailable_reason(self):
        missing = [lib for lib in self.LIBS if ctypes.util.find_library(lib) is None]
        if missing:
            return "ROCm runtime libraries not found: " + ", ".join(missing)
        return "ROCm libraries are present but this build carries sm_100a kernels only"
