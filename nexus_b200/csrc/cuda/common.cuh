// Device helpers shared by the memory-bound kernels: warp/block reductions, typed loads/stores,
// grid sizing.  Parity: src/cuda/common.cuh:30-137 of the reference (warp_sum/block_sum,
// blocks_for, Num<T> load/store); written for 32-wide warps only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nx {

constexpr int kNumSmsB200 = 148;

// Lets a following kernel that was launched with the programmatic-serialization attribute (the tensor-core GEMM)
// begin its prologue early; that kernel still waits for this grid to complete before it reads anything.  A no-op
// when the next launch is an ordinary one.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide reductions; `scratch` holds 32 values of T in shared memory.  Every thread gets the
// result.  Safe to call repeatedly with the same scratch.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  T r = (lane < nwarps) ? scratch[lane] : T(0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  return warp_max(r);
}

inline int blocks_for(int64_t n, int threads, int max_blocks = kNumSmsB200 * 16) {
  int64_t b = (n + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

#define NX_GRID_STRIDE(i, n)                                                                       \
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < (n);          \
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)

template <typename T>
struct Num;
template <>
struct Num<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <>
struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <>
struct Num<__half> {
  static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};

// dtype codes follow NxDType in nx_api.h: 0 bf16, 1 f32, 2 f16.
__device__ __forceinline__ float load_as_float(const void* base, int dtype, int64_t i) {
  if (dtype == 1) return reinterpret_cast<const float*>(base)[i];
  if (dtype == 0) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  return __half2float(reinterpret_cast<const __half*>(base)[i]);
}
__device__ __forceinline__ void store_from_float(void* base, int dtype, int64_t i, float v) {
  if (dtype == 1)
    reinterpret_cast<float*>(base)[i] = v;
  else if (dtype == 0)
    reinterpret_cast<__nv_bfloat16*>(base)[i] = __float2bfloat16_rn(v);
  else
    reinterpret_cast<__half*>(base)[i] = __float2half_rn(v);
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? 0 : -2; }

}  // namespace nx
