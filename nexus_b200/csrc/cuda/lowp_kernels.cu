// Low-precision kernels: FP8 (E4M3 / E5M2) quantise with amax, per-row dynamic quantise, dequantise;
// 8-bit blockwise AdamW whose moments are stored as hardware FP8 codes relative to a per-block absmax
// (first moment: E4M3 of m / absmax; second moment: E4M3 of sqrt(v / absmax)), with the clip factor read
// from device memory so that the update can run layer by layer inside the backward pass (delayed clip);
// gradient square-sum accumulation and the delayed-clip finish.
// Parity: src/cuda/kernels_fp8.cu and src/cuda/kernels_train.cu:860-1010 (adamw8bit_kernel,
// grad_sq_accumulate, delayed_clip) of the reference, which uses a 256-entry dynamic code table.
#include "common.cuh"
#include "nx_api_kernels.h"
#include "nx_api_lowp.h"

#include <cuda_fp8.h>

namespace {
using namespace nx;

__device__ __forceinline__ uint8_t enc_fp8(float x, int fmt) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, fmt == NX_E4M3 ? __NV_E4M3 : __NV_E5M2));
}
__device__ __forceinline__ float dec_fp8(uint8_t b, int fmt) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), fmt == NX_E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// dst = fp8(x * scale[0]); amax[0] = max(amax[0], max|x|)   (scale / amax may be null: scale 1, no amax)
__global__ void fp8_quantize_kernel(const void* __restrict__ src, int src_dtype, uint8_t* __restrict__ dst, int fmt,
                                    int64_t n, const float* __restrict__ scale, unsigned int* __restrict__ amax) {
  __shared__ float s_scratch[32];
  const float sc = scale ? *scale : 1.0f;
  float am = 0.0f;
  NX_GRID_STRIDE(i, n) {
    const float x = load_as_float(src, src_dtype, i);
    am = fmaxf(am, fabsf(x));
    dst[i] = enc_fp8(x * sc, fmt);
  }
  if (amax != nullptr) {
    am = block_max(am, s_scratch);
    if (threadIdx.x == 0 && am > 0.0f) atomicMax(amax, __float_as_uint(am));
  }
}

// per-row dynamic scaling: dst[r] = fp8(x[r] * fmax / amax_r), scale_inv[r] = amax_r / fmax
__global__ void fp8_quantize_rows_kernel(const void* __restrict__ src, int src_dtype, uint8_t* __restrict__ dst,
                                         int fmt, int cols, float* __restrict__ scale_inv) {
  __shared__ float s_scratch[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * cols;
  float am = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) am = fmaxf(am, fabsf(load_as_float(src, src_dtype, base + c)));
  am = block_max(am, s_scratch);
  const float fmax = fmt == NX_E4M3 ? 448.0f : 57344.0f;
  const float sc = am > 0.0f ? fmax / am : 1.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[base + c] = enc_fp8(load_as_float(src, src_dtype, base + c) * sc, fmt);
  if (threadIdx.x == 0) scale_inv[blockIdx.x] = am > 0.0f ? am / fmax : 1.0f;
}

__global__ void fp8_dequantize_kernel(const uint8_t* __restrict__ src, int fmt, void* __restrict__ dst, int dst_dtype,
                                      int64_t n, const float* __restrict__ scale_inv) {
  const float si = scale_inv ? *scale_inv : 1.0f;
  NX_GRID_STRIDE(i, n) store_from_float(dst, dst_dtype, i, dec_fp8(src[i], fmt) * si);
}

// ------------------------------------------------------------------------------------------------
constexpr int kQBlock = 2048, kQThreads = 256, kQPer = kQBlock / kQThreads;

__global__ void __launch_bounds__(kQThreads)
adamw8_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow, float* __restrict__ grad,
              uint8_t* __restrict__ qm, uint8_t* __restrict__ qv, float* __restrict__ absmax_m,
              float* __restrict__ absmax_v, int64_t n, const NxOptState* __restrict__ st, float wd_scale, float lr_scale,
              const float* __restrict__ clip_ptr, int zero_grad) {
  if (st->found_inf) return;
  __shared__ float s_scratch[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kQBlock;
  const float am = absmax_m[blockIdx.x], av = absmax_v[blockIdx.x];
  const float clip = clip_ptr ? *clip_ptr : st->clip_coef;
  const float lr = __fmul_rn(st->lr, lr_scale);
  const float lrwd = __fmul_rn(lr, __fmul_rn(st->weight_decay, wd_scale));
  const float b1 = st->beta1, b2 = st->beta2, omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  const float i1 = st->inv_bias1, i2 = st->inv_bias2, eps = st->eps;
  float mt[kQPer], vt[kQPer];
  float lm = 0.0f, lv = 0.0f;
#pragma unroll
  for (int k = 0; k < kQPer; ++k) {
    const int64_t i = base + threadIdx.x + static_cast<int64_t>(k) * kQThreads;
    mt[k] = vt[k] = 0.0f;
    if (i >= n) continue;
    float p = master ? master[i] : __bfloat162float(shadow[i]);
    const float g = __fmul_rn(grad[i], clip);
    p = __fsub_rn(p, __fmul_rn(lrwd, p));
    const float m0 = dec_fp8(qm[i], NX_E4M3) * (am * (1.0f / 448.0f));
    const float u0 = dec_fp8(qv[i], NX_E4M3) * (1.0f / 448.0f);
    const float v0 = u0 * u0 * av;
    mt[k] = __fadd_rn(__fmul_rn(b1, m0), __fmul_rn(omb1, g));
    vt[k] = __fadd_rn(__fmul_rn(b2, v0), __fmul_rn(omb2, __fmul_rn(g, g)));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr, __fmul_rn(mt[k], i1)), __fadd_rn(__fsqrt_rn(__fmul_rn(vt[k], i2)), eps)));
    if (master) master[i] = p;
    if (shadow) shadow[i] = __float2bfloat16_rn(p);
    if (zero_grad) grad[i] = 0.0f;
    lm = fmaxf(lm, fabsf(mt[k]));
    lv = fmaxf(lv, vt[k]);
  }
  const float nm = block_max(lm, s_scratch);
  const float nv = block_max(lv, s_scratch);
  const float sm = nm > 0.0f ? 448.0f / nm : 0.0f;
  const float sv = nv > 0.0f ? 1.0f / nv : 0.0f;
#pragma unroll
  for (int k = 0; k < kQPer; ++k) {
    const int64_t i = base + threadIdx.x + static_cast<int64_t>(k) * kQThreads;
    if (i >= n) continue;
    qm[i] = enc_fp8(mt[k] * sm, NX_E4M3);
    qv[i] = enc_fp8(sqrtf(vt[k] * sv) * 448.0f, NX_E4M3);
  }
  if (threadIdx.x == 0) {
    absmax_m[blockIdx.x] = nm;
    absmax_v[blockIdx.x] = nv;
  }
}

__global__ void grad_sq_accumulate_kernel(const float* __restrict__ g, int64_t n, double* __restrict__ accum) {
  __shared__ double s_scratch[32];
  double acc = 0.0;
  NX_GRID_STRIDE(i, n) acc += static_cast<double>(g[i]) * g[i];
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) atomicAdd(accum, acc);
}

__global__ void delayed_clip_finish_kernel(float* clip, float* norm_out, double* accum, double max_norm) {
  const double norm = sqrt(*accum);
  if (norm_out) *norm_out = static_cast<float>(norm);
  *clip = (max_norm > 0.0 && isfinite(norm)) ? static_cast<float>(fmin(1.0, max_norm / (norm + 1e-6))) : 1.0f;
  *accum = 0.0;
}
}  // namespace

extern "C" int nx_fp8_quantize(const void* src, int src_dtype, void* dst, int fmt, int64_t n, const float* scale,
                               float* amax, nx_stream_t stream) {
  if (n <= 0) return 0;
  if ((fmt != NX_E4M3 && fmt != NX_E5M2) || src_dtype < 0 || src_dtype > NX_F16) return -1;
  fp8_quantize_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, src_dtype, static_cast<uint8_t*>(dst), fmt, n, scale, reinterpret_cast<unsigned int*>(amax));
  return launch_status();
}

extern "C" int nx_fp8_quantize_rows(const void* src, int src_dtype, void* dst, int fmt, int rows, int cols,
                                    float* scale_inv, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((fmt != NX_E4M3 && fmt != NX_E5M2) || src_dtype < 0 || src_dtype > NX_F16 || scale_inv == nullptr) return -1;
  fp8_quantize_rows_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, src_dtype, static_cast<uint8_t*>(dst),
                                                                               fmt, cols, scale_inv);
  return launch_status();
}

extern "C" int nx_fp8_dequantize(const void* src, int fmt, void* dst, int dst_dtype, int64_t n, const float* scale_inv,
                                 nx_stream_t stream) {
  if (n <= 0) return 0;
  if ((fmt != NX_E4M3 && fmt != NX_E5M2) || dst_dtype < 0 || dst_dtype > NX_F16) return -1;
  fp8_dequantize_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), fmt, dst, dst_dtype, n, scale_inv);
  return launch_status();
}

extern "C" int nx_adamw8_block(void) { return kQBlock; }

extern "C" int nx_adamw8(float* master, void* shadow, float* grad, void* qm, void* qv, float* absmax_m, float* absmax_v,
                         int64_t n, const NxOptState* state, float wd_scale, float lr_scale, const float* clip,
                         int zero_grad, nx_stream_t stream) {
  if (n <= 0) return 0;
  if ((master == nullptr && shadow == nullptr) || grad == nullptr || qm == nullptr || qv == nullptr) return -1;
  const int blocks = static_cast<int>((n + kQBlock - 1) / kQBlock);
  adamw8_kernel<<<blocks, kQThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      master, static_cast<__nv_bfloat16*>(shadow), grad, static_cast<uint8_t*>(qm), static_cast<uint8_t*>(qv), absmax_m,
      absmax_v, n, state, wd_scale, lr_scale, clip, zero_grad);
  return launch_status();
}

extern "C" int nx_grad_sq_accumulate(const float* grad, int64_t n, double* accum, nx_stream_t stream) {
  if (n <= 0) return 0;
  grad_sq_accumulate_kernel<<<blocks_for(n, 256, 148 * 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(grad, n, accum);
  return launch_status();
}

extern "C" int nx_delayed_clip_finish(float* clip, float* norm_out, double* accum, double max_norm, nx_stream_t stream) {
  delayed_clip_finish_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(clip, norm_out, accum, max_norm);
  return launch_status();
}
