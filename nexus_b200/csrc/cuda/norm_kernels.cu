// LayerNorm / RMSNorm forward (optionally fused with the residual add that feeds them) and a
// deterministic backward: dx per row (optionally fused with the residual-path gradient) plus
// column-wise parameter gradients reduced in a fixed order through caller-provided partials.
// Statistics are always FP32.  Parity: src/cuda/kernels_norm.cu:80-434 of the reference
// (layernorm_forward, residual_layernorm_forward, rmsnorm_forward, norm backward + 2-stage
// deterministic parameter reduce).
#include "common.cuh"
#include <cstdlib>
#include "nx_api_kernels.h"

#include <algorithm>

namespace {
using namespace nx;

template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    uint2 q = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&q.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&q.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t*>(&a);
    q.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = q;
  }
};

// One warp per row; the row is re-read from L1/L2 for the second and third pass.
template <typename XT, typename PT, typename YT, bool kRms>
__global__ void norm_fwd_kernel(const XT* __restrict__ x, const XT* __restrict__ res, XT* __restrict__ sum_out,
                                const PT* __restrict__ gamma, const PT* __restrict__ beta, YT* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int cols,
                                float eps) {
  pdl_trigger();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 2;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const XT* xr = x + static_cast<int64_t>(row) * cols;
    const XT* rr = res ? res + static_cast<int64_t>(row) * cols : nullptr;
    XT* sr = sum_out ? sum_out + static_cast<int64_t>(row) * cols : nullptr;
    float s = 0.0f;
    for (int i = lane; i < nvec; i += 32) {
      float v[4];
      Vec4<XT>::load(xr + 4 * i, v);
      if (rr) {
        float q[4];
        Vec4<XT>::load(rr + 4 * i, q);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += q[j];
        if (sr) Vec4<XT>::store(sr + 4 * i, v);
      }
      s += kRms ? (v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3]) : (v[0] + v[1] + v[2] + v[3]);
    }
    if (rr && sr) __syncwarp();
    // After the fused add the normalised input is the sum; read it back from where it was written.
    const XT* src = (rr && sr) ? sr : xr;
    s = warp_sum(s);
    float mean = 0.0f, rstd;
    if (kRms) {
      rstd = rsqrtf(s / cols + eps);
    } else {
      mean = s / cols;
      float var = 0.0f;
      for (int i = lane; i < nvec; i += 32) {
        float v[4];
        Vec4<XT>::load(src + 4 * i, v);
        if (rr && !sr) {
          float q[4];
          Vec4<XT>::load(rr + 4 * i, q);
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] += q[j];
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) var += (v[j] - mean) * (v[j] - mean);
      }
      var = warp_sum(var);
      rstd = rsqrtf(var / cols + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    YT* yr = y + static_cast<int64_t>(row) * cols;
    for (int i = lane; i < nvec; i += 32) {
      float v[4], g[4], o[4];
      Vec4<XT>::load(src + 4 * i, v);
      if (rr && !sr) {
        float q[4];
        Vec4<XT>::load(rr + 4 * i, q);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += q[j];
      }
      Vec4<PT>::load(gamma + 4 * i, g);
      if (!kRms && beta) {
        float b[4];
        Vec4<PT>::load(beta + 4 * i, b);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (v[j] - mean) * rstd * g[j] + b[j];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (v[j] - mean) * rstd * g[j];
      }
      Vec4<YT>::store(yr + 4 * i, o);
    }
  }
}

// Rows of 128 * VPL columns: a warp keeps its row in registers (VPL vectors of four per lane), so the row is read
// from memory once with all of its loads in flight together, and gamma / beta are loaded once per warp.  Same
// arithmetic and summation order as norm_fwd_kernel.
template <typename XT, typename PT, typename YT, bool kRms, int VPL>
__global__ void __launch_bounds__(256)
norm_fwd_reg_kernel(const XT* __restrict__ x, const XT* __restrict__ res, XT* __restrict__ sum_out,
                    const PT* __restrict__ gamma, const PT* __restrict__ beta, YT* __restrict__ y,
                    float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, float eps) {
  pdl_trigger();
  constexpr int kCols = 128 * VPL;
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  float g[VPL][4], b[VPL][4];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    Vec4<PT>::load(gamma + 4 * (lane + 32 * i), g[i]);
    if (!kRms && beta) {
      Vec4<PT>::load(beta + 4 * (lane + 32 * i), b[i]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) b[i][j] = 0.0f;
    }
  }
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const XT* xr = x + static_cast<int64_t>(row) * kCols;
    float v[VPL][4];
#pragma unroll
    for (int i = 0; i < VPL; ++i) Vec4<XT>::load(xr + 4 * (lane + 32 * i), v[i]);
    if (res) {
      const XT* rr = res + static_cast<int64_t>(row) * kCols;
      float q[VPL][4];
#pragma unroll
      for (int i = 0; i < VPL; ++i) Vec4<XT>::load(rr + 4 * (lane + 32 * i), q[i]);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[i][j] += q[i][j];
      }
      if (sum_out) {
        XT* sr = sum_out + static_cast<int64_t>(row) * kCols;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
          Vec4<XT>::store(sr + 4 * (lane + 32 * i), v[i]);
          // what the later passes normalise is the stored (rounded) sum
          Vec4<XT>::load(sr + 4 * (lane + 32 * i), v[i]);
        }
      }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      s += kRms ? (v[i][0] * v[i][0] + v[i][1] * v[i][1] + v[i][2] * v[i][2] + v[i][3] * v[i][3])
                : (v[i][0] + v[i][1] + v[i][2] + v[i][3]);
    s = warp_sum(s);
    float mean = 0.0f, rstd;
    if (kRms) {
      rstd = rsqrtf(s / kCols + eps);
    } else {
      mean = s / kCols;
      float var = 0.0f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) var += (v[i][j] - mean) * (v[i][j] - mean);
      }
      var = warp_sum(var);
      rstd = rsqrtf(var / kCols + eps);
    }
    if (lane == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
    YT* yr = y + static_cast<int64_t>(row) * kCols;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float o[4];
      if (!kRms && beta) {
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (v[i][j] - mean) * rstd * g[i][j] + b[i][j];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = (v[i][j] - mean) * rstd * g[i][j];
      }
      Vec4<YT>::store(yr + 4 * (lane + 32 * i), o);
    }
  }
}

// dx[row] = (add ? add[row] : 0) + rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat))        (LayerNorm)
// dx[row] = (add ? add[row] : 0) + rstd * (g*dy - xhat * mean(g*dy*xhat))                     (RMSNorm)
template <typename XT, typename PT, typename GT, typename DT, bool kRms>
__global__ void norm_bwd_dx_kernel(const GT* __restrict__ dy, const XT* __restrict__ x,
                                   const PT* __restrict__ gamma, const float* __restrict__ mean,
                                   const float* __restrict__ rstd, const DT* __restrict__ add, DT* __restrict__ dx,
                                   __nv_bfloat16* __restrict__ dx_lp, int rows, int cols) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = cols >> 2;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const XT* xr = x + static_cast<int64_t>(row) * cols;
    const GT* gr = dy + static_cast<int64_t>(row) * cols;
    const float mu = kRms ? 0.0f : mean[row];
    const float rs = rstd[row];
    float s1 = 0.0f, s2 = 0.0f;
    for (int i = lane; i < nvec; i += 32) {
      float v[4], d[4], g[4];
      Vec4<XT>::load(xr + 4 * i, v);
      Vec4<GT>::load(gr + 4 * i, d);
      Vec4<PT>::load(gamma + 4 * i, g);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gd = g[j] * d[j];
        s1 += gd;
        s2 += gd * (v[j] - mu) * rs;
      }
    }
    s1 = warp_sum(s1) / cols;
    s2 = warp_sum(s2) / cols;
    if (kRms) s1 = 0.0f;
    DT* dxr = dx + static_cast<int64_t>(row) * cols;
    const DT* ar = add ? add + static_cast<int64_t>(row) * cols : nullptr;
    for (int i = lane; i < nvec; i += 32) {
      float v[4], d[4], g[4], o[4];
      Vec4<XT>::load(xr + 4 * i, v);
      Vec4<GT>::load(gr + 4 * i, d);
      Vec4<PT>::load(gamma + 4 * i, g);
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = rs * (g[j] * d[j] - s1 - (v[j] - mu) * rs * s2);
      if (ar) {
        float a[4];
        Vec4<DT>::load(ar + 4 * i, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] += a[j];
      }
      Vec4<DT>::store(dxr + 4 * i, o);
      if (dx_lp) Vec4<__nv_bfloat16>::store(dx_lp + static_cast<int64_t>(row) * cols + 4 * i, o);
    }
  }
}

// Column partials: block (32 columns x 8 row lanes) covers one column strip and one row chunk.
// partial[chunk][0][c] = sum dy*xhat, partial[chunk][1][c] = sum dy, both in a fixed order.
template <typename XT, typename GT, bool kRms>
__global__ void norm_bwd_param_partial_kernel(const GT* __restrict__ dy, const XT* __restrict__ x,
                                              const float* __restrict__ mean, const float* __restrict__ rstd,
                                              float* __restrict__ partial, int rows, int cols,
                                              int rows_per_chunk) {
  __shared__ float sg[8][33];
  __shared__ float sb[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int chunk = blockIdx.y;
  const int r_begin = chunk * rows_per_chunk;
  const int r_end = min(rows, r_begin + rows_per_chunk);
  float ag = 0.0f, ab = 0.0f;
  if (c < cols) {
    for (int r = r_begin + threadIdx.y; r < r_end; r += 8) {
      const float d = Num<GT>::load(dy + static_cast<int64_t>(r) * cols + c);
      const float xv = Num<XT>::load(x + static_cast<int64_t>(r) * cols + c);
      const float xhat = (xv - (kRms ? 0.0f : mean[r])) * rstd[r];
      ag += d * xhat;
      ab += d;
    }
  }
  sg[threadIdx.y][threadIdx.x] = ag;
  sb[threadIdx.y][threadIdx.x] = ab;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float tg = 0.0f, tb = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tg += sg[k][threadIdx.x];
      tb += sb[k][threadIdx.x];
    }
    partial[(static_cast<int64_t>(chunk) * 2 + 0) * cols + c] = tg;
    partial[(static_cast<int64_t>(chunk) * 2 + 1) * cols + c] = tb;
  }
}

__global__ void norm_bwd_param_final_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                            float* __restrict__ dbeta, int cols, int chunks, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float tg = 0.0f, tb = 0.0f;
  for (int k = 0; k < chunks; ++k) {
    tg += partial[(static_cast<int64_t>(k) * 2 + 0) * cols + c];
    tb += partial[(static_cast<int64_t>(k) * 2 + 1) * cols + c];
  }
  if (dgamma) dgamma[c] = accumulate ? dgamma[c] + tg : tg;
  if (dbeta) dbeta[c] = accumulate ? dbeta[c] + tb : tb;
}

template <typename XT, typename PT, typename YT>
int launch_fwd(bool rms, const void* x, const void* res, void* sum_out, const void* gamma, const void* beta, void* y,
               float* mean, float* rstd, int rows, int cols, float eps, cudaStream_t st) {
  const int threads = 256, wpb = threads / 32;
  const int blocks = std::min((rows + wpb - 1) / wpb, kNumSmsB200 * 8);
  static const bool no_reg = std::getenv("NX_NORM_FWD_GENERIC") != nullptr;  // measurement switch
  if (!no_reg && cols % 128 == 0 && cols / 128 <= 8) {
#define NX_FWD_REG(V_)                                                                                                   \
  case V_:                                                                                                               \
    if (rms)                                                                                                             \
      norm_fwd_reg_kernel<XT, PT, YT, true, V_><<<blocks, threads, 0, st>>>(                                             \
          (const XT*)x, (const XT*)res, (XT*)sum_out, (const PT*)gamma, (const PT*)beta, (YT*)y, mean, rstd, rows, eps); \
    else                                                                                                                 \
      norm_fwd_reg_kernel<XT, PT, YT, false, V_><<<blocks, threads, 0, st>>>(                                            \
          (const XT*)x, (const XT*)res, (XT*)sum_out, (const PT*)gamma, (const PT*)beta, (YT*)y, mean, rstd, rows, eps); \
    return launch_status();
    switch (cols / 128) {
      NX_FWD_REG(1) NX_FWD_REG(2) NX_FWD_REG(3) NX_FWD_REG(4) NX_FWD_REG(5) NX_FWD_REG(6) NX_FWD_REG(7) NX_FWD_REG(8)
    }
#undef NX_FWD_REG
  }
  if (rms)
    norm_fwd_kernel<XT, PT, YT, true><<<blocks, threads, 0, st>>>(
        (const XT*)x, (const XT*)res, (XT*)sum_out, (const PT*)gamma, (const PT*)beta, (YT*)y, mean, rstd, rows, cols,
        eps);
  else
    norm_fwd_kernel<XT, PT, YT, false><<<blocks, threads, 0, st>>>(
        (const XT*)x, (const XT*)res, (XT*)sum_out, (const PT*)gamma, (const PT*)beta, (YT*)y, mean, rstd, rows, cols,
        eps);
  return launch_status();
}

template <typename XT, typename PT, typename GT, typename DT>
int launch_bwd_dx(bool rms, const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                  const void* add, void* dx, void* dx_lp, int rows, int cols, cudaStream_t st) {
  const int threads = 256, wpb = threads / 32;
  const int blocks = std::min((rows + wpb - 1) / wpb, kNumSmsB200 * 8);
  if (rms)
    norm_bwd_dx_kernel<XT, PT, GT, DT, true><<<blocks, threads, 0, st>>>(
        (const GT*)dy, (const XT*)x, (const PT*)gamma, mean, rstd, (const DT*)add, (DT*)dx, (__nv_bfloat16*)dx_lp, rows,
        cols);
  else
    norm_bwd_dx_kernel<XT, PT, GT, DT, false><<<blocks, threads, 0, st>>>(
        (const GT*)dy, (const XT*)x, (const PT*)gamma, mean, rstd, (const DT*)add, (DT*)dx, (__nv_bfloat16*)dx_lp, rows,
        cols);
  return launch_status();
}


// Fused backward for rows of 128*VPL columns: one pass over dy and x.  A warp keeps its row in
// registers (VPL float4 per lane), writes dx, and accumulates the column sums of dy*xhat and dy for its
// own columns over every row it owns; the block then folds its warps through shared memory (fixed
// order) into partial[block][2][cols].  Rows are assigned round-robin, so the result is deterministic.
// kSum: also accumulate the column sums of the BF16 copy of dx (partial[block][2][cols]): the bias gradient of the
// linear layer whose output gradient that copy is, without another pass over it.
template <typename XT, typename PT, typename GT, typename DT, bool kRms, int VPL, bool kSum>
__global__ void __launch_bounds__(256)
norm_bwd_fused_kernel(const GT* __restrict__ dy, const XT* __restrict__ x, const PT* __restrict__ gamma,
                      const float* __restrict__ mean, const float* __restrict__ rstd, const DT* __restrict__ add,
                      DT* __restrict__ dx, __nv_bfloat16* __restrict__ dx_lp, float* __restrict__ partial, int rows) {
  constexpr int kCols = 128 * VPL;
  constexpr int kParts = kSum ? 3 : 2;
  __shared__ float s_red[8][128];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float g[VPL][4], ag[VPL][4], ab[VPL][4], as[kSum ? VPL : 1][4];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    Vec4<PT>::load(gamma + 4 * (lane + 32 * i), g[i]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ag[i][j] = ab[i][j] = 0.0f;
      if (kSum) as[i][j] = 0.0f;
    }
  }
  // The loads of a warp's next row are issued before the arithmetic and the stores of the current one, so a warp
  // always has a row of x and dy in flight (the kernel runs one block of eight warps per SM).
  float xn[VPL][4], dn[VPL][4];
  float mu_n = 0.0f, rs_n = 0.0f;
  const int row_step = gridDim.x * 8;
  {
    const int row = blockIdx.x * 8 + warp;
    if (row < rows) {
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        Vec4<XT>::load(x + static_cast<int64_t>(row) * kCols + 4 * (lane + 32 * i), xn[i]);
        Vec4<GT>::load(dy + static_cast<int64_t>(row) * kCols + 4 * (lane + 32 * i), dn[i]);
      }
      mu_n = kRms ? 0.0f : mean[row];
      rs_n = rstd[row];
    }
  }
  for (int row = blockIdx.x * 8 + warp; row < rows; row += row_step) {
    const float mu = mu_n;
    const float rs = rs_n;
    float xh[VPL][4], d[VPL][4];
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[i][j] = xn[i][j];
        d[i][j] = dn[i][j];
      }
    }
    if (row + row_step < rows) {
      const int64_t nrow = row + row_step;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        Vec4<XT>::load(x + nrow * kCols + 4 * (lane + 32 * i), xn[i]);
        Vec4<GT>::load(dy + nrow * kCols + 4 * (lane + 32 * i), dn[i]);
      }
      mu_n = kRms ? 0.0f : mean[nrow];
      rs_n = rstd[nrow];
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xh[i][j] = (xh[i][j] - mu) * rs;
        const float gd = g[i][j] * d[i][j];
        s1 += gd;
        s2 += gd * xh[i][j];
        ag[i][j] += d[i][j] * xh[i][j];
        ab[i][j] += d[i][j];
      }
    }
    s1 = warp_sum(s1) / kCols;
    s2 = warp_sum(s2) / kCols;
    if (kRms) s1 = 0.0f;
    if (dx != nullptr) {
      DT* dxr = dx + static_cast<int64_t>(row) * kCols;
      const DT* ar = add ? add + static_cast<int64_t>(row) * kCols : nullptr;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        float o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = rs * (g[i][j] * d[i][j] - s1 - xh[i][j] * s2);
        if (ar) {
          float a[4];
          Vec4<DT>::load(ar + 4 * (lane + 32 * i), a);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] += a[j];
        }
        Vec4<DT>::store(dxr + 4 * (lane + 32 * i), o);
        if (dx_lp) Vec4<__nv_bfloat16>::store(dx_lp + static_cast<int64_t>(row) * kCols + 4 * (lane + 32 * i), o);
        if (kSum) {
#pragma unroll
          for (int j = 0; j < 4; ++j) as[i][j] += __bfloat162float(__float2bfloat16_rn(o[j]));  // what the copy holds
        }
      }
    }
  }
  if (partial == nullptr) return;
  float* out = partial + static_cast<int64_t>(blockIdx.x) * kParts * kCols;
#pragma unroll 1
  for (int which = 0; which < kParts; ++which) {
#pragma unroll 1
    for (int i = 0; i < VPL; ++i) {
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 4; ++j)
        s_red[warp][lane * 4 + j] = which == 0 ? ag[i][j] : (which == 1 ? ab[i][j] : as[kSum ? i : 0][j]);
      __syncthreads();
      if (threadIdx.x < 128) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += s_red[w][threadIdx.x];
        out[which * kCols + 128 * i + threadIdx.x] = t;
      }
    }
  }
}

// dgamma / dbeta (/ dsum) = sum over chunks of partial[chunk][0/1(/2)][c]; block (32 columns x 8 chunk lanes).
__global__ void norm_bwd_param_final2_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                             float* __restrict__ dbeta, float* __restrict__ dsum, int parts, int cols,
                                             int chunks, int accumulate) {
  pdl_trigger();
  __shared__ float sg[8][33];
  __shared__ float sb[8][33];
  __shared__ float ss[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float tg = 0.0f, tb = 0.0f, ts = 0.0f;
  if (c < cols) {
    for (int k = threadIdx.y; k < chunks; k += 8) {
      tg += partial[(static_cast<int64_t>(k) * parts + 0) * cols + c];
      tb += partial[(static_cast<int64_t>(k) * parts + 1) * cols + c];
      if (parts == 3) ts += partial[(static_cast<int64_t>(k) * parts + 2) * cols + c];
    }
  }
  sg[threadIdx.y][threadIdx.x] = tg;
  sb[threadIdx.y][threadIdx.x] = tb;
  ss[threadIdx.y][threadIdx.x] = ts;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    tg = tb = ts = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tg += sg[k][threadIdx.x];
      tb += sb[k][threadIdx.x];
      ts += ss[k][threadIdx.x];
    }
    if (dgamma) dgamma[c] = accumulate ? dgamma[c] + tg : tg;
    if (dbeta) dbeta[c] = accumulate ? dbeta[c] + tb : tb;
    if (dsum && parts == 3) dsum[c] = accumulate ? dsum[c] + ts : ts;
  }
}

constexpr int kFusedBwdBlocks = kNumSmsB200 * 2;

template <typename XT, typename PT, typename GT, typename DT, int VPL>
int launch_bwd_fused_v(bool rms, const void* dy, const void* x, const void* gamma, const float* mean,
                       const float* rstd, const void* add, void* dx, void* dx_lp, float* partial, int rows,
                       bool colsum, cudaStream_t st) {
  const int blocks = std::min(kFusedBwdBlocks, (rows + 7) / 8);
#define NX_K(RMS, SUM)                                                                                              \
  norm_bwd_fused_kernel<XT, PT, GT, DT, RMS, VPL, SUM><<<blocks, 256, 0, st>>>(                                       \
      (const GT*)dy, (const XT*)x, (const PT*)gamma, mean, rstd, (const DT*)add, (DT*)dx, (__nv_bfloat16*)dx_lp, \
      partial, rows)
  if (rms) {
    if (colsum) NX_K(true, true);
    else NX_K(true, false);
  } else {
    if (colsum) NX_K(false, true);
    else NX_K(false, false);
  }
#undef NX_K
  return launch_status() != 0 ? -2 : blocks;
}

// Returns the number of partial chunks written (> 0), 0 when the shape has no fused instance, < 0 on error.
template <typename XT, typename PT, typename GT, typename DT>
int launch_bwd_fused(bool rms, const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                     const void* add, void* dx, void* dx_lp, float* partial, int rows, int cols, bool colsum,
                     cudaStream_t st) {
#define NX_V(V) case V: return launch_bwd_fused_v<XT, PT, GT, DT, V>(rms, dy, x, gamma, mean, rstd, add, dx, dx_lp, partial, rows, colsum, st)
  if (cols % 128) return 0;
  switch (cols / 128) {
    NX_V(2); NX_V(4); NX_V(6); NX_V(8);
    default: return 0;
  }
#undef NX_V
}

}  // namespace

#include <algorithm>

extern "C" int nx_norm_fwd(int rms, const void* x, int x_dtype, const void* residual, void* sum_out,
                           const void* gamma, const void* beta, int param_dtype, void* y, int y_dtype, float* mean,
                           float* rstd, int rows, int cols, float eps, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 3)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool r = rms != 0;
#define NX_FWD(XT, PT, YT) \
  return launch_fwd<XT, PT, YT>(r, x, residual, sum_out, gamma, beta, y, mean, rstd, rows, cols, eps, st)
  if (x_dtype == NX_F32 && param_dtype == NX_F32 && y_dtype == NX_BF16) NX_FWD(float, float, __nv_bfloat16);
  if (x_dtype == NX_F32 && param_dtype == NX_F32 && y_dtype == NX_F32) NX_FWD(float, float, float);
  if (x_dtype == NX_BF16 && param_dtype == NX_F32 && y_dtype == NX_BF16) NX_FWD(__nv_bfloat16, float, __nv_bfloat16);
  if (x_dtype == NX_BF16 && param_dtype == NX_BF16 && y_dtype == NX_BF16)
    NX_FWD(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  if (x_dtype == NX_F32 && param_dtype == NX_BF16 && y_dtype == NX_BF16) NX_FWD(float, __nv_bfloat16, __nv_bfloat16);
#undef NX_FWD
  return -1;
}

static size_t nx_norm_bwd_partial_floats(int rows, int cols) {
  const int chunks = std::max(kFusedBwdBlocks, std::max(1, std::min(64, (rows + 255) / 256)));
  return static_cast<size_t>(chunks) * 3 * cols;
}

extern "C" size_t nx_norm_bwd_scratch_bytes(int rows, int cols) {
  return nx_norm_bwd_partial_floats(rows, cols) * sizeof(float);
}

extern "C" int nx_norm_bwd(int rms, const void* dy, int dy_dtype, const void* x, int x_dtype, const void* gamma,
                           int param_dtype, const float* mean, const float* rstd, const void* add, void* dx,
                           int dx_dtype, void* dx_lp, float* dgamma, float* dbeta, int accumulate_params,
                           float* scratch, int rows, int cols, nx_stream_t stream) {
  return nx_norm_bwd_colsum(rms, dy, dy_dtype, x, x_dtype, gamma, param_dtype, mean, rstd, add, dx, dx_dtype, dx_lp, dgamma,
                            dbeta, nullptr, accumulate_params, scratch, rows, cols, stream);
}

// `dx_colsum` (optional, [cols]): column sums of the BF16 copy `dx_lp`, accumulated like dgamma / dbeta.  Only the
// single-pass instances produce it; returns -4 when the shape or the types have none.
extern "C" int nx_norm_bwd_colsum(int rms, const void* dy, int dy_dtype, const void* x, int x_dtype, const void* gamma,
                                  int param_dtype, const float* mean, const float* rstd, const void* add, void* dx,
                                  int dx_dtype, void* dx_lp, float* dgamma, float* dbeta, float* dx_colsum,
                                  int accumulate_params, float* scratch, int rows, int cols, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 3)) return -1;
  if (dx_colsum != nullptr && (dx == nullptr || dx_lp == nullptr)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool r = rms != 0;
  int rc = -1;
  const bool want_params = dgamma != nullptr || dbeta != nullptr || dx_colsum != nullptr;
  if (want_params && scratch == nullptr) return -1;
  {  // single-pass path (dx and the parameter partials from one read of dy and x)
    int chunks = 0;
#define NX_FUSED(XT, PT, GT, DT) \
  chunks = launch_bwd_fused<XT, PT, GT, DT>(r, dy, x, gamma, mean, rstd, add, dx, dx_lp, want_params ? scratch : nullptr, rows, cols, dx_colsum != nullptr, st)
    if (x_dtype == NX_F32 && param_dtype == NX_F32 && dy_dtype == NX_BF16 && (dx == nullptr || dx_dtype == NX_F32))
      NX_FUSED(float, float, __nv_bfloat16, float);
    else if (x_dtype == NX_BF16 && param_dtype == NX_F32 && dy_dtype == NX_BF16 && (dx == nullptr || dx_dtype == NX_BF16))
      NX_FUSED(__nv_bfloat16, float, __nv_bfloat16, __nv_bfloat16);
#undef NX_FUSED
    if (chunks < 0) return chunks;
    if (chunks > 0) {
      if (!want_params) return 0;
      dim3 grid2((cols + 31) / 32), block2(32, 8);
      norm_bwd_param_final2_kernel<<<grid2, block2, 0, st>>>(scratch, dgamma, dbeta, dx_colsum, dx_colsum ? 3 : 2, cols,
                                                             chunks, accumulate_params);
      return launch_status();
    }
  }
  if (dx_colsum != nullptr) return -4;
#define NX_BWD(XT, PT, GT, DT) rc = launch_bwd_dx<XT, PT, GT, DT>(r, dy, x, gamma, mean, rstd, add, dx, dx_lp, rows, cols, st)
  if (dx != nullptr) {
    if (x_dtype == NX_F32 && param_dtype == NX_F32 && dy_dtype == NX_BF16 && dx_dtype == NX_F32)
      NX_BWD(float, float, __nv_bfloat16, float);
    else if (x_dtype == NX_F32 && param_dtype == NX_F32 && dy_dtype == NX_F32 && dx_dtype == NX_F32)
      NX_BWD(float, float, float, float);
    else if (x_dtype == NX_BF16 && param_dtype == NX_F32 && dy_dtype == NX_BF16 && dx_dtype == NX_BF16)
      NX_BWD(__nv_bfloat16, float, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == NX_BF16 && param_dtype == NX_BF16 && dy_dtype == NX_BF16 && dx_dtype == NX_BF16)
      NX_BWD(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == NX_F32 && param_dtype == NX_BF16 && dy_dtype == NX_BF16 && dx_dtype == NX_F32)
      NX_BWD(float, __nv_bfloat16, __nv_bfloat16, float);
    else
      return -1;
    if (rc != 0) return rc;
  }
#undef NX_BWD
  if (dgamma == nullptr && dbeta == nullptr) return 0;
  if (scratch == nullptr) return -1;
  const int chunks = std::max(1, std::min(64, (rows + 255) / 256));
  const int rows_per_chunk = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 31) / 32, chunks), block(32, 8);
#define NX_PP(XT, GT)                                                                                     \
  do {                                                                                                    \
    if (r)                                                                                                \
      norm_bwd_param_partial_kernel<XT, GT, true><<<grid, block, 0, st>>>((const GT*)dy, (const XT*)x, mean, rstd, \
                                                                         scratch, rows, cols, rows_per_chunk);     \
    else                                                                                                  \
      norm_bwd_param_partial_kernel<XT, GT, false><<<grid, block, 0, st>>>((const GT*)dy, (const XT*)x, mean, rstd, \
                                                                          scratch, rows, cols, rows_per_chunk);    \
  } while (0)
  if (x_dtype == NX_F32 && dy_dtype == NX_BF16) NX_PP(float, __nv_bfloat16);
  else if (x_dtype == NX_F32 && dy_dtype == NX_F32) NX_PP(float, float);
  else if (x_dtype == NX_BF16 && dy_dtype == NX_BF16) NX_PP(__nv_bfloat16, __nv_bfloat16);
  else return -1;
#undef NX_PP
  if (launch_status() != 0) return -2;
  norm_bwd_param_final_kernel<<<(cols + 255) / 256, 256, 0, st>>>(scratch, dgamma, dbeta, cols, chunks,
                                                                  accumulate_params);
  return launch_status();
}
