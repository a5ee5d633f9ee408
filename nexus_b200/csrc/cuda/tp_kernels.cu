// Memory-bound kernels of the tensor-parallel language-model path (see nx_api_tp.h): vocabulary-parallel embedding
// by peer loads, its gradient, and the local halves of the vocabulary-parallel cross-entropy.  The statistics
// exchange between the two CE halves is nx_vocab_ce_exchange (comm_kernels.cu).
#include <algorithm>

#include "common.cuh"
#include "nx_api_tp.h"

namespace {
using namespace nx;

__global__ void __launch_bounds__(128)
tp_embed_gather_kernel(const int32_t* __restrict__ tokens, NxPeerTable tables, int n_ranks, int v_per, int d,
                       float* __restrict__ out, int rows) {
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int tok = tokens[r];
    int owner = tok / v_per;
    if (tok < 0 || owner >= n_ranks) {  // out-of-range id: a zero row, like a padding entry
      for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4)
        *reinterpret_cast<float4*>(out + static_cast<int64_t>(r) * d + c) = make_float4(0.f, 0.f, 0.f, 0.f);
      continue;
    }
    const __nv_bfloat16* src =
        reinterpret_cast<const __nv_bfloat16*>(tables.ptr[owner]) + static_cast<int64_t>(tok - owner * v_per) * d;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float4 lo, hi;
      float2 f = __bfloat1622float2(h[0]); lo.x = f.x; lo.y = f.y;
      f = __bfloat1622float2(h[1]); lo.z = f.x; lo.w = f.y;
      f = __bfloat1622float2(h[2]); hi.x = f.x; hi.y = f.y;
      f = __bfloat1622float2(h[3]); hi.z = f.x; hi.w = f.y;
      float* dst = out + static_cast<int64_t>(r) * d + c;
      *reinterpret_cast<float4*>(dst) = lo;
      *reinterpret_cast<float4*>(dst + 4) = hi;
    }
  }
}

__global__ void __launch_bounds__(128)
tp_embed_bwd_kernel(const int32_t* __restrict__ tokens_all, int total, NxPeerTable dh, int rows_per_rank, int v0,
                    int v_per, int d, float* __restrict__ dtable) {
  for (int i = blockIdx.x; i < total; i += gridDim.x) {
    const int tok = tokens_all[i];
    if (tok < v0 || tok >= v0 + v_per) continue;
    const int owner = i / rows_per_rank;
    const __nv_bfloat16* src =
        reinterpret_cast<const __nv_bfloat16*>(dh.ptr[owner]) + static_cast<int64_t>(i - owner * rows_per_rank) * d;
    float* dst = dtable + static_cast<int64_t>(tok - v0) * d;
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        atomicAdd(dst + c + 2 * j, f.x);
        atomicAdd(dst + c + 2 * j + 1, f.y);
      }
    }
  }
}

// One block per row; single read of the row: online (max, sum-exp).
__global__ void __launch_bounds__(256)
tp_ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, int64_t ld, int rows, int cols,
                   const int32_t* __restrict__ targets, int v0, float* __restrict__ stats) {
  __shared__ float s_scratch[32];
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const __nv_bfloat16* row = logits + static_cast<int64_t>(r) * ld;
    float m = -INFINITY, s = 0.0f;
    const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    if (vec) {
      const int nv = cols / 8;
      for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + i * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
        float v[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          v[2 * j] = f.x;
          v[2 * j + 1] = f.y;
        }
        float lm = v[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) lm = fmaxf(lm, v[j]);
        if (lm > m) {
          s *= __expf(m - lm);
          m = lm;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) s += __expf(v[j] - m);
      }
      for (int c = nv * 8 + threadIdx.x; c < cols; c += blockDim.x) {
        const float v = __bfloat162float(row[c]);
        if (v > m) {
          s *= __expf(m - v);
          m = v;
        }
        s += __expf(v - m);
      }
    } else {
      for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = __bfloat162float(row[c]);
        if (v > m) {
          s *= __expf(m - v);
          m = v;
        }
        s += __expf(v - m);
      }
    }
    const float gm = block_max(m, s_scratch);
    const float contrib = (m == -INFINITY) ? 0.0f : s * __expf(m - gm);
    const float gs = block_sum<float>(contrib, s_scratch);
    if (threadIdx.x == 0) {
      const int t = targets[r] - v0;
      stats[r * 3] = gm;
      stats[r * 3 + 1] = gs;
      stats[r * 3 + 2] = (targets[r] >= 0 && t >= 0 && t < cols) ? __bfloat162float(row[t]) : 0.0f;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
tp_ce_grad_kernel(__nv_bfloat16* __restrict__ logits, int64_t ld, int rows, int cols,
                  const int32_t* __restrict__ targets, int v0, const float* __restrict__ merged,
                  const float* __restrict__ scale_p) {
  const float scale = *scale_p;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    __nv_bfloat16* row = logits + static_cast<int64_t>(r) * ld;
    const int tg = targets[r];
    const bool valid = tg >= 0;
    const float lse = merged[r * 3] + __logf(merged[r * 3 + 1]);
    const int t = tg - v0;
    const bool vec = ((ld & 7) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
    const int nv = vec ? cols / 8 : 0;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      uint4 raw = *reinterpret_cast<const uint4*>(row + i * 8);
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        const int c = i * 8 + 2 * j;
        f.x = valid ? (__expf(f.x - lse) - (c == t ? 1.0f : 0.0f)) * scale : 0.0f;
        f.y = valid ? (__expf(f.y - lse) - (c + 1 == t ? 1.0f : 0.0f)) * scale : 0.0f;
        h[j] = __floats2bfloat162_rn(f.x, f.y);
      }
      *reinterpret_cast<uint4*>(row + i * 8) = raw;
    }
    for (int c = nv * 8 + threadIdx.x; c < cols; c += blockDim.x) {
      const float v = __bfloat162float(row[c]);
      row[c] = __float2bfloat16_rn(valid ? (__expf(v - lse) - (c == t ? 1.0f : 0.0f)) * scale : 0.0f);
    }
  }
}

__global__ void __launch_bounds__(1024)
tp_ce_loss_kernel(const float* __restrict__ merged, const int32_t* __restrict__ targets, int rows, float inv_valid,
                  float weight, int accumulate, float* __restrict__ loss_out) {
  __shared__ double s_scratch[32];
  double acc = 0.0;
  for (int r = threadIdx.x; r < rows; r += blockDim.x)
    if (targets[r] >= 0) acc += static_cast<double>(merged[r * 3] + __logf(merged[r * 3 + 1]) - merged[r * 3 + 2]);
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) {
    const float v = static_cast<float>(acc * inv_valid) * weight;
    *loss_out = accumulate ? *loss_out + v : v;
  }
}

}  // namespace

extern "C" int nx_tp_embed_gather(const int32_t* tokens, const NxPeerTable* tables, int n_ranks, int v_per, int d,
                                  float* out, int rows, nx_stream_t stream) {
  if (tokens == nullptr || tables == nullptr || out == nullptr || n_ranks < 1 || n_ranks > NX_MAX_PEERS || v_per <= 0 ||
      d <= 0 || (d & 7) || rows <= 0)
    return -1;
  tp_embed_gather_kernel<<<std::min(rows, 148 * 16), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens, *tables, n_ranks, v_per, d, out, rows);
  return launch_status();
}

extern "C" int nx_tp_embed_bwd(const int32_t* tokens_all, int total, const NxPeerTable* dh, int rows_per_rank, int v0,
                               int v_per, int d, float* dtable, nx_stream_t stream) {
  if (tokens_all == nullptr || dh == nullptr || dtable == nullptr || total <= 0 || rows_per_rank <= 0 || v_per <= 0 ||
      d <= 0 || (d & 7))
    return -1;
  tp_embed_bwd_kernel<<<std::min(total, 148 * 16), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      tokens_all, total, *dh, rows_per_rank, v0, v_per, d, dtable);
  return launch_status();
}

extern "C" int nx_tp_ce_stats(const void* logits, int64_t ld, int rows, int cols, const int32_t* targets, int v0,
                              float* stats, nx_stream_t stream) {
  if (logits == nullptr || targets == nullptr || stats == nullptr || rows <= 0 || cols <= 0 || ld < cols) return -1;
  tp_ce_stats_kernel<<<std::min(rows, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, rows, cols, targets, v0, stats);
  return launch_status();
}

extern "C" int nx_tp_ce_grad(void* logits, int64_t ld, int rows, int cols, const int32_t* targets, int v0,
                             const float* merged, const float* scale, nx_stream_t stream) {
  if (logits == nullptr || targets == nullptr || merged == nullptr || scale == nullptr || rows <= 0 || cols <= 0 ||
      ld < cols)
    return -1;
  tp_ce_grad_kernel<<<std::min(rows, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(logits), ld, rows, cols, targets, v0, merged, scale);
  return launch_status();
}

extern "C" int nx_tp_ce_loss(const float* merged, const int32_t* targets, int rows, float inv_valid, float weight,
                             int accumulate, float* loss_out, nx_stream_t stream) {
  if (merged == nullptr || targets == nullptr || loss_out == nullptr || rows <= 0) return -1;
  tp_ce_loss_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(merged, targets, rows, inv_valid, weight,
                                                                        accumulate, loss_out);
  return launch_status();
}
