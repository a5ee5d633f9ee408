// Inference kernels: paged KV cache append (BF16 / INT8 / FP8-E4M3 with per-(slot, head) scales), paged
// attention for decode with split-KV and a combine pass, skinny GEMM for small batches (result of a
// row does not depend on the batch it is in), row gather, single-kernel sampler (repetition /
// frequency / presence penalties, temperature, top-k, top-p, min-p, Philox draw, greedy ties ->
// lowest id), token counting, NLL, RoPE (rotate-half and interleaved), SwiGLU / GeGLU forward and
// backward, weight-only INT8 / INT4 (group-wise) GEMV and dequantisation, activation row quantisation.
// Parity: src/cuda/infer_kernels.cu:49-571 and src/cuda/kernels_lm.cu:28-183 of the reference.
#include "common.cuh"
#include "nx_api_infer.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"
#include <cstdlib>

#include <cuda_fp8.h>

namespace {
using namespace nx;

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  unpack_bf16x2(q.x, v[0], v[1]);
  unpack_bf16x2(q.y, v[2], v[3]);
  unpack_bf16x2(q.z, v[4], v[5]);
  unpack_bf16x2(q.w, v[6], v[7]);
}

// ------------------------------------------------------------------------------------------------
// KV append: new K/V rows [tokens, Hkv, D] scattered to cache slot (block * block_size + offset)
// ------------------------------------------------------------------------------------------------
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 int64_t k_row_stride, int64_t v_row_stride, const int32_t* __restrict__ slots,
                                 __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc, int tokens, int hd) {
  const int vec = hd >> 3;  // Hkv*D in 16-byte vectors
  NX_GRID_STRIDE(i, static_cast<int64_t>(tokens) * vec) {
    const int t = static_cast<int>(i / vec), c = static_cast<int>(i % vec);
    const int64_t s = slots[t];
    if (s < 0) continue;
    reinterpret_cast<uint4*>(kc + s * hd)[c] = reinterpret_cast<const uint4*>(k + t * k_row_stride)[c];
    reinterpret_cast<uint4*>(vc + s * hd)[c] = reinterpret_cast<const uint4*>(v + t * v_row_stride)[c];
  }
}

// 8-bit cache: one warp per (token, head); scale = amax / qmax stored per (slot, head).
template <bool kFp8>
__global__ void kv_append_q8_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                    int64_t k_row_stride, int64_t v_row_stride, const int32_t* __restrict__ slots,
                                    uint8_t* __restrict__ kc, uint8_t* __restrict__ vc, float* __restrict__ kscale,
                                    float* __restrict__ vscale, int tokens, int heads, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens * heads) return;
  const int t = warp / heads, h = warp % heads;
  const int64_t s = slots[t];
  if (s < 0) return;
  const float qmax = kFp8 ? 448.0f : 127.0f;
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* src = (which ? v + t * v_row_stride : k + t * k_row_stride) + h * D;
    float amax = 0.0f;
    for (int d = lane; d < D; d += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[d])));
    amax = warp_max(amax);
    const float scale = amax > 0.0f ? amax / qmax : 1.0f;
    uint8_t* dst = (which ? vc : kc) + (s * heads + h) * D;
    for (int d = lane; d < D; d += 32) {
      const float x = __bfloat162float(src[d]) / scale;
      if (kFp8) {
        dst[d] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
      } else {
        dst[d] = static_cast<uint8_t>(static_cast<int8_t>(max(-127, min(127, __float2int_rn(x)))));
      }
    }
    if (lane == 0) (which ? vscale : kscale)[s * heads + h] = scale;
  }
}

__device__ __forceinline__ float fp8_e4m3_to_float(uint8_t b) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// ------------------------------------------------------------------------------------------------
// paged attention, decode: grid (rows, heads, splits), 128 threads.  LPT = lanes per token
// (head_dim / 8): each lane group scores one cached token per step with 16-byte loads.
// kv_kind: 0 BF16, 1 INT8, 2 FP8-E4M3 (8-bit kinds: per-(slot, head) scales).
// ------------------------------------------------------------------------------------------------
template <int D, int KV>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int64_t q_row_stride, const void* __restrict__ kc,
                    const void* __restrict__ vc, const float* __restrict__ kscale, const float* __restrict__ vscale,
                    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ row_seq,
                    const int32_t* __restrict__ ctx_len, int block_size, int heads, int kv_heads, float scale,
                    int splits, __nv_bfloat16* __restrict__ out, int64_t o_row_stride, float* __restrict__ part_o,
                    float* __restrict__ part_ml) {
  constexpr int LPT = D / 8;        // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  // heads vary fastest over the grid: the blocks that run together read the adjacent head rows of the same cached
  // tokens (one token's K or V row is [kv_heads][D] contiguous), which keeps their DRAM bursts in the same pages
  const int h = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const int hk = h / (heads / kv_heads);
  const int seq = row_seq[row];
  const int ctx = ctx_len[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPT, sub = lane % LPT;
  const int per = (ctx + splits - 1) / splits;
  const int t_begin = split * per, t_end = min(ctx, t_begin + per);
  float qv[8];
  unpack8(*reinterpret_cast<const uint4*>(q + row * q_row_stride + h * D + sub * 8), qv);
#pragma unroll
  for (int j = 0; j < 8; ++j) qv[j] *= scale * 1.4426950408889634f;
  float m = -INFINITY, l = 0.0f, acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  const int32_t* bt = block_table + static_cast<int64_t>(seq) * max_blocks;
  // The loop bound is warp-uniform: the shuffles below need every lane of the warp.  Each trip takes kU tokens per
  // lane group: their block-table entries, then all their K and V loads, are issued before any arithmetic, so a lane
  // keeps 2 * kU loads in flight (the kernel is bound by KV bytes), and the running maximum is updated once per trip.
  constexpr int kU = 4;
  for (int tb = t_begin + warp * TPW; tb < t_end; tb += 4 * TPW * kU) {
    bool valid[kU];
    int64_t slot[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int tt = tb + u * 4 * TPW + grp;
      valid[u] = tt < t_end;
      const int t = valid[u] ? tt : t_end - 1;
      slot[u] = static_cast<int64_t>(bt[t / block_size]) * block_size + t % block_size;
    }
    uint4 kr[kU], vr[kU];     // BF16: 8 values; 8-bit kinds: the low 8 bytes are used
    float ks[kU], vs[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int64_t base = (slot[u] * kv_heads + hk) * D + sub * 8;
      if (KV == 0) {
        kr[u] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(kc) + base);
        vr[u] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(vc) + base);
      } else {
        const uint2 kq = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(kc) + base);
        const uint2 vq = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(vc) + base);
        kr[u] = make_uint4(kq.x, kq.y, 0u, 0u);
        vr[u] = make_uint4(vq.x, vq.y, 0u, 0u);
        ks[u] = kscale[slot[u] * kv_heads + hk];
        vs[u] = vscale[slot[u] * kv_heads + hk];
      }
    }
    float sc[kU];
    float mn = m;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      float kv[8];
      if (KV == 0) {
        unpack8(kr[u], kv);
      } else {
        const uint8_t* kb = reinterpret_cast<const uint8_t*>(&kr[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          kv[j] = (KV == 1 ? static_cast<float>(static_cast<int8_t>(kb[j])) : fp8_e4m3_to_float(kb[j])) * ks[u];
      }
      float t = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += qv[j] * kv[j];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      sc[u] = t;
      if (valid[u]) mn = fmaxf(mn, t);
    }
    if (mn == -INFINITY) continue;  // nothing valid for this lane group yet
    const float alpha = exp2f(m - mn);
    l *= alpha;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= alpha;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      if (!valid[u]) continue;
      float vv[8];
      if (KV == 0) {
        unpack8(vr[u], vv);
      } else {
        const uint8_t* vb = reinterpret_cast<const uint8_t*>(&vr[u]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          vv[j] = (KV == 1 ? static_cast<float>(static_cast<int8_t>(vb[j])) : fp8_e4m3_to_float(vb[j])) * vs[u];
      }
      const float pw = exp2f(sc[u] - mn);
      l += pw;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += pw * vv[j];
    }
    m = mn;
  }
  // merge the token groups of the warp, then the warps of the block
  __shared__ float s_m[4 * 8], s_l[4 * 8], s_acc[4 * 8][D];
  const int slot_id = warp * TPW + grp;
  if (sub == 0) {
    s_m[slot_id] = m;
    s_l[slot_id] = l;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_acc[slot_id][sub * 8 + j] = acc[j];
  __syncthreads();
  if (threadIdx.x < D) {
    const int d = threadIdx.x;
    float gm = -INFINITY;
    for (int i = 0; i < 4 * TPW; ++i) gm = fmaxf(gm, s_m[i]);
    float gl = 0.0f, go = 0.0f;
    for (int i = 0; i < 4 * TPW; ++i) {
      const float w = (s_m[i] == -INFINITY) ? 0.0f : exp2f(s_m[i] - gm);
      gl += s_l[i] * w;
      go += s_acc[i][d] * w;
    }
    if (splits == 1) {
      out[row * o_row_stride + h * D + d] = __float2bfloat16_rn(gl > 0.0f ? go / gl : 0.0f);
    } else {
      const int64_t pi = (static_cast<int64_t>(row) * heads + h) * splits + split;
      part_o[pi * D + d] = go;
      if (d == 0) {
        part_ml[pi * 2] = gm;
        part_ml[pi * 2 + 1] = gl;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// paged attention, decode, BF16 cache with 16-token pages: the K and V page of a head ([16][D], rows
// kv_heads * D apart) arrive by one tiled TMA copy each into a ring of kStages shared-memory stages,
// issued by one thread as soon as a stage has been consumed; with several resident CTAs an SM keeps
// 100-200 KiB of cache reads in flight, which is what a bandwidth-bound kernel needs.  Scoring and
// the running softmax are those of the kernel above: 128 threads, D / 8 lanes per cached token,
// every lane group keeps its own (max, sum, 8 output columns) and the groups merge at the end.
// grid (heads, rows, splits).
// ------------------------------------------------------------------------------------------------
constexpr int kPagedStages = 6;
constexpr int kPagedWaitStatus = 7;  // status-word value: a page did not arrive within the wait limit

template <int D>
__global__ void __launch_bounds__(128)
paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                        const __nv_bfloat16* __restrict__ q, int64_t q_row_stride,
                        const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ row_seq,
                        const int32_t* __restrict__ ctx_len, int heads, int kv_heads, float scale, int splits,
                        __nv_bfloat16* __restrict__ out, int64_t o_row_stride, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int* __restrict__ status) {
  constexpr int LPT = D / 8;          // lanes per token
  constexpr int TPP = 128 / LPT;      // tokens per pass of the block (16 at D = 64, 8 at D = 128)
  constexpr int kPage = 16;
  constexpr int kPageBytes = kPage * D * 2;
  extern __shared__ __align__(128) uint8_t pd_smem[];
  uint8_t* sK = pd_smem;                               // [kStages][16][D]
  uint8_t* sV = sK + kPagedStages * kPageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(sV + kPagedStages * kPageBytes);
  __shared__ int s_abort;
  const int h = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const int hk = h / (heads / kv_heads);
  const int seq = row_seq[row];
  const int ctx = ctx_len[row];
  const int tid = threadIdx.x;
  const int grp = tid / LPT, sub = tid % LPT;
  const int per = (ctx + splits - 1) / splits;
  const int t_begin = split * per, t_end = min(ctx, t_begin + per);
  const int p_begin = t_begin / kPage, p_end = t_end > t_begin ? (t_end + kPage - 1) / kPage : p_begin;
  const int32_t* bt = block_table + static_cast<int64_t>(seq) * max_blocks;
  if (tid == 0) {
    for (int s = 0; s < kPagedStages; ++s) nx::mbar_init(&full[s], 1);
    s_abort = 0;
    nx::fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int page) {   // thread 0: K and V page `page` of this head into stage (page - p_begin) % kStages
    const int s = (page - p_begin) % kPagedStages;
    const int blk = bt[page];
    nx::mbar_arrive_expect_tx(&full[s], 2 * kPageBytes);
    nx::tma_load_3d(sK + s * kPageBytes, &tm_k, &full[s], hk * D, blk * kPage, 0);
    nx::tma_load_3d(sV + s * kPageBytes, &tm_v, &full[s], hk * D, blk * kPage, 0);
  };
  if (tid == 0)
    for (int pg = p_begin; pg < min(p_end, p_begin + kPagedStages); ++pg) issue(pg);
  float qv[8];
  unpack8(*reinterpret_cast<const uint4*>(q + row * q_row_stride + h * D + sub * 8), qv);
#pragma unroll
  for (int j = 0; j < 8; ++j) qv[j] *= scale * 1.4426950408889634f;
  float m = -INFINITY, l = 0.0f, acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  for (int pg = p_begin; pg < p_end; ++pg) {
    const int n = pg - p_begin;
    const int s = n % kPagedStages;
    const bool arrived = nx::mbar_wait_bounded(&full[s], (n / kPagedStages) & 1, &s_abort);
    if (!arrived) atomicCAS(status, 0, kPagedWaitStatus);
#pragma unroll
    for (int pass = 0; arrived && pass < kPage / TPP; ++pass) {
      const int tok = pg * kPage + pass * TPP + grp;
      const bool valid = tok >= t_begin && tok < t_end;
      float kv[8], vv[8];
      unpack8(*reinterpret_cast<const uint4*>(sK + s * kPageBytes + ((pass * TPP + grp) * D + sub * 8) * 2), kv);
      unpack8(*reinterpret_cast<const uint4*>(sV + s * kPageBytes + ((pass * TPP + grp) * D + sub * 8) * 2), vv);
      float t = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) t += qv[j] * kv[j];
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (valid) {
        const float mn = fmaxf(m, t);
        const float alpha = exp2f(m - mn);   // m == -inf: 0
        const float pw = exp2f(t - mn);
        l = l * alpha + pw;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = acc[j] * alpha + pw * vv[j];
        m = mn;
      }
    }
    // every thread has read stage s; a page that did not arrive ends the loop for the whole block (status is set)
    if (__syncthreads_or(arrived ? 0 : 1)) break;
    if (tid == 0 && pg + kPagedStages < p_end) issue(pg + kPagedStages);
  }
  // merge the lane groups of the block
  __shared__ float s_m[TPP], s_l[TPP], s_acc[TPP][D];
  if (sub == 0) {
    s_m[grp] = m;
    s_l[grp] = l;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_acc[grp][sub * 8 + j] = acc[j];
  __syncthreads();
  if (tid < D) {
    const int d = tid;
    float gm = -INFINITY;
    for (int i = 0; i < TPP; ++i) gm = fmaxf(gm, s_m[i]);
    float gl = 0.0f, go = 0.0f;
    for (int i = 0; i < TPP; ++i) {
      const float w = (s_m[i] == -INFINITY) ? 0.0f : exp2f(s_m[i] - gm);
      gl += s_l[i] * w;
      go += s_acc[i][d] * w;
    }
    if (splits == 1) {
      out[row * o_row_stride + h * D + d] = __float2bfloat16_rn(gl > 0.0f ? go / gl : 0.0f);
    } else {
      const int64_t pi = (static_cast<int64_t>(row) * heads + h) * splits + split;
      part_o[pi * D + d] = go;
      if (d == 0) {
        part_ml[pi * 2] = gm;
        part_ml[pi * 2 + 1] = gl;
      }
    }
  }
}

template <int D>
__global__ void paged_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int splits,
                                     int heads, __nv_bfloat16* __restrict__ out, int64_t o_row_stride) {
  const int row = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int64_t base = (static_cast<int64_t>(row) * heads + h) * splits;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, part_ml[(base + s) * 2]);
  float gl = 0.0f, go = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const float mm = part_ml[(base + s) * 2];
    const float w = (mm == -INFINITY) ? 0.0f : exp2f(mm - gm);
    gl += part_ml[(base + s) * 2 + 1] * w;
    go += part_o[(base + s) * D + d] * w;
  }
  out[row * o_row_stride + h * D + d] = __float2bfloat16_rn(gl > 0.0f ? go / gl : 0.0f);
}

// ------------------------------------------------------------------------------------------------
// skinny GEMM: y[m][n] = act(sum_k x[m][k] * w[n][k] + bias[n]) (+ residual / accumulate), m <= 16.
// One warp per output column; the reduction order of a row is fixed (independent of m).
// ------------------------------------------------------------------------------------------------
constexpr int kSkinnyMaxRows = 16;

template <int M, typename YT>
__global__ void __launch_bounds__(256)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ w, int64_t ldw,
                   const __nv_bfloat16* __restrict__ bias, const YT* residual, int64_t ldr, YT* y, int64_t ldy, int n,
                   int k, int act) {
  const int col = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (col >= n) return;
  float acc[M];
#pragma unroll
  for (int i = 0; i < M; ++i) acc[i] = 0.0f;
  const __nv_bfloat16* wr = w + static_cast<int64_t>(col) * ldw;
  for (int c = lane * 8; c < k; c += 256) {
    float wv[8];
    unpack8(*reinterpret_cast<const uint4*>(wr + c), wv);
#pragma unroll
    for (int i = 0; i < M; ++i) {
      float xv[8];
      unpack8(*reinterpret_cast<const uint4*>(x + i * ldx + c), xv);
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += xv[j] * wv[j];
      acc[i] += s;
    }
  }
#pragma unroll
  for (int i = 0; i < M; ++i) {
    float s = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    acc[i] = s;
  }
  if (lane == 0) {
    const float b = bias ? __bfloat162float(bias[col]) : 0.0f;
#pragma unroll
    for (int i = 0; i < M; ++i) {
      float v = acc[i] + b;
      if (act == NX_ACT_GELU) v = gelu_tanh_f(v);
      else if (act == NX_ACT_RELU) v = fmaxf(v, 0.0f);
      else if (act == NX_ACT_SILU) v = silu_f(v);
      if (residual) v += Num<YT>::load(residual + i * ldr + col);
      Num<YT>::store(y + i * ldy + col, v);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// row gather / token counts / NLL
// ------------------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ out, int n, int cols) {
  const int vec = cols >> 3;
  NX_GRID_STRIDE(i, static_cast<int64_t>(n) * vec) {
    const int r = static_cast<int>(i / vec), c = static_cast<int>(i % vec);
    reinterpret_cast<uint4*>(out + static_cast<int64_t>(r) * cols)[c] =
        reinterpret_cast<const uint4*>(x + static_cast<int64_t>(rows[r]) * cols)[c];
  }
}

__global__ void count_tokens_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ row_of,
                                    int32_t* __restrict__ counts, int n, int vocab) {
  NX_GRID_STRIDE(i, n) {
    const int t = tokens[i];
    if (t >= 0 && t < vocab) atomicAdd(counts + static_cast<int64_t>(row_of[i]) * vocab + t, 1);
  }
}

__global__ void nll_kernel(const float* __restrict__ logits, int64_t ld, const int32_t* __restrict__ targets,
                           float* __restrict__ out, int vocab) {
  __shared__ float s_scratch[32];
  const int row = blockIdx.x;
  const float* lr = logits + row * ld;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) mx = fmaxf(mx, lr[c]);
  mx = block_max(mx, s_scratch);
  float se = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) se += __expf(lr[c] - mx);
  se = block_sum<float>(se, s_scratch);
  if (threadIdx.x == 0) out[row] = mx + logf(se) - lr[targets[row]];
}

// ------------------------------------------------------------------------------------------------
// sampler: one block (1024 threads) per row
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void philox_draw(uint64_t seed, uint64_t offset, float& u) {
  uint32_t c[4] = {static_cast<uint32_t>(offset), static_cast<uint32_t>(offset >> 32), 0u, 0u};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  u = static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int64_t ld, int vocab, const NxSampleParams* __restrict__ params,
              const int32_t* __restrict__ counts_all, const int32_t* __restrict__ counts_out,
              const int32_t* __restrict__ count_row, const uint64_t* __restrict__ offsets, float* __restrict__ work,
              int32_t* __restrict__ out, int row_in_smem) {
  extern __shared__ float s_row[];  // the row's working values when they fit (vocab floats): every later pass reads them
  __shared__ float s_f[32];
  __shared__ float s_g[32];
  __shared__ int s_i[32];
  __shared__ float s_bcast;
  __shared__ int s_pick;
  const int row = blockIdx.x;
  const NxSampleParams p = params[row];
  const float* lr = logits + row * ld;
  float* wk = row_in_smem ? s_row : work + static_cast<int64_t>(row) * vocab;
  const int64_t crow = count_row ? count_row[row] : row;
  const int32_t* cnt_all = counts_all ? counts_all + crow * vocab : nullptr;  // prompt + generated tokens
  const int32_t* cnt_out = counts_out ? counts_out + crow * vocab : nullptr;  // generated tokens only
  // penalties + temperature; track max (ties -> lowest id)
  float mx = -INFINITY;
  int arg = 0x7fffffff;
  const float invt = p.temperature > 0.0f ? 1.0f / p.temperature : 1.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    float v = lr[c];
    if (cnt_all && p.repetition_penalty != 1.0f && cnt_all[c] > 0)
      v = v > 0.0f ? v / p.repetition_penalty : v * p.repetition_penalty;
    if (cnt_out) {
      const int n = cnt_out[c];
      if (n > 0) v -= p.frequency_penalty * n + p.presence_penalty;
    }
    v *= invt;
    wk[c] = v;
    if (v > mx || (v == mx && c < arg)) {
      mx = v;
      arg = c;
    }
  }
  // block arg-max with lowest-id tie break
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (om > mx || (om == mx && oa < arg)) {
      mx = om;
      arg = oa;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    s_f[threadIdx.x >> 5] = mx;
    s_i[threadIdx.x >> 5] = arg;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 32; ++i)
      if (s_f[i] > s_f[0] || (s_f[i] == s_f[0] && s_i[i] < s_i[0])) {
        s_f[0] = s_f[i];
        s_i[0] = s_i[i];
      }
    s_bcast = s_f[0];
    s_pick = s_i[0];
  }
  __syncthreads();
  const float gmax = s_bcast;
  if (p.temperature <= 0.0f) {  // greedy
    if (threadIdx.x == 0) out[row] = s_pick;
    return;
  }
  __syncthreads();
  // probabilities relative to the max (unnormalised): e_c = exp(v_c - max) in (0, 1]
  float se = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float e = __expf(wk[c] - gmax);
    wk[c] = e;
    se += e;
  }
  const float total = block_sum<float>(se, s_f);
  // threshold on e: keep {e >= thr}.  min-p: thr >= min_p (the top token has e = 1).
  float thr = p.min_p > 0.0f ? p.min_p : 0.0f;
  const bool want_k = p.top_k > 0 && p.top_k < vocab;       // largest thr such that count(e >= thr) >= top_k
  const bool want_p = p.top_p > 0.0f && p.top_p < 1.0f;     // largest thr such that mass(e >= thr) >= top_p * total
  if (want_k || want_p) {
    // the two bisections on e are independent: they share each pass over the row
    float lo_k = 0.0f, hi_k = 1.0f, lo_p = 0.0f, hi_p = 1.0f;
    for (int it = 0; it < 30; ++it) {
      const float mid_k = 0.5f * (lo_k + hi_k), mid_p = 0.5f * (lo_p + hi_p);
      float n = 0.0f, ms = 0.0f;
      for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
        const float e = wk[c];
        n += e >= mid_k ? 1.0f : 0.0f;
        ms += e >= mid_p ? e : 0.0f;
      }
      if (want_k) {
        n = block_sum<float>(n, s_f);
        if (n >= static_cast<float>(p.top_k)) lo_k = mid_k; else hi_k = mid_k;
      }
      if (want_p) {
        ms = block_sum<float>(ms, s_g);
        if (ms >= p.top_p * total) lo_p = mid_p; else hi_p = mid_p;
      }
    }
    if (want_k) thr = fmaxf(thr, lo_k);
    if (want_p) thr = fmaxf(thr, lo_p);
  }
  float kept = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) kept += wk[c] >= thr ? wk[c] : 0.0f;
  kept = block_sum<float>(kept, s_f);
  // inverse CDF over the kept tokens in id order: contiguous id ranges per thread
  float u;
  philox_draw(p.seed, offsets ? offsets[row] : 0ull, u);
  const float target = u * kept;
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int c0 = threadIdx.x * per, c1 = min(vocab, c0 + per);
  float mine = 0.0f;
  for (int c = c0; c < c1; ++c) mine += wk[c] >= thr ? wk[c] : 0.0f;
  __shared__ float s_scan[1024];
  s_scan[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.0f;
    int owner = -1;
    for (int t = 0; t < static_cast<int>(blockDim.x); ++t) {
      if (s_scan[t] > 0.0f) owner = t;
      if (run + s_scan[t] > target && s_scan[t] > 0.0f) {
        owner = t;
        s_bcast = run;
        break;
      }
      run += s_scan[t];
      s_bcast = run - s_scan[t];
    }
    s_pick = owner;
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) == s_pick) {
    float run = s_bcast;
    int pick = -1;
    for (int c = c0; c < c1; ++c) {
      if (wk[c] < thr) continue;
      pick = c;
      run += wk[c];
      if (run > target) break;
    }
    out[row] = pick >= 0 ? pick : 0;
  }
}

// ------------------------------------------------------------------------------------------------
// RoPE in place on [rows, heads, D] (row stride given); cos/sin [positions, rot/2]
// ------------------------------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, int64_t row_stride, const int32_t* __restrict__ positions,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rows, int heads,
                            int D, int half, int inverse, int interleaved) {
  NX_GRID_STRIDE(i, static_cast<int64_t>(rows) * heads * half) {
    const int j = static_cast<int>(i % half);
    const int h = static_cast<int>((i / half) % heads);
    const int64_t r = i / (static_cast<int64_t>(half) * heads);
    const int pos = positions[r];
    const float c = cos_t[static_cast<int64_t>(pos) * half + j];
    float s = sin_t[static_cast<int64_t>(pos) * half + j];
    if (inverse) s = -s;
    __nv_bfloat16* base = x + r * row_stride + h * D;
    const int i0 = interleaved ? 2 * j : j, i1 = interleaved ? 2 * j + 1 : j + half;
    const float a = __bfloat162float(base[i0]), b = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16_rn(a * c - b * s);
    base[i1] = __float2bfloat16_rn(b * c + a * s);
  }
}

// gated activation on [n, 2F] = [gate | up]: y = act(gate) * up;  act: 0 SiLU (SwiGLU), 1 GELU-tanh (GeGLU)
__global__ void gated_fwd_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ y, int64_t n, int F,
                                 int act) {
  NX_GRID_STRIDE(i, n * F) {
    const int64_t r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = __bfloat162float(h[r * 2 * F + c]), u = __bfloat162float(h[r * 2 * F + F + c]);
    y[i] = __float2bfloat16_rn((act == 0 ? silu_f(g) : gelu_tanh_f(g)) * u);
  }
}
__global__ void gated_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ dy,
                                 __nv_bfloat16* __restrict__ dh, int64_t n, int F, int act) {
  NX_GRID_STRIDE(i, n * F) {
    const int64_t r = i / F;
    const int c = static_cast<int>(i % F);
    const float g = __bfloat162float(h[r * 2 * F + c]), u = __bfloat162float(h[r * 2 * F + F + c]);
    const float d = __bfloat162float(dy[i]);
    float a, da;
    if (act == 0) {
      const float sg = 1.0f / (1.0f + __expf(-g));
      a = g * sg;
      da = sg * (1.0f + g * (1.0f - sg));
    } else {
      a = gelu_tanh_f(g);
      da = dgelu_tanh_f(g);
    }
    dh[r * 2 * F + c] = __float2bfloat16_rn(d * u * da);
    dh[r * 2 * F + F + c] = __float2bfloat16_rn(d * a);
  }
}

// ------------------------------------------------------------------------------------------------
// weight-only quantised GEMV (m <= 16): INT8 per-output-row scale, INT4 group-wise (AWQ-style,
// two nibbles per byte, value = (nibble - 8) * scale[group]); plus dequantisation to BF16.
// ------------------------------------------------------------------------------------------------
template <int M, int BITS>
__global__ void __launch_bounds__(256)
wq_gemv_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const uint8_t* __restrict__ wq,
               const float* __restrict__ scales, int group, const __nv_bfloat16* __restrict__ bias,
               __nv_bfloat16* __restrict__ y, int64_t ldy, int n, int k) {
  const int col = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (col >= n) return;
  float acc[M];
#pragma unroll
  for (int i = 0; i < M; ++i) acc[i] = 0.0f;
  const int64_t wrow = static_cast<int64_t>(col) * (BITS == 8 ? k : k / 2);
  const int groups = BITS == 4 ? k / group : 1;
  for (int c = lane * 8; c < k; c += 256) {
    float wv[8];
    if (BITS == 8) {
      const uint2 q = *reinterpret_cast<const uint2*>(wq + wrow + c);
      const int8_t* b = reinterpret_cast<const int8_t*>(&q);
      const float s = scales[col];
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[j] = static_cast<float>(b[j]) * s;
    } else {
      const uint32_t q = *reinterpret_cast<const uint32_t*>(wq + wrow + c / 2);
      const float s = scales[static_cast<int64_t>(col) * groups + c / group];
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[j] = static_cast<float>(static_cast<int>((q >> (4 * j)) & 15u) - 8) * s;
    }
#pragma unroll
    for (int i = 0; i < M; ++i) {
      float xv[8];
      unpack8(*reinterpret_cast<const uint4*>(x + i * ldx + c), xv);
      float s = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += xv[j] * wv[j];
      acc[i] += s;
    }
  }
#pragma unroll
  for (int i = 0; i < M; ++i) {
    float s = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) y[i * ldy + col] = __float2bfloat16_rn(s + (bias ? __bfloat162float(bias[col]) : 0.0f));
  }
}

__global__ void wq_dequant_kernel(const uint8_t* __restrict__ wq, const float* __restrict__ scales, int group,
                                  __nv_bfloat16* __restrict__ w, int n, int k, int bits) {
  NX_GRID_STRIDE(i, static_cast<int64_t>(n) * k) {
    const int r = static_cast<int>(i / k), c = static_cast<int>(i % k);
    float v;
    if (bits == 8) {
      v = static_cast<float>(static_cast<int8_t>(wq[i])) * scales[r];
    } else {
      const uint8_t b = wq[static_cast<int64_t>(r) * (k / 2) + c / 2];
      v = static_cast<float>(static_cast<int>((b >> (4 * (c & 1))) & 15) - 8) * scales[static_cast<int64_t>(r) * (k / group) + c / group];
    }
    w[i] = __float2bfloat16_rn(v);
  }
}

// per-row symmetric INT8 activation quantisation with optional SmoothQuant inverse column scales
__global__ void quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ inv_smooth,
                                  int8_t* __restrict__ q, __nv_bfloat16* __restrict__ fq,
                                  float* __restrict__ row_scale, int cols) {
  __shared__ float s_scratch[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + static_cast<int64_t>(row) * cols;
  float amax = 0.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x)
    amax = fmaxf(amax, fabsf(__bfloat162float(xr[c]) * (inv_smooth ? inv_smooth[c] : 1.0f)));
  amax = block_max(amax, s_scratch);
  const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = __bfloat162float(xr[c]) * (inv_smooth ? inv_smooth[c] : 1.0f) / scale;
    const int qi = max(-127, min(127, __float2int_rn(v)));
    if (q) q[static_cast<int64_t>(row) * cols + c] = static_cast<int8_t>(qi);
    if (fq) fq[static_cast<int64_t>(row) * cols + c] = __float2bfloat16_rn(static_cast<float>(qi) * scale);
  }
  if (threadIdx.x == 0 && row_scale) row_scale[row] = scale;
}

}  // namespace

// ================================================================================================
extern "C" int nx_kv_append(const void* k, const void* v, int64_t k_row_stride, int64_t v_row_stride,
                            const int32_t* slots, void* kc, void* vc, float* kscale, float* vscale, int tokens,
                            int kv_heads, int D, int kv_kind, nx_stream_t stream) {
  if (tokens <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int hd = kv_heads * D;
  if (kv_kind == 0) {
    if (hd & 7) return -1;
    kv_append_kernel<<<blocks_for(static_cast<int64_t>(tokens) * (hd / 8), 256), 256, 0, st>>>(
        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_row_stride, v_row_stride, slots, (__nv_bfloat16*)kc,
        (__nv_bfloat16*)vc, tokens, hd);
  } else {
    const int warps = tokens * kv_heads;
    const int blocks = (warps + 7) / 8;
    if (kv_kind == 1)
      kv_append_q8_kernel<false><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_row_stride, v_row_stride, slots, (uint8_t*)kc, (uint8_t*)vc, kscale, vscale, tokens, kv_heads, D);
    else
      kv_append_q8_kernel<true><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)k, (const __nv_bfloat16*)v, k_row_stride, v_row_stride, slots, (uint8_t*)kc, (uint8_t*)vc, kscale, vscale, tokens, kv_heads, D);
  }
  return launch_status();
}

extern "C" int nx_paged_attention_decode(const NxPagedArgs* a, nx_stream_t stream) {
  if (a == nullptr || a->rows <= 0) return a == nullptr ? -1 : 0;
  if ((a->head_dim != 64 && a->head_dim != 128) || a->heads % a->kv_heads) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int splits = a->splits < 1 ? 1 : a->splits;
  if (splits > 1 && (a->part_o == nullptr || a->part_ml == nullptr)) return -1;
  if (a->rows > 65535) return -1;
  dim3 grid(a->heads, a->rows, splits);
  // BF16 cache, 16-token pages, known pool size: pages come in by TMA (NEXUS_B200_PAGED_TMA=0 keeps the plain loads)
  static const bool tma_on = [] {
    const char* e = std::getenv("NEXUS_B200_PAGED_TMA");
    return e == nullptr || std::atoi(e) != 0;
  }();
  if (tma_on && a->kv_kind == 0 && a->block_size == 16 && a->num_blocks > 0 && a->status != nullptr) {
    const int D = a->head_dim;
    CUtensorMap tk, tv;
    const uint64_t cols = static_cast<uint64_t>(a->kv_heads) * D, rows_total = static_cast<uint64_t>(a->num_blocks) * 16;
    if (nx::make_tensor_map_3d(&tk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->k_cache, cols, rows_total, 1, cols, 0, D, 16,
                               CU_TENSOR_MAP_SWIZZLE_NONE) ||
        nx::make_tensor_map_3d(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->v_cache, cols, rows_total, 1, cols, 0, D, 16,
                               CU_TENSOR_MAP_SWIZZLE_NONE))
      return -3;
    const int smem = 2 * kPagedStages * 16 * D * 2 + kPagedStages * 8;
    if (D == 64)
      paged_decode_tma_kernel<64><<<grid, 128, smem, st>>>(tk, tv, (const __nv_bfloat16*)a->q, a->q_row_stride, a->block_table,
          a->max_blocks, a->row_seq, a->ctx_len, a->heads, a->kv_heads, a->scale, splits, (__nv_bfloat16*)a->out,
          a->o_row_stride, a->part_o, a->part_ml, a->status);
    else {
      static bool once = false;
      if (!once) {
        if (cudaFuncSetAttribute(paged_decode_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
          return -2;
        once = true;
      }
      paged_decode_tma_kernel<128><<<grid, 128, smem, st>>>(tk, tv, (const __nv_bfloat16*)a->q, a->q_row_stride, a->block_table,
          a->max_blocks, a->row_seq, a->ctx_len, a->heads, a->kv_heads, a->scale, splits, (__nv_bfloat16*)a->out,
          a->o_row_stride, a->part_o, a->part_ml, a->status);
    }
    if (launch_status() != 0) return -2;
    if (splits > 1) {
      dim3 g2(a->rows, a->heads);
      if (D == 64)
        paged_combine_kernel<64><<<g2, 64, 0, st>>>(a->part_o, a->part_ml, splits, a->heads, (__nv_bfloat16*)a->out, a->o_row_stride);
      else
        paged_combine_kernel<128><<<g2, 128, 0, st>>>(a->part_o, a->part_ml, splits, a->heads, (__nv_bfloat16*)a->out, a->o_row_stride);
    }
    return launch_status();
  }
#define NX_PD(D_, KV_)                                                                                              \
  paged_decode_kernel<D_, KV_><<<grid, 128, 0, st>>>((const __nv_bfloat16*)a->q, a->q_row_stride, a->k_cache, a->v_cache, \
      a->k_scale, a->v_scale, a->block_table, a->max_blocks, a->row_seq, a->ctx_len, a->block_size, a->heads,        \
      a->kv_heads, a->scale, splits, (__nv_bfloat16*)a->out, a->o_row_stride, a->part_o, a->part_ml)
  if (a->head_dim == 64) {
    if (a->kv_kind == 0) NX_PD(64, 0); else if (a->kv_kind == 1) NX_PD(64, 1); else NX_PD(64, 2);
  } else {
    if (a->kv_kind == 0) NX_PD(128, 0); else if (a->kv_kind == 1) NX_PD(128, 1); else NX_PD(128, 2);
  }
#undef NX_PD
  if (launch_status() != 0) return -2;
  if (splits > 1) {
    dim3 g2(a->rows, a->heads);
    if (a->head_dim == 64)
      paged_combine_kernel<64><<<g2, 64, 0, st>>>(a->part_o, a->part_ml, splits, a->heads, (__nv_bfloat16*)a->out, a->o_row_stride);
    else
      paged_combine_kernel<128><<<g2, 128, 0, st>>>(a->part_o, a->part_ml, splits, a->heads, (__nv_bfloat16*)a->out, a->o_row_stride);
  }
  return launch_status();
}

extern "C" int nx_skinny_max_rows(void) { return kSkinnyMaxRows; }

extern "C" int nx_skinny_gemm(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias,
                              const void* residual, int64_t ldr, void* y, int64_t ldy, int out_dtype, int m, int n,
                              int k, int act, nx_stream_t stream) {
  if (m < 1 || m > kSkinnyMaxRows || n <= 0 || k <= 0 || (k & 7) || (ldx & 7) || (ldw & 7)) return -1;
  if (out_dtype != NX_BF16 && out_dtype != NX_F32) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = (n + 7) / 8;
#define NX_SK(M_)                                                                                                      \
  case M_:                                                                                                             \
    if (out_dtype == NX_F32)                                                                                     \
      skinny_gemm_kernel<M_, float><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, ldw, \
          (const __nv_bfloat16*)bias, (const float*)residual, ldr, (float*)y, ldy, n, k, act);                          \
    else                                                                                                               \
      skinny_gemm_kernel<M_, __nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, ldx,                       \
          (const __nv_bfloat16*)w, ldw, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)residual, ldr,                \
          (__nv_bfloat16*)y, ldy, n, k, act);                                                                          \
    break
  switch (m) {
    NX_SK(1); NX_SK(2); NX_SK(3); NX_SK(4); NX_SK(5); NX_SK(6); NX_SK(7); NX_SK(8);
    NX_SK(9); NX_SK(10); NX_SK(11); NX_SK(12); NX_SK(13); NX_SK(14); NX_SK(15); NX_SK(16);
  }
#undef NX_SK
  return launch_status();
}

extern "C" int nx_gather_rows(const void* x, const int32_t* rows, void* out, int n, int cols, nx_stream_t stream) {
  if (n <= 0) return 0;
  if (cols & 7) return -1;
  gather_rows_kernel<<<blocks_for(static_cast<int64_t>(n) * (cols / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, rows, (__nv_bfloat16*)out, n, cols);
  return launch_status();
}

extern "C" int nx_count_tokens(const int32_t* tokens, const int32_t* row_of, int32_t* counts, int n, int vocab,
                               nx_stream_t stream) {
  if (n <= 0) return 0;
  count_tokens_kernel<<<blocks_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(tokens, row_of, counts, n, vocab);
  return launch_status();
}

extern "C" int nx_nll(const float* logits, int64_t ld, const int32_t* targets, float* out, int rows, int vocab,
                      nx_stream_t stream) {
  if (rows <= 0) return 0;
  nll_kernel<<<rows, 512, 0, static_cast<cudaStream_t>(stream)>>>(logits, ld, targets, out, vocab);
  return launch_status();
}

extern "C" int nx_sample(const float* logits, int64_t ld, int vocab, const NxSampleParams* params,
                         const int32_t* counts_all, const int32_t* counts_out, const int32_t* count_row,
                         const uint64_t* offsets, float* work, int32_t* out, int rows, nx_stream_t stream) {
  if (rows <= 0) return 0;
  if (work == nullptr) return -1;
  // rows of up to ~55 k entries live in shared memory for the threshold searches
  const size_t row_bytes = static_cast<size_t>(vocab) * sizeof(float);
  const bool in_smem = row_bytes <= 220 * 1024;
  static bool attr_set = false;
  if (in_smem && !attr_set) {
    if (cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  sample_kernel<<<rows, 1024, in_smem ? row_bytes : 0, static_cast<cudaStream_t>(stream)>>>(
      logits, ld, vocab, params, counts_all, counts_out, count_row, offsets, work, out, in_smem ? 1 : 0);
  return launch_status();
}

extern "C" int nx_rope(void* x, int64_t row_stride, const int32_t* positions, const float* cos_t, const float* sin_t,
                       int rows, int heads, int D, int rot_dim, int inverse, int interleaved, nx_stream_t stream) {
  if (rows <= 0) return 0;
  if (rot_dim <= 0 || rot_dim > D || (rot_dim & 1)) return -1;
  const int half = rot_dim / 2;
  rope_kernel<<<blocks_for(static_cast<int64_t>(rows) * heads * half, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (__nv_bfloat16*)x, row_stride, positions, cos_t, sin_t, rows, heads, D, half, inverse, interleaved);
  return launch_status();
}

extern "C" int nx_gated_fwd(const void* h, void* y, int64_t n, int F, int act, nx_stream_t stream) {
  if (n <= 0) return 0;
  gated_fwd_kernel<<<blocks_for(n * F, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>((const __nv_bfloat16*)h, (__nv_bfloat16*)y, n, F, act);
  return launch_status();
}

extern "C" int nx_gated_bwd(const void* h, const void* dy, void* dh, int64_t n, int F, int act, nx_stream_t stream) {
  if (n <= 0) return 0;
  gated_bwd_kernel<<<blocks_for(n * F, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dh, n, F, act);
  return launch_status();
}

extern "C" int nx_wq_gemv(const void* x, int64_t ldx, const void* wq, const float* scales, int bits, int group,
                          const void* bias, void* y, int64_t ldy, int m, int n, int k, nx_stream_t stream) {
  if (m < 1 || m > kSkinnyMaxRows || (k & 7) || (bits != 8 && bits != 4)) return -1;
  if (bits == 4 && (group <= 0 || (group & 7) || k % group)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = (n + 7) / 8;
#define NX_WQ(M_, B_) wq_gemv_kernel<M_, B_><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, (const uint8_t*)wq, scales, group, (const __nv_bfloat16*)bias, (__nv_bfloat16*)y, ldy, n, k)
#define NX_WQM(M_) case M_: if (bits == 8) NX_WQ(M_, 8); else NX_WQ(M_, 4); break
  switch (m) {
    NX_WQM(1); NX_WQM(2); NX_WQM(3); NX_WQM(4); NX_WQM(5); NX_WQM(6); NX_WQM(7); NX_WQM(8);
    NX_WQM(9); NX_WQM(10); NX_WQM(11); NX_WQM(12); NX_WQM(13); NX_WQM(14); NX_WQM(15); NX_WQM(16);
  }
#undef NX_WQM
#undef NX_WQ
  return launch_status();
}

extern "C" int nx_wq_dequant(const void* wq, const float* scales, int bits, int group, void* w, int n, int k,
                             nx_stream_t stream) {
  if (bits != 8 && bits != 4) return -1;
  wq_dequant_kernel<<<blocks_for(static_cast<int64_t>(n) * k, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint8_t*)wq, scales, group, (__nv_bfloat16*)w, n, k, bits);
  return launch_status();
}

extern "C" int nx_quant_rows(const void* x, const float* inv_smooth, void* q, void* fake_quant, float* row_scale,
                             int rows, int cols, nx_stream_t stream) {
  if (rows <= 0) return 0;
  quant_rows_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>((const __nv_bfloat16*)x, inv_smooth, (int8_t*)q,
                                                                         (__nv_bfloat16*)fake_quant, row_scale, cols);
  return launch_status();
}
