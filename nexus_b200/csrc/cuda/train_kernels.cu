// Training kernels: embedding+position forward, embedding backward (atomic and deterministic),
// fused shifted cross-entropy (in place, label smoothing, z-loss, ignore_index, padded rows),
// Philox4x32-10 dropout, global gradient norm, multi-tensor AdamW over chunk descriptors with FP32
// master weights and a narrow shadow copy, dynamic loss scale, non-finite guard, bias gradient.
// Parity: src/cuda/kernels_train.cu:35-1107 and src/fused/training.cpp:53-459 of the reference.
#include <atomic>

#include "common.cuh"
#include "nx_api_kernels.h"

#include <algorithm>
#include <cstdio>

namespace {
using namespace nx;

// ------------------------------------------------------------------------------------------------
// embedding
// ------------------------------------------------------------------------------------------------
template <typename WT, typename OT>
__global__ void embedding_pos_fwd_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ positions,
                                         const WT* __restrict__ wte, const WT* __restrict__ wpe, OT* __restrict__ out,
                                         int64_t rows, int seq_len, int cols) {
  const int vec = cols >> 2;
  NX_GRID_STRIDE(i, rows * vec) {
    const int64_t r = i / vec;
    const int c = static_cast<int>(i % vec) * 4;
    const int tok = tokens[r];
    const int pos = positions ? positions[r] : static_cast<int>(r % seq_len);
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = Num<WT>::load(wte + static_cast<int64_t>(tok) * cols + c + j);
      if (wpe) v += Num<WT>::load(wpe + static_cast<int64_t>(pos) * cols + c + j);
      o[j] = v;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) Num<OT>::store(out + r * cols + c + j, o[j]);
  }
}

template <typename GT>
__global__ void embedding_bwd_atomic_kernel(const int32_t* __restrict__ tokens, const GT* __restrict__ dx,
                                            float* __restrict__ dwte, int64_t rows, int cols) {
  NX_GRID_STRIDE(i, rows * cols) {
    const int64_t r = i / cols;
    const int c = static_cast<int>(i % cols);
    atomicAdd(dwte + static_cast<int64_t>(tokens[r]) * cols + c, Num<GT>::load(dx + i));
  }
}

// `order` lists row indices sorted by (token, row); one block per sorted position that starts a run.
template <typename GT>
__global__ void embedding_bwd_segment_kernel(const int32_t* __restrict__ sorted_tokens,
                                             const int64_t* __restrict__ order, const GT* __restrict__ dx,
                                             float* __restrict__ dwte, int64_t rows, int cols) {
  for (int64_t s = blockIdx.x; s < rows; s += gridDim.x) {
    const int tok = sorted_tokens[s];
    if (s > 0 && sorted_tokens[s - 1] == tok) continue;  // not a run start (block-uniform)
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float acc = 0.0f;
      for (int64_t j = s; j < rows && sorted_tokens[j] == tok; ++j)
        acc += Num<GT>::load(dx + order[j] * cols + c);
      dwte[static_cast<int64_t>(tok) * cols + c] += acc;
    }
  }
}

template <typename GT>
__global__ void wpe_bwd_kernel(const GT* __restrict__ dx, float* __restrict__ dwpe, int batch, int seq_len,
                               int cols) {
  NX_GRID_STRIDE(i, static_cast<int64_t>(seq_len) * cols) {
    float acc = 0.0f;
    for (int b = 0; b < batch; ++b) acc += Num<GT>::load(dx + static_cast<int64_t>(b) * seq_len * cols + i);
    dwpe[i] += acc;
  }
}

// ------------------------------------------------------------------------------------------------
// shifted cross-entropy
// ------------------------------------------------------------------------------------------------
struct CeState {        // device-resident, 4 floats + 2 ints
  float inv_valid;      // 1 / number of valid targets (0 when none)
  float loss;           // mean loss over valid targets
  int valid;            // number of valid targets
  int bad_target;       // 1 when a target is outside [0, vocab) and is not ignore_index
  float grad_mul;       // device-resident multiplier of the gradient (dynamic loss scale), 1 when none is given
};

__device__ __forceinline__ int ce_target(const int32_t* tokens, const int32_t* targets, int64_t row, int seq_len) {
  if (targets) return targets[row];
  const int t = static_cast<int>(row % seq_len);
  return (t == seq_len - 1) ? -100 : tokens[row + 1];
}

__global__ void ce_count_kernel(const int32_t* __restrict__ tokens, const int32_t* __restrict__ targets,
                                int64_t rows, int seq_len, int vocab, int ignore_index, CeState* st,
                                const float* __restrict__ grad_mul) {
  __shared__ int s_scratch[32];
  int count = 0, bad = 0;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) {
    int tg = ce_target(tokens, targets, r, seq_len);
    if (tg == ignore_index || (targets == nullptr && tg == -100)) continue;
    if (tg < 0 || tg >= vocab) bad = 1;
    else ++count;
  }
  count = block_sum<int>(count, s_scratch);
  bad = block_sum<int>(bad, s_scratch);
  if (threadIdx.x == 0) {
    st->valid = count;
    st->inv_valid = count > 0 ? 1.0f / static_cast<float>(count) : 0.0f;
    st->bad_target = bad ? 1 : 0;
    st->grad_mul = grad_mul != nullptr ? *grad_mul : 1.0f;
  }
}

// One block per row.  Pass 1: online max / sum-exp (+ sum of logits for label smoothing).  Pass 2:
// gradient written over the logits:  g = (p - s/V + 2 z lse p - (1-s)[j==target]) * scale / valid.
template <typename LT>
__global__ void ce_row_kernel(LT* __restrict__ logits, const int32_t* __restrict__ tokens,
                              const int32_t* __restrict__ targets, float* __restrict__ row_loss, int64_t rows,
                              int seq_len, int vocab, int64_t ld, int ignore_index, float smoothing, float z_loss,
                              float grad_scale, const CeState* __restrict__ st, int write_grad) {
  __shared__ float s_scratch[32];
  const int64_t row = blockIdx.x;
  LT* lr = logits + row * ld;
  const int tg = ce_target(tokens, targets, row, seq_len);
  const bool valid = !(tg == ignore_index || (targets == nullptr && tg == -100)) && tg >= 0 && tg < vocab;
  if (!valid) {
    if (threadIdx.x == 0) row_loss[row] = 0.0f;
    if (write_grad)
      for (int64_t c = threadIdx.x; c < ld; c += blockDim.x) Num<LT>::store(lr + c, 0.0f);
    return;
  }
  float mx = -INFINITY, se = 0.0f, sl = 0.0f;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float v = Num<LT>::load(lr + c);
    sl += v;
    if (v > mx) {
      se = se * __expf(mx - v) + 1.0f;
      mx = v;
    } else {
      se += __expf(v - mx);
    }
  }
  const float bmx = block_max(mx, s_scratch);
  se = (mx == -INFINITY) ? 0.0f : se * __expf(mx - bmx);
  se = block_sum<float>(se, s_scratch);
  sl = block_sum<float>(sl, s_scratch);
  const float lse = bmx + logf(se);
  const float tlogit = Num<LT>::load(lr + tg);
  // loss = (1-s) * (lse - x_t) + s * (lse - mean(x)) + z * lse^2
  const float loss = (1.0f - smoothing) * (lse - tlogit) + smoothing * (lse - sl / vocab) + z_loss * lse * lse;
  if (threadIdx.x == 0) row_loss[row] = loss;
  if (!write_grad) return;
  __syncthreads();  // every thread has read lr[tg] before anyone overwrites it
  const float k = grad_scale * st->inv_valid * st->grad_mul;
  const float pz = 1.0f + 2.0f * z_loss * lse;
  const float sv = smoothing / vocab;
  for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
    const float pr = __expf(Num<LT>::load(lr + c) - lse);
    float g = pr * pz - sv;
    if (c == tg) g -= (1.0f - smoothing);
    Num<LT>::store(lr + c, g * k);
  }
  for (int64_t c = vocab + threadIdx.x; c < ld; c += blockDim.x) Num<LT>::store(lr + c, 0.0f);
}

// 16-byte vector access to a logits row: 8 bf16 or 4 fp32 per load.
template <typename LT>
struct RowVec;
template <>
struct RowVec<__nv_bfloat16> {
  static constexpr int kN = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      v[2 * i] = __low2float(h);
      v[2 * i + 1] = __high2float(h);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct RowVec<float> {
  static constexpr int kN = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};

// Vectorised variant of ce_row_kernel: rows are 16-byte aligned (ld a multiple of the vector width).
// Pass 1 streams the row from HBM (online max / sum-exp in the log2 domain); pass 2 re-reads it
// (L2 resident: one row is ~100 KB) and writes the gradient in place.
template <typename LT>
__global__ void __launch_bounds__(512) ce_row_vec_kernel(LT* __restrict__ logits, const int32_t* __restrict__ tokens,
                                  const int32_t* __restrict__ targets, float* __restrict__ row_loss, int64_t rows,
                                  int seq_len, int vocab, int64_t ld, int ignore_index, float smoothing,
                                  float z_loss, float grad_scale, const CeState* __restrict__ st, int write_grad) {
  constexpr int VN = RowVec<LT>::kN;
  constexpr float kL2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
  __shared__ float s_scratch[32];
  const int64_t row = blockIdx.x;
  LT* lr = logits + row * ld;
  const int tg = ce_target(tokens, targets, row, seq_len);
  const bool valid = !(tg == ignore_index || (targets == nullptr && tg == -100)) && tg >= 0 && tg < vocab;
  const int nvec = static_cast<int>(ld / VN);
  if (!valid) {
    if (threadIdx.x == 0) row_loss[row] = 0.0f;
    if (write_grad) {
      float z[VN];
#pragma unroll
      for (int j = 0; j < VN; ++j) z[j] = 0.0f;
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) RowVec<LT>::store(lr + i * VN, z);
    }
    return;
  }
  const int full = vocab / VN;  // vectors entirely inside the vocabulary
  const int nuse = (vocab + VN - 1) / VN;  // vectors that hold at least one vocabulary entry
  float mx = -INFINITY, se = 0.0f, sl = 0.0f;
  auto absorb = [&](int i, float (&v)[VN]) {
    float vm = -INFINITY;
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      if (i >= full && i * VN + j >= vocab) v[j] = -INFINITY;
      vm = fmaxf(vm, v[j]);
    }
    if (vm > mx) {
      se *= exp2f((mx - vm) * kL2e);
      mx = vm;
    }
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      se += exp2f((v[j] - mx) * kL2e);
      sl += (v[j] == -INFINITY) ? 0.0f : v[j];
    }
  };
  {
    // four independent loads in flight per thread: one row is read once from HBM and latency is what limits it
    const int step = blockDim.x;
    int i = threadIdx.x;
    for (; i + 3 * step < nuse; i += 4 * step) {
      float v0[VN], v1[VN], v2[VN], v3[VN];
      RowVec<LT>::load(lr + i * VN, v0);
      RowVec<LT>::load(lr + (i + step) * VN, v1);
      RowVec<LT>::load(lr + (i + 2 * step) * VN, v2);
      RowVec<LT>::load(lr + (i + 3 * step) * VN, v3);
      absorb(i, v0);
      absorb(i + step, v1);
      absorb(i + 2 * step, v2);
      absorb(i + 3 * step, v3);
    }
    for (; i < nuse; i += step) {
      float v[VN];
      RowVec<LT>::load(lr + i * VN, v);
      absorb(i, v);
    }
  }
  const float bmx = block_max(mx, s_scratch);
  se = (mx == -INFINITY) ? 0.0f : se * exp2f((mx - bmx) * kL2e);
  se = block_sum<float>(se, s_scratch);
  sl = block_sum<float>(sl, s_scratch);
  const float lse = bmx + log2f(se) * kLn2;
  const float tlogit = Num<LT>::load(lr + tg);
  const float loss = (1.0f - smoothing) * (lse - tlogit) + smoothing * (lse - sl / vocab) + z_loss * lse * lse;
  if (threadIdx.x == 0) row_loss[row] = loss;
  if (!write_grad) return;
  __syncthreads();  // every thread has read lr[tg] before anyone overwrites it
  const float k = grad_scale * st->inv_valid * st->grad_mul;
  const float pz = (1.0f + 2.0f * z_loss * lse) * k;
  const float sv = smoothing / vocab * k;
  const float onehot = (1.0f - smoothing) * k;
  const float lse2 = lse * kL2e;
  auto grad_store = [&](int i, float (&v)[VN]) {
#pragma unroll
    for (int j = 0; j < VN; ++j) {
      const int c = i * VN + j;
      float g = exp2f(fmaf(v[j], kL2e, -lse2)) * pz - sv;
      if (c == tg) g -= onehot;
      v[j] = (c < vocab) ? g : 0.0f;
    }
    RowVec<LT>::store(lr + i * VN, v);
  };
  {
    // the row is rewritten in place: the loads of a group are issued before its stores
    const int step = blockDim.x;
    int i = threadIdx.x;
    for (; i + 3 * step < nuse; i += 4 * step) {
      float v0[VN], v1[VN], v2[VN], v3[VN];
      RowVec<LT>::load(lr + i * VN, v0);
      RowVec<LT>::load(lr + (i + step) * VN, v1);
      RowVec<LT>::load(lr + (i + 2 * step) * VN, v2);
      RowVec<LT>::load(lr + (i + 3 * step) * VN, v3);
      grad_store(i, v0);
      grad_store(i + step, v1);
      grad_store(i + 2 * step, v2);
      grad_store(i + 3 * step, v3);
    }
    for (; i < nuse; i += step) {
      float v[VN];
      RowVec<LT>::load(lr + i * VN, v);
      grad_store(i, v);
    }
    float z[VN];
#pragma unroll
    for (int j = 0; j < VN; ++j) z[j] = 0.0f;
    for (i = nuse + threadIdx.x; i < nvec; i += step) RowVec<LT>::store(lr + i * VN, z);  // padding columns
  }
}

__global__ void ce_reduce_kernel(const float* __restrict__ row_loss, int64_t rows, CeState* st,
                                 float* __restrict__ loss_out, float loss_weight, int accumulate) {
  pdl_trigger();
  __shared__ double s_scratch[32];
  double acc = 0.0;
  for (int64_t r = threadIdx.x; r < rows; r += blockDim.x) acc += row_loss[r];
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) {
    float loss = st->bad_target ? NAN : static_cast<float>(acc * st->inv_valid);
    st->loss = loss;
    if (loss_out) *loss_out = accumulate ? *loss_out + loss * loss_weight : loss * loss_weight;
  }
}

// ------------------------------------------------------------------------------------------------
// Philox4x32-10: block = offset + i/4, lane = i%4, u = top 24 bits / 2^24, keep iff u >= p.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void philox4x32_10(uint32_t (&ctr)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, ctr[0]), lo0 = M0 * ctr[0];
    const uint32_t hi1 = __umulhi(M1, ctr[2]), lo1 = M1 * ctr[2];
    const uint32_t n0 = hi1 ^ ctr[1] ^ k0, n1 = lo1, n2 = hi0 ^ ctr[3] ^ k1, n3 = lo0;
    ctr[0] = n0; ctr[1] = n1; ctr[2] = n2; ctr[3] = n3;
    k0 += W0;
    k1 += W1;
  }
}

template <typename T, bool kBackward>
__global__ void dropout_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, float p, uint64_t seed,
                               uint64_t offset) {
  const float scale = 1.0f / (1.0f - p);
  const int64_t nblk = (n + 3) / 4;
  NX_GRID_STRIDE(b, nblk) {
    const uint64_t blk = offset + static_cast<uint64_t>(b);
    uint32_t ctr[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u};
    philox4x32_10(ctr, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t i = b * 4 + j;
      if (i < n) {
        const float u = static_cast<float>(ctr[j] >> 8) * (1.0f / 16777216.0f);
        const float v = Num<T>::load(in + i);
        Num<T>::store(out + i, u >= p ? v * scale : 0.0f);
      }
    }
  }
}

__global__ void philox_uniform_kernel(float* __restrict__ out, int64_t n, uint64_t seed, uint64_t offset) {
  const int64_t nblk = (n + 3) / 4;
  NX_GRID_STRIDE(b, nblk) {
    const uint64_t blk = offset + static_cast<uint64_t>(b);
    uint32_t ctr[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u};
    philox4x32_10(ctr, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (b * 4 + j < n) out[b * 4 + j] = static_cast<float>(ctr[j] >> 8) * (1.0f / 16777216.0f);
  }
}

// ------------------------------------------------------------------------------------------------
// optimizer
// ------------------------------------------------------------------------------------------------
constexpr int kNormChunk = 65536;

template <typename GT>
__global__ void grad_norm_partial_kernel(const GT* __restrict__ g, int64_t n, double* __restrict__ partial) {
  __shared__ double s_scratch[32];
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kNormChunk;
  const int64_t end = min(n, begin + kNormChunk);
  double acc = 0.0;
  for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = Num<GT>::load(g + i);
    acc += static_cast<double>(v) * v;
  }
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// Sums the partials (plus an optional externally reduced square sum), derives the clip coefficient
// and the bias corrections for this step, and advances the accepted-step counter.
__global__ void grad_norm_final_kernel(const double* __restrict__ partial, int nparts, NxOptState* st,
                                       const double* __restrict__ extra_sq, int use_partials_only) {
  __shared__ double s_scratch[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x != 0) return;
  if (use_partials_only) {  // only publish the local square sum (the caller all-reduces it)
    st->local_sq = acc;
    return;
  }
  if (extra_sq) acc = *extra_sq;
  const double inv_scale = st->loss_scale > 0.0f ? 1.0 / st->loss_scale : 1.0;
  const double norm = sqrt(acc) * inv_scale;
  const bool finite = isfinite(norm);
  st->grad_norm = static_cast<float>(norm);
  st->found_inf = finite ? 0 : 1;
  double coef = 1.0;
  if (st->max_grad_norm > 0.0f) coef = fmin(1.0, static_cast<double>(st->max_grad_norm) / (norm + 1e-6));
  st->clip_coef = static_cast<float>(coef * inv_scale);
  if (finite) {
    st->step += 1;
    const double t = static_cast<double>(st->step);
    st->inv_bias1 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(st->beta1), t)));
    st->inv_bias2 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(st->beta2), t)));
  } else {
    st->skipped += 1;
  }
}

// One block per chunk descriptor.  No fused multiply-add: op order matches the CPU oracle bit for bit.
template <typename GT, typename ST>
__global__ void adamw_kernel(float* __restrict__ master, const GT* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, ST* __restrict__ shadow, const NxAdamChunk* __restrict__ chunks,
                             const NxOptState* __restrict__ st, int zero_grad, uint64_t sr_seed) {
  const NxAdamChunk ch = chunks[blockIdx.x];
  if (st->found_inf) {  // skipped step: the weights stay, the (non-finite) gradients still go
    if (zero_grad) {
      GT* gw = const_cast<GT*>(grad);
      for (int64_t i = ch.offset + threadIdx.x; i < ch.offset + ch.count; i += blockDim.x) Num<GT>::store(gw + i, 0.0f);
    }
    return;
  }
  const float lr = __fmul_rn(st->lr, ch.lr_scale);
  const float wd = __fmul_rn(st->weight_decay, ch.wd_scale);
  const float b1 = st->beta1, b2 = st->beta2, omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  const float i1 = st->inv_bias1, i2 = st->inv_bias2, eps = st->eps, clip = st->clip_coef;
  const float lrwd = __fmul_rn(lr, wd);
  if (sizeof(GT) == 4 && sizeof(ST) == 2 && sr_seed == 0 && shadow != nullptr && (ch.offset & 3) == 0 &&
      (ch.count & 3) == 0) {
    // 16-byte path (same per-element op order): one pass updates p/m/v, the shadow and clears the gradient
    float4* g4 = reinterpret_cast<float4*>(const_cast<GT*>(grad) + ch.offset);
    float4* p4 = reinterpret_cast<float4*>(master + ch.offset);
    float4* m4 = reinterpret_cast<float4*>(m + ch.offset);
    float4* v4 = reinterpret_cast<float4*>(v + ch.offset);
    uint2* s2 = reinterpret_cast<uint2*>(shadow + ch.offset);
    const int n4 = static_cast<int>(ch.count >> 2);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 gq = g4[i];
      float4 pq = p4[i], mq = m4[i], vq = v4[i];
      float gg[4] = {gq.x, gq.y, gq.z, gq.w}, pp[4] = {pq.x, pq.y, pq.z, pq.w}, mm[4] = {mq.x, mq.y, mq.z, mq.w},
            vv[4] = {vq.x, vq.y, vq.z, vq.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float g = __fmul_rn(gg[j], clip);
        float p = pp[j];
        p = __fsub_rn(p, __fmul_rn(lrwd, p));
        const float mi = __fadd_rn(__fmul_rn(b1, mm[j]), __fmul_rn(omb1, g));
        const float vi = __fadd_rn(__fmul_rn(b2, vv[j]), __fmul_rn(omb2, __fmul_rn(g, g)));
        p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr, __fmul_rn(mi, i1)), __fadd_rn(__fsqrt_rn(__fmul_rn(vi, i2)), eps)));
        pp[j] = p;
        mm[j] = mi;
        vv[j] = vi;
      }
      p4[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      m4[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
      v4[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
      s2[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
      if (zero_grad) g4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    return;
  }
  for (int64_t i = ch.offset + threadIdx.x; i < ch.offset + ch.count; i += blockDim.x) {
    const float g = __fmul_rn(Num<GT>::load(grad + i), clip);
    float p = master[i];
    p = __fsub_rn(p, __fmul_rn(lrwd, p));
    const float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(omb1, g));
    const float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(omb2, __fmul_rn(g, g)));
    const float mh = __fmul_rn(mi, i1);
    const float vh = __fmul_rn(vi, i2);
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr, mh), __fadd_rn(__fsqrt_rn(vh), eps)));
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    if (shadow) {
      if (sr_seed != 0 && sizeof(ST) == 2) {
        // stochastic rounding to BF16: add uniform noise below the kept mantissa, then truncate
        uint32_t ctr[4] = {static_cast<uint32_t>(i), static_cast<uint32_t>(i >> 32), static_cast<uint32_t>(st->step),
                           0u};
        philox4x32_10(ctr, static_cast<uint32_t>(sr_seed), static_cast<uint32_t>(sr_seed >> 32));
        uint32_t bits = __float_as_uint(p);
        bits += ctr[0] & 0xFFFFu;
        bits &= 0xFFFF0000u;
        Num<ST>::store(shadow + i, __uint_as_float(bits));
      } else {
        Num<ST>::store(shadow + i, p);
      }
    }
  }
  if (zero_grad) {
    GT* gw = const_cast<GT*>(grad);
    for (int64_t i = ch.offset + threadIdx.x; i < ch.offset + ch.count; i += blockDim.x) Num<GT>::store(gw + i, 0.0f);
  }
}

// Dynamic loss scale: halve on overflow, double after `growth_interval` clean steps.
__global__ void loss_scale_update_kernel(NxOptState* st, float growth, float backoff, int growth_interval,
                                         float min_scale, float max_scale) {
  if (st->found_inf) {
    st->loss_scale = fmaxf(min_scale, st->loss_scale * backoff);
    st->good_steps = 0;
  } else {
    st->good_steps += 1;
    if (st->good_steps >= growth_interval) {
      st->loss_scale = fminf(max_scale, st->loss_scale * growth);
      st->good_steps = 0;
    }
  }
}

template <typename T>
__global__ void count_nonfinite_kernel(const T* __restrict__ x, int64_t n, int* __restrict__ count) {
  int local = 0;
  NX_GRID_STRIDE(i, n) {
    const float v = Num<T>::load(x + i);
    if (!isfinite(v)) ++local;
  }
  local = __reduce_add_sync(0xffffffffu, local);
  if ((threadIdx.x & 31) == 0 && local) atomicAdd(count, local);
}

// Column sums of a [rows, cols] matrix (bias gradient), deterministic two-stage reduce.
template <typename GT>
__global__ void colsum_partial_kernel(const GT* __restrict__ dy, float* __restrict__ partial, int rows, int cols,
                                      int64_t ld, int rows_per_chunk) {
  __shared__ float s[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const int r_begin = blockIdx.y * rows_per_chunk, r_end = min(rows, r_begin + rows_per_chunk);
  float acc = 0.0f;
  if (c < cols)
    for (int r = r_begin + threadIdx.y; r < r_end; r += 8) acc += Num<GT>::load(dy + static_cast<int64_t>(r) * ld + c);
  s[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += s[k][threadIdx.x];
    partial[static_cast<int64_t>(blockIdx.y) * cols + c] = t;
  }
}
// BF16 fast path: each thread owns 8 adjacent columns (one 16-byte load per row); block = 32 column
// groups x 8 row lanes = a 256-column strip of one row chunk.  Same partial layout as above.
__global__ void colsum_partial_vec_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ partial,
                                          int rows, int cols, int64_t ld, int rows_per_chunk) {
  __shared__ float s[8][32][9];
  const int c0 = (blockIdx.x * 32 + threadIdx.x) * 8;
  const int r_begin = blockIdx.y * rows_per_chunk, r_end = min(rows, r_begin + rows_per_chunk);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  if (c0 < cols) {
    int r = r_begin + threadIdx.y;
    // four rows per trip: their loads are all issued before the first sum (more bytes in flight per thread)
    for (; r + 24 < r_end; r += 32) {
      float v[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) RowVec<__nv_bfloat16>::load(dy + static_cast<int64_t>(r + 8 * u) * ld + c0, v[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += v[u][j];
      }
    }
    for (; r < r_end; r += 8) {
      float v[8];
      RowVec<__nv_bfloat16>::load(dy + static_cast<int64_t>(r) * ld + c0, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s[threadIdx.y][threadIdx.x][j] = acc[j];
  __syncthreads();
  if (threadIdx.y == 0 && c0 < cols) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float t = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += s[k][threadIdx.x][j];
      partial[static_cast<int64_t>(blockIdx.y) * cols + c0 + j] = t;
    }
  }
}
__global__ void colsum_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int cols, int chunks,
                                    int accumulate) {
  pdl_trigger();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.0f;
  for (int k = 0; k < chunks; ++k) t += partial[static_cast<int64_t>(k) * cols + c];
  out[c] = accumulate ? out[c] + t : t;
}

}  // namespace

// ================================================================================================
// C entry points
// ================================================================================================
extern "C" int nx_embedding_pos_fwd(const int32_t* tokens, const int32_t* positions, const void* wte,
                                    const void* wpe, int w_dtype, void* out, int out_dtype, int64_t rows,
                                    int seq_len, int cols, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0 || (cols & 3)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = blocks_for(rows * (cols / 4), 256);
#define NX_E(WT, OT)                                                                                          \
  embedding_pos_fwd_kernel<WT, OT><<<blocks, 256, 0, st>>>(tokens, positions, (const WT*)wte, (const WT*)wpe, \
                                                           (OT*)out, rows, seq_len, cols)
  if (w_dtype == NX_F32 && out_dtype == NX_F32) NX_E(float, float);
  else if (w_dtype == NX_F32 && out_dtype == NX_BF16) NX_E(float, __nv_bfloat16);
  else if (w_dtype == NX_BF16 && out_dtype == NX_F32) NX_E(__nv_bfloat16, float);
  else if (w_dtype == NX_BF16 && out_dtype == NX_BF16) NX_E(__nv_bfloat16, __nv_bfloat16);
  else return -1;
#undef NX_E
  return launch_status();
}

extern "C" int nx_embedding_bwd(const int32_t* tokens, const int32_t* sorted_tokens, const int64_t* order,
                                const void* dx, int dx_dtype, float* dwte, float* dwpe, int batch, int seq_len,
                                int cols, nx_stream_t stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t rows = static_cast<int64_t>(batch) * seq_len;
  if (rows <= 0 || cols <= 0) return -1;
  if (dwte) {
    if (sorted_tokens && order) {
      const int blocks = static_cast<int>(std::min<int64_t>(rows, 148 * 32));
      if (dx_dtype == NX_F32)
        embedding_bwd_segment_kernel<float><<<blocks, 128, 0, st>>>(sorted_tokens, order, (const float*)dx, dwte, rows, cols);
      else
        embedding_bwd_segment_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>(sorted_tokens, order, (const __nv_bfloat16*)dx, dwte, rows, cols);
    } else {
      const int blocks = blocks_for(rows * cols, 256);
      if (dx_dtype == NX_F32)
        embedding_bwd_atomic_kernel<float><<<blocks, 256, 0, st>>>(tokens, (const float*)dx, dwte, rows, cols);
      else
        embedding_bwd_atomic_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(tokens, (const __nv_bfloat16*)dx, dwte, rows, cols);
    }
    if (launch_status() != 0) return -2;
  }
  if (dwpe) {
    const int blocks = blocks_for(static_cast<int64_t>(seq_len) * cols, 256);
    if (dx_dtype == NX_F32)
      wpe_bwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)dx, dwpe, batch, seq_len, cols);
    else
      wpe_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dx, dwpe, batch, seq_len, cols);
  }
  return launch_status();
}

extern "C" size_t nx_ce_state_bytes(void) { return sizeof(CeState); }

extern "C" int nx_cross_entropy_shifted_scaled(void* logits, int logits_dtype, const int32_t* tokens,
                                               const int32_t* targets, float* row_loss, void* ce_state, float* loss_out,
                                               float loss_weight, int accumulate_loss, int64_t rows, int seq_len,
                                               int vocab, int64_t ld, int ignore_index, float smoothing, float z_loss,
                                               float grad_scale, const float* grad_scale_dev, int write_grad,
                                               nx_stream_t stream);

extern "C" int nx_cross_entropy_shifted(void* logits, int logits_dtype, const int32_t* tokens,
                                        const int32_t* targets, float* row_loss, void* ce_state, float* loss_out,
                                        float loss_weight, int accumulate_loss, int64_t rows, int seq_len, int vocab,
                                        int64_t ld, int ignore_index, float smoothing, float z_loss, float grad_scale,
                                        int write_grad, nx_stream_t stream) {
  return nx_cross_entropy_shifted_scaled(logits, logits_dtype, tokens, targets, row_loss, ce_state, loss_out, loss_weight,
                                         accumulate_loss, rows, seq_len, vocab, ld, ignore_index, smoothing, z_loss,
                                         grad_scale, nullptr, write_grad, stream);
}

extern "C" int nx_cross_entropy_shifted_scaled(void* logits, int logits_dtype, const int32_t* tokens,
                                               const int32_t* targets, float* row_loss, void* ce_state, float* loss_out,
                                               float loss_weight, int accumulate_loss, int64_t rows, int seq_len,
                                               int vocab, int64_t ld, int ignore_index, float smoothing, float z_loss,
                                               float grad_scale, const float* grad_scale_dev, int write_grad,
                                               nx_stream_t stream) {
  if (rows <= 0 || vocab <= 0 || ld < vocab || seq_len <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CeState* cs = static_cast<CeState*>(ce_state);
  ce_count_kernel<<<1, 1024, 0, st>>>(tokens, targets, rows, seq_len, vocab, ignore_index, cs, grad_scale_dev);
  const bool aligned = (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (logits_dtype == NX_F32 && aligned && (ld % 4) == 0)
    ce_row_vec_kernel<float><<<static_cast<unsigned>(rows), 512, 0, st>>>((float*)logits, tokens, targets, row_loss, rows, seq_len, vocab, ld, ignore_index, smoothing, z_loss, grad_scale, cs, write_grad);
  else if (logits_dtype == NX_BF16 && aligned && (ld % 8) == 0)
    ce_row_vec_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 512, 0, st>>>((__nv_bfloat16*)logits, tokens, targets, row_loss, rows, seq_len, vocab, ld, ignore_index, smoothing, z_loss, grad_scale, cs, write_grad);
  else if (logits_dtype == NX_F32)
    ce_row_kernel<float><<<static_cast<unsigned>(rows), 512, 0, st>>>((float*)logits, tokens, targets, row_loss, rows, seq_len, vocab, ld, ignore_index, smoothing, z_loss, grad_scale, cs, write_grad);
  else if (logits_dtype == NX_BF16)
    ce_row_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), 512, 0, st>>>((__nv_bfloat16*)logits, tokens, targets, row_loss, rows, seq_len, vocab, ld, ignore_index, smoothing, z_loss, grad_scale, cs, write_grad);
  else
    return -1;
  ce_reduce_kernel<<<1, 1024, 0, st>>>(row_loss, rows, cs, loss_out, loss_weight, accumulate_loss);
  return launch_status();
}

extern "C" int nx_dropout(const void* in, void* out, int dtype, int64_t n, float p, uint64_t seed, uint64_t offset,
                          int backward, nx_stream_t stream) {
  if (n <= 0 || p < 0.0f || p >= 1.0f) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = blocks_for((n + 3) / 4, 256);
  // forward and backward apply the same mask; the flag only exists for API symmetry
  (void)backward;
  if (dtype == NX_F32)
    dropout_kernel<float, false><<<blocks, 256, 0, st>>>((const float*)in, (float*)out, n, p, seed, offset);
  else if (dtype == NX_BF16)
    dropout_kernel<__nv_bfloat16, false><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n, p, seed, offset);
  else
    return -1;
  return launch_status();
}

extern "C" int nx_philox_uniform(float* out, int64_t n, uint64_t seed, uint64_t offset, nx_stream_t stream) {
  if (n <= 0) return -1;
  philox_uniform_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(out, n, seed, offset);
  return launch_status();
}

extern "C" int64_t nx_grad_norm_partials(int64_t n) { return (n + kNormChunk - 1) / kNormChunk; }

extern "C" int nx_grad_norm(const void* grad, int grad_dtype, int64_t n, double* partial, NxOptState* state,
                            const double* extra_sq, int local_only, nx_stream_t stream) {
  if (n <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nparts = static_cast<int>((n + kNormChunk - 1) / kNormChunk);
  if (extra_sq == nullptr || local_only) {
    if (grad_dtype == NX_F32)
      grad_norm_partial_kernel<float><<<nparts, 256, 0, st>>>((const float*)grad, n, partial);
    else if (grad_dtype == NX_BF16)
      grad_norm_partial_kernel<__nv_bfloat16><<<nparts, 256, 0, st>>>((const __nv_bfloat16*)grad, n, partial);
    else
      return -1;
  }
  grad_norm_final_kernel<<<1, 1024, 0, st>>>(partial, (extra_sq && !local_only) ? 0 : nparts, state, local_only ? nullptr : extra_sq, local_only);
  return launch_status();
}

extern "C" int nx_adamw(float* master, const void* grad, int grad_dtype, float* m, float* v, void* shadow,
                        int shadow_dtype, const NxAdamChunk* chunks, int nchunks, const NxOptState* state,
                        int zero_grad, uint64_t sr_seed, nx_stream_t stream) {
  if (nchunks <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define NX_A(GT, ST) adamw_kernel<GT, ST><<<nchunks, 256, 0, st>>>(master, (const GT*)grad, m, v, (ST*)shadow, chunks, state, zero_grad, sr_seed)
  if (grad_dtype == NX_F32 && (shadow == nullptr || shadow_dtype == NX_BF16)) NX_A(float, __nv_bfloat16);
  else if (grad_dtype == NX_F32 && shadow_dtype == NX_F16) NX_A(float, __half);
  else if (grad_dtype == NX_F32 && shadow_dtype == NX_F32) NX_A(float, float);
  else if (grad_dtype == NX_BF16 && (shadow == nullptr || shadow_dtype == NX_BF16)) NX_A(__nv_bfloat16, __nv_bfloat16);
  else return -1;
#undef NX_A
  return launch_status();
}

extern "C" int nx_loss_scale_update(NxOptState* state, float growth, float backoff, int growth_interval,
                                    float min_scale, float max_scale, nx_stream_t stream) {
  loss_scale_update_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(state, growth, backoff, growth_interval, min_scale, max_scale);
  return launch_status();
}

extern "C" int nx_count_nonfinite(const void* x, int dtype, int64_t n, int* count, nx_stream_t stream) {
  if (n <= 0) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = blocks_for(n, 256);
  if (dtype == NX_F32) count_nonfinite_kernel<float><<<blocks, 256, 0, st>>>((const float*)x, n, count);
  else if (dtype == NX_BF16) count_nonfinite_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, n, count);
  else return -1;
  return launch_status();
}

extern "C" size_t nx_colsum_scratch_bytes(int rows, int cols) {
  const int chunks = std::max(1, std::min(64, (rows + 255) / 256));
  return static_cast<size_t>(chunks) * cols * sizeof(float);
}

extern "C" int nx_colsum(const void* dy, int dtype, float* out, float* scratch, int rows, int cols, int64_t ld,
                         int accumulate, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0 || scratch == nullptr) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunks = std::max(1, std::min(64, (rows + 255) / 256));
  const int rpc = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 31) / 32, chunks), block(32, 8);
  if (dtype == NX_BF16 && (cols % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0) {
    dim3 vgrid((cols + 255) / 256, chunks);
    colsum_partial_vec_kernel<<<vgrid, block, 0, st>>>((const __nv_bfloat16*)dy, scratch, rows, cols, ld, rpc);
  } else if (dtype == NX_F32) colsum_partial_kernel<float><<<grid, block, 0, st>>>((const float*)dy, scratch, rows, cols, ld, rpc);
  else if (dtype == NX_BF16) colsum_partial_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)dy, scratch, rows, cols, ld, rpc);
  else return -1;
  colsum_final_kernel<<<(cols + 255) / 256, 256, 0, st>>>(scratch, out, cols, chunks, accumulate);
  return launch_status();
}

// ================================================================================================
// Column sums without caller-provided scratch (see nx_colsum_static in nx_api_kernels.h).
// ================================================================================================
namespace {

constexpr int kStaticColsumMaxCols = 8192;
constexpr int kStaticColsumMaxChunks = 64;

// Partial sums [chunk][col] of one call.  Lives in the module image: every GPU that loads this
// library holds these 2 MiB from load until the process exits.
static __device__ __align__(256) float g_colsum_static_scratch[kStaticColsumMaxChunks * kStaticColsumMaxCols];

constexpr int kMaxDevices = 64;
// device address of the array, per device ordinal; atomics because two host threads may make the first call at once
// (both would look up the same address, so a lost race only repeats the lookup)
std::atomic<float*> g_colsum_static_ptr[kMaxDevices];

// In host code `g_colsum_static_scratch` is only a handle for the symbol, not a device address, so
// the address a kernel can use is asked for once per device (with that device current).
int colsum_static_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -2;
  float* cached = g_colsum_static_ptr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "nx_colsum_static: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return -2;
    }
    cached = static_cast<float*>(p);
    g_colsum_static_ptr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return 0;
}

}  // namespace

extern "C" int nx_colsum_static_max_cols(void) { return kStaticColsumMaxCols; }

extern "C" int nx_colsum_static(const void* dy, int dtype, float* out, int rows, int cols, int64_t ld, int accumulate,
                                nx_stream_t stream) {
  if (dy == nullptr || out == nullptr || rows <= 0 || cols <= 0 || ld < cols) return -1;
  if (cols > kStaticColsumMaxCols) {
    fprintf(stderr, "nx_colsum_static: %d columns exceed the built-in scratch (max %d); use nx_colsum with "
                    "caller-provided scratch instead\n", cols, kStaticColsumMaxCols);
    return -5;
  }
  float* scratch = nullptr;
  const int rc = colsum_static_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  {
    // the array that was looked up belongs to the CURRENT device; data on another device would make the
    // kernels write partial sums into memory they cannot reach, so a mismatch is refused, not launched
    cudaPointerAttributes attr{};
    int dev = -1;
    cudaGetDevice(&dev);
    const cudaError_t pe = cudaPointerGetAttributes(&attr, out);
    if (pe != cudaSuccess) cudaGetLastError();  // an unknown pointer is not this check's business
    if (pe == cudaSuccess && attr.type == cudaMemoryTypeDevice && attr.device != dev) {
      fprintf(stderr, "nx_colsum_static: output lives on device %d but device %d is current; make the data's "
                      "device (and the stream's) current before the call\n", attr.device, dev);
      return -6;
    }
  }
  const int chunks = std::max(1, std::min(kStaticColsumMaxChunks, (rows + 255) / 256));
  const int rpc = (rows + chunks - 1) / chunks;
  dim3 grid((cols + 31) / 32, chunks), block(32, 8);
  // every (chunk, column) partial that the final pass reads is written by the first pass of this
  // same call, so nothing in the shared array has to be cleared between calls
  if (dtype == NX_BF16 && (cols % 8) == 0 && (ld % 8) == 0 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0) {
    dim3 vgrid((cols + 255) / 256, chunks);
    colsum_partial_vec_kernel<<<vgrid, block, 0, st>>>((const __nv_bfloat16*)dy, scratch, rows, cols, ld, rpc);
  } else if (dtype == NX_F32) {
    colsum_partial_kernel<float><<<grid, block, 0, st>>>((const float*)dy, scratch, rows, cols, ld, rpc);
  } else if (dtype == NX_BF16) {
    colsum_partial_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)dy, scratch, rows, cols, ld, rpc);
  } else {
    return -1;
  }
  colsum_final_kernel<<<(cols + 255) / 256, 256, 0, st>>>(scratch, out, cols, chunks, accumulate);
  return launch_status();
}
