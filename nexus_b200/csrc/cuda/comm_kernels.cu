// Kernels that fuse computation with NVLink / NVSwitch communication through peer-mapped
// (symmetric) memory: every rank passes a table of device pointers, one per rank, to buffers of
// identical layout; loads and stores through a peer's pointer travel over NVLink.
//
//   * cross-GPU barrier and flag signalling with BOUNDED waits (a wait that runs out records
//     kStatusTimeoutPeer in the status word and the kernel returns; nothing spins for ever);
//   * gradient reduce-scatter by owner-pull: the owner of a shard sums the shard over all ranks in a
//     fixed order (deterministic), fused with the FP64 square sum for the global norm;
//   * global-norm exchange (each rank publishes its square sum into every peer's slot) fused with
//     the clip coefficient / bias-correction computation of the optimizer state;
//   * AdamW on the owned shard fused with the all-gather of the updated BF16 weights: the narrow
//     copy is stored straight into every rank's parameter buffer;
//   * MoE dispatch (rows stored into the expert owner's capacity buffer) and combine (rows pulled
//     back from the owners, gate-weighted) for expert parallelism;
//   * vocabulary-parallel cross-entropy statistics exchange.
//
// No kernel here uses TMA multicast or multimem; plain peer loads/stores only, so a rank that
// exits between steps cannot fault its peers.
// Replaces (reference, CPU only): FsdpEngine::launch_reduce + step (src/dist/fsdp.cpp:387-568),
// MoeExpertParallel (src/dist/moe_ep.cpp:45-90), vocab-parallel CE (src/dist/parallel_lm.cpp:611-665).
#include <algorithm>

#include "common.cuh"
#include "nx_api_comm.h"
#include "sm100_ptx.cuh"

namespace {
using namespace nx;

constexpr uint64_t kPeerWaitNs = 2000000000ull;

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Thread t < n: tell rank t that `rank` reached `epoch`, then wait until rank t told us the same.
// flags.ptr[q] is rank q's flag array (n ints), as mapped into this process.
__device__ __forceinline__ bool signal_and_wait(const NxPeerTable& flags, int rank, int n, int epoch, int* status) {
  const int t = threadIdx.x;
  bool ok = true;
  if (t < n) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.ptr[t]) + rank, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.ptr[rank]) + t;
    const uint64_t t0 = globaltimer_ns();
    while (ld_acquire_sys(mine) < epoch) {
      if (globaltimer_ns() - t0 > kPeerWaitNs) {
        atomicCAS(status, 0, kStatusTimeoutPeer);
        ok = false;
        break;
      }
      __nanosleep(200);
    }
  }
  return ok;
}

// The barrier generation lives in device memory (`counter`, one int per rank, advanced in lockstep by every
// barrier-bearing kernel of the group), not in a kernel argument: a CUDA graph that captured such a kernel
// waits for a fresh generation on every replay.
__device__ __forceinline__ int next_epoch(const int* counter) { return *reinterpret_cast<const volatile int*>(counter) + 1; }

__global__ void barrier_kernel(NxPeerTable flags, int rank, int n, int* counter, int* status) {
  const int epoch = next_epoch(counter);
  __syncwarp();
  signal_and_wait(flags, rank, n, epoch, status);
  __syncwarp();
  if (threadIdx.x == 0) *counter = epoch;
}

// ------------------------------------------------------------------------------------------------
// owner-pull reduce-scatter + square sum
// ------------------------------------------------------------------------------------------------
constexpr int kReduceChunk = 16384;  // elements per block

__global__ void __launch_bounds__(256)
reduce_shard_kernel(NxPeerTable grads, int n, int64_t shard_off, int64_t count, float scale,
                    float* __restrict__ out, double* __restrict__ partial) {
  __shared__ double s_scratch[32];
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kReduceChunk;
  const int64_t end = min(count, begin + kReduceChunk);
  double sq = 0.0;
  // shard_off and every chunk start are multiples of 4 elements: 16-byte vector loads
  for (int64_t i = begin + threadIdx.x * 4; i < end; i += blockDim.x * 4) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i + 4 <= end) {
#pragma unroll 1
      for (int p = 0; p < n; ++p) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.ptr[p]) + shard_off + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      *reinterpret_cast<float4*>(out + i) = acc;
      sq += static_cast<double>(acc.x) * acc.x + static_cast<double>(acc.y) * acc.y +
            static_cast<double>(acc.z) * acc.z + static_cast<double>(acc.w) * acc.w;
    } else {
      for (int64_t j = i; j < end; ++j) {
        float a = 0.f;
        for (int p = 0; p < n; ++p) a += reinterpret_cast<const float*>(grads.ptr[p])[shard_off + j];
        a *= scale;
        out[j] = a;
        sq += static_cast<double>(a) * a;
      }
    }
  }
  sq = block_sum<double>(sq, s_scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = sq;
}

// One block.  Local square sum -> every peer's slot -> wait for all -> global norm -> optimizer state.
__global__ void norm_exchange_kernel(const double* __restrict__ partial, int nparts, NxPeerTable slots,
                                     NxPeerTable flags, int rank, int n, int* counter, NxOptState* st, int* status) {
  __shared__ double s_scratch[32];
  __shared__ int s_ok;
  const int epoch = next_epoch(counter);
  double acc = 0.0;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) acc += partial[i];
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) {
    st->local_sq = acc;
    s_ok = 1;
  }
  if (threadIdx.x < n) reinterpret_cast<double*>(slots.ptr[threadIdx.x])[rank] = acc;
  __syncthreads();
  const bool ok = signal_and_wait(flags, rank, n, epoch, status);
  if (!ok) s_ok = 0;
  __syncthreads();
  if (threadIdx.x != 0) return;
  *counter = epoch;
  if (!s_ok) {
    st->found_inf = 1;  // no update on a step whose exchange failed
    return;
  }
  double total = 0.0;
  const volatile double* mine = reinterpret_cast<const volatile double*>(slots.ptr[rank]);
  for (int q = 0; q < n; ++q) total += mine[q];
  const double inv_scale = st->loss_scale > 0.0f ? 1.0 / st->loss_scale : 1.0;
  const double norm = sqrt(total) * inv_scale;
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

// AdamW on the owned shard; chunk descriptors use GLOBAL element offsets clipped to the shard, the
// FP32 state arrays (master/grad/m/v) are shard-local (index = global - shard_off); the BF16 result
// goes to every rank's full shadow buffer at the global index.  Same op order as adamw_kernel.
__global__ void __launch_bounds__(256)
adamw_shard_allgather_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                             float* __restrict__ v, NxPeerTable shadows, NxPeerTable tails, int64_t tail_off,
                             int n, int64_t shard_off, const NxAdamChunk* __restrict__ chunks,
                             const NxOptState* __restrict__ st) {
  if (st->found_inf) return;
  const NxAdamChunk ch = chunks[blockIdx.x];
  const float lr = __fmul_rn(st->lr, ch.lr_scale);
  const float wd = __fmul_rn(st->weight_decay, ch.wd_scale);
  const float b1 = st->beta1, b2 = st->beta2, omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  const float i1 = st->inv_bias1, i2 = st->inv_bias2, eps = st->eps, clip = st->clip_coef;
  const float lrwd = __fmul_rn(lr, wd);
  for (int64_t gi = ch.offset + threadIdx.x; gi < ch.offset + ch.count; gi += blockDim.x) {
    const int64_t i = gi - shard_off;
    const float g = __fmul_rn(grad[i], clip);
    float p = master[i];
    p = __fsub_rn(p, __fmul_rn(lrwd, p));
    const float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(omb1, g));
    const float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(omb2, __fmul_rn(g, g)));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr, __fmul_rn(mi, i1)), __fadd_rn(__fsqrt_rn(__fmul_rn(vi, i2)), eps)));
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    const __nv_bfloat16 lp = __float2bfloat16_rn(p);
#pragma unroll 1
    for (int q = 0; q < n; ++q) reinterpret_cast<__nv_bfloat16*>(shadows.ptr[q])[gi] = lp;
    if (tail_off >= 0 && gi >= tail_off) {  // parameters that the model reads in FP32 (norm scales, biases)
#pragma unroll 1
      for (int q = 0; q < n; ++q) reinterpret_cast<float*>(tails.ptr[q])[gi - tail_off] = p;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// all-reduce over peer memory with the cast fused in: the owner of [shard_off, shard_off + count) pulls
// that range from every rank's input buffer (FP32 or BF16), sums in rank order in FP32, scales, and
// stores the result (FP32 or BF16) into the output buffer of n_out ranks (n_out = n: two-shot
// all-reduce; n_out = 1: only this rank's copy, i.e. a one-shot all-reduce when the range is the whole
// buffer).  16-byte accesses: offsets and counts are multiples of 8 elements.
// ------------------------------------------------------------------------------------------------
template <typename IT, typename OT>
__global__ void __launch_bounds__(256)
allreduce_shard_kernel(NxPeerTable in, int n_in, NxPeerTable out, int n_out, int64_t shard_off, int64_t count,
                       float scale) {
  constexpr int V = 8;
  const int64_t nvec = count / V;
  NX_GRID_STRIDE(i, nvec) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.0f;
#pragma unroll 1
    for (int p = 0; p < n_in; ++p) {
      const IT* src = reinterpret_cast<const IT*>(in.ptr[p]) + shard_off + i * V;
      if (sizeof(IT) == 4) {
        const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      } else {
        const uint4 q = *reinterpret_cast<const uint4*>(src);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
          acc[2 * j] += __low2float(h);
          acc[2 * j + 1] += __high2float(h);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] *= scale;
#pragma unroll 1
    for (int q = 0; q < n_out; ++q) {
      OT* dst = reinterpret_cast<OT*>(out.ptr[q]) + shard_off + i * V;
      if (sizeof(OT) == 4) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
      } else {
        uint4 w;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[4], acc[5]), h3 = __floats2bfloat162_rn(acc[6], acc[7]);
        w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
        w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(dst) = w;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Ulysses all-to-all by peer stores.  mode 0 (sequence -> heads): x is this rank's [B, Tl, H, D];
// head h goes to rank h / Hl as out[q][b, rank * Tl + t, h % Hl, :] with out [B, n * Tl, Hl, D].
// mode 1 (heads -> sequence): x is [B, n * Tl, Hl, D]; row t goes to rank t / Tl as
// out[q][b, t % Tl, rank * Hl + h, :] with out [B, Tl, H, D].  16-byte vectors (D % 8 == 0).
// ------------------------------------------------------------------------------------------------
__global__ void a2a_heads_kernel(const __nv_bfloat16* __restrict__ x, NxPeerTable out, int B, int Tl, int H, int D,
                                 int rank, int n, int mode) {
  const int Hl = H / n, vec = D >> 3;
  const int64_t total = static_cast<int64_t>(B) * Tl * H * vec;  // same element count in both modes
  NX_GRID_STRIDE(i, total) {
    const int dv = static_cast<int>(i % vec);
    int64_t r = i / vec;
    int64_t dst;
    int q;
    if (mode == 0) {
      const int h = static_cast<int>(r % H);
      const int t = static_cast<int>((r / H) % Tl);
      const int b = static_cast<int>(r / (static_cast<int64_t>(H) * Tl));
      q = h / Hl;
      dst = ((static_cast<int64_t>(b) * n * Tl + rank * Tl + t) * Hl + h % Hl) * vec + dv;
    } else {
      const int h = static_cast<int>(r % Hl);
      const int t = static_cast<int>((r / Hl) % (n * Tl));
      const int b = static_cast<int>(r / (static_cast<int64_t>(Hl) * n * Tl));
      q = t / Tl;
      dst = ((static_cast<int64_t>(b) * Tl + t % Tl) * H + rank * Hl + h) * vec + dv;
    }
    reinterpret_cast<uint4*>(out.ptr[q])[dst] = reinterpret_cast<const uint4*>(x)[i];
  }
}

// ------------------------------------------------------------------------------------------------
// MoE expert-parallel dispatch / combine over peer memory
// ------------------------------------------------------------------------------------------------
// Row r of the permuted token matrix belongs to global expert e = expert_of[r] at slot slot_of[r]
// (< capacity) of that expert; it is stored into the owner's buffer [local_experts, capacity, d].
__global__ void moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ token_of,
                                    const int32_t* __restrict__ expert_of, const int32_t* __restrict__ slot_of,
                                    NxPeerTable bufs, int rows, int d, int local_experts, int capacity,
                                    int src_rank, int n_ranks, const float* __restrict__ row_scale, int rows_per_token) {
  const int vec = d >> 3;  // 16-byte vectors
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    if (slot_of[r] < 0) continue;  // dropped by the capacity limit
    const int e = expert_of[r];
    const int owner = e / local_experts, le = e % local_experts;
    // each source rank owns a disjoint slice of the capacity: slot indices are global per expert
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.ptr[owner]) +
                         (static_cast<int64_t>(le) * capacity + slot_of[r]) * d;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(token_of ? token_of[r] : r / rows_per_token) * d);
    if (row_scale == nullptr) {
      for (int i = threadIdx.x; i < vec; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = src[i];
    } else {  // scaled copy (backward of the gate-weighted combine)
      const float sc = row_scale[r];
      for (int i = threadIdx.x; i < vec; i += blockDim.x) {
        const uint4 q = src[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          unpack_bf16x2(w[j], lo, hi);
          o[j] = pack_bf16x2(lo * sc, hi * sc);
        }
        reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  (void)src_rank;
  (void)n_ranks;
}

// y[t] = sum_j gate[t,j] * out_buf[owner(e_tj)][le][slot_tj]   (slot < 0: dropped assignment)
__global__ void moe_combine_kernel(NxPeerTable bufs, const int32_t* __restrict__ expert, const int32_t* __restrict__ slot,
                                   const float* __restrict__ gate, __nv_bfloat16* __restrict__ y, int tokens, int top_k,
                                   int d, int local_experts, int capacity) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
      for (int k = 0; k < top_k; ++k) {
        const int s = slot[t * top_k + k];
        if (s < 0) continue;
        const int e = expert[t * top_k + k];
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(bufs.ptr[e / local_experts]) +
                                   (static_cast<int64_t>(e % local_experts) * capacity + s) * d + c;
        const uint4 q = *reinterpret_cast<const uint4*>(src);
        const float g = gate[t * top_k + k];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float lo, hi;
          unpack_bf16x2(w[j], lo, hi);
          acc[2 * j] += g * lo;
          acc[2 * j + 1] += g * hi;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(y + static_cast<int64_t>(t) * d + c) = o;
    }
  }
}

// dgate[t, j] = dy[t] . out_buf[owner(e_tj)][le][slot_tj] read from the owner's memory (0 for dropped assignments);
// one warp per (t, j)
__global__ void moe_gate_grad_peers_kernel(const __nv_bfloat16* __restrict__ dy, NxPeerTable bufs,
                                           const int32_t* __restrict__ expert, const int32_t* __restrict__ slot,
                                           float* __restrict__ dgate, int entries, int k, int d, int local_experts,
                                           int capacity) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= entries) return;
  const int s = slot[i];
  float acc = 0.0f;
  if (s >= 0) {
    const int e = expert[i];
    const __nv_bfloat16* a = dy + static_cast<int64_t>(i / k) * d;
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(bufs.ptr[e / local_experts]) +
                             (static_cast<int64_t>(e % local_experts) * capacity + s) * d;
    for (int c = lane * 8; c < d; c += 256) {
      const uint4 x = *reinterpret_cast<const uint4*>(a + c);
      const uint4 y = *reinterpret_cast<const uint4*>(b + c);
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float xl, xh, yl, yh;
        unpack_bf16x2(xw[j], xl, xh);
        unpack_bf16x2(yw[j], yl, yh);
        acc += xl * yl + xh * yh;
      }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dgate[i] = acc;
}

// ------------------------------------------------------------------------------------------------
// vocabulary-parallel cross-entropy: exchange of per-row statistics
// ------------------------------------------------------------------------------------------------
// stats[rank] holds [rows][3] = (local max, local sum-exp relative to the local max, target logit or 0).
// Every rank publishes its rows into every peer's table, waits, then merges in rank order:
//   gmax = max_q max_q;  sumexp = sum_q se_q * exp(max_q - gmax);  tlogit = sum_q t_q.
__global__ void vocab_ce_exchange_kernel(const float* __restrict__ local_stats, NxPeerTable tables, NxPeerTable flags,
                                         int rank, int n, int rows, int* counter, float* __restrict__ merged, int* status) {
  __shared__ int s_ok;
  const int epoch = next_epoch(counter);
  for (int i = threadIdx.x; i < rows * 3; i += blockDim.x) {
    const float v = local_stats[i];
    for (int q = 0; q < n; ++q) reinterpret_cast<float*>(tables.ptr[q])[static_cast<int64_t>(rank) * rows * 3 + i] = v;
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const bool ok = signal_and_wait(flags, rank, n, epoch, status);
  if (!ok) s_ok = 0;
  __syncthreads();
  if (threadIdx.x == 0) *counter = epoch;
  if (!s_ok) return;
  const volatile float* mine = reinterpret_cast<const volatile float*>(tables.ptr[rank]);
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    float gmax = -INFINITY;
    for (int q = 0; q < n; ++q) gmax = fmaxf(gmax, mine[(static_cast<int64_t>(q) * rows + r) * 3]);
    float se = 0.0f, tl = 0.0f;
    for (int q = 0; q < n; ++q) {
      const int64_t b = (static_cast<int64_t>(q) * rows + r) * 3;
      se += mine[b + 1] * __expf(mine[b] - gmax);
      tl += mine[b + 2];
    }
    merged[r * 3] = gmax;
    merged[r * 3 + 1] = se;
    merged[r * 3 + 2] = tl;
  }
}

// ------------------------------------------------------------------------------------------------
// owner's half of the slot form of GEMM -> reduce-scatter: out = residual + sum over the n BF16 slots (rank order)
// ------------------------------------------------------------------------------------------------
template <typename RT, typename OT>
__global__ void __launch_bounds__(256)
sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, int n, int rows, int cols, int64_t ld_slots,
                 const RT* __restrict__ residual, int64_t ld_res, OT* __restrict__ out, int64_t ld_out,
                 __nv_bfloat16* __restrict__ out_lp, int64_t ld_lp, const __nv_bfloat16* __restrict__ own_rows, int own_rank) {
  constexpr int V = 8;
  const int vec_per_row = cols / V;
  const int64_t total = static_cast<int64_t>(rows) * vec_per_row;
  const int64_t slot_stride = static_cast<int64_t>(rows) * ld_slots;
  NX_GRID_STRIDE(i, total) {
    const int r = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i % vec_per_row) * V;
    float acc[V];
    if (residual != nullptr) {
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = Num<RT>::load(residual + static_cast<int64_t>(r) * ld_res + c + j);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.0f;
    }
#pragma unroll 1
    for (int q = 0; q < n; ++q) {
      const __nv_bfloat16* base = (own_rows != nullptr && q == own_rank) ? own_rows : slots + q * slot_stride;
      const uint4 raw = *reinterpret_cast<const uint4*>(base + static_cast<int64_t>(r) * ld_slots + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) Num<OT>::store(out + static_cast<int64_t>(r) * ld_out + c + j, acc[j]);
    if (out_lp != nullptr) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out_lp + static_cast<int64_t>(r) * ld_lp + c) = o;
    }
  }
}

__global__ void bump_kernel(int* counter) { *counter += 1; }

}  // namespace

// ================================================================================================
extern "C" int nx_comm_bump(int* counter, nx_stream_t stream) {
  if (counter == nullptr) return -1;
  bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(counter);
  return launch_status();
}

extern "C" int nx_comm_sum_slots(const void* slots, int n, int rows, int cols, int64_t ld_slots, const void* residual,
                                 int res_dtype, int64_t ld_res, void* out, int out_dtype, int64_t ld_out, void* out_lp,
                                 int64_t ld_lp, const void* own_rows, int own_rank, nx_stream_t stream) {
  if (slots == nullptr || out == nullptr || n < 1 || n > NX_MAX_PEERS || rows <= 0 || cols <= 0 || (cols & 7) ||
      (ld_slots & 7) || (reinterpret_cast<uintptr_t>(slots) & 15) || (out_lp != nullptr && ((ld_lp & 7) ||
      (reinterpret_cast<uintptr_t>(out_lp) & 15))))
    return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t total = static_cast<int64_t>(rows) * (cols / 8);
  const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 16));
  const __nv_bfloat16* sl = static_cast<const __nv_bfloat16*>(slots);
  __nv_bfloat16* lp = static_cast<__nv_bfloat16*>(out_lp);
#define NX_SS(RT, OT) sum_slots_kernel<RT, OT><<<blocks, 256, 0, st>>>(sl, n, rows, cols, ld_slots, static_cast<const RT*>(residual), ld_res, static_cast<OT*>(out), ld_out, lp, ld_lp, static_cast<const __nv_bfloat16*>(own_rows), own_rank)
  const int rd = residual == nullptr ? out_dtype : res_dtype;
  if (rd == NX_F32 && out_dtype == NX_F32) NX_SS(float, float);
  else if (rd == NX_BF16 && out_dtype == NX_BF16) NX_SS(__nv_bfloat16, __nv_bfloat16);
  else if (rd == NX_F32 && out_dtype == NX_BF16) NX_SS(float, __nv_bfloat16);
  else if (rd == NX_BF16 && out_dtype == NX_F32) NX_SS(__nv_bfloat16, float);
  else return -1;
#undef NX_SS
  return launch_status();
}

extern "C" int nx_comm_barrier(const NxPeerTable* flags, int rank, int n, int* counter, int* status, nx_stream_t stream) {
  if (flags == nullptr || n < 1 || n > NX_MAX_PEERS || rank < 0 || rank >= n || status == nullptr || counter == nullptr)
    return -1;
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(*flags, rank, n, counter, status);
  return launch_status();
}

extern "C" int64_t nx_comm_reduce_partials(int64_t count) { return (count + kReduceChunk - 1) / kReduceChunk; }

extern "C" int nx_comm_reduce_shard(const NxPeerTable* grads, int n, int64_t shard_off, int64_t count, float scale,
                                    float* out, double* partial, nx_stream_t stream) {
  if (grads == nullptr || n < 1 || n > NX_MAX_PEERS || count <= 0 || (shard_off & 3)) return -1;
  const int blocks = static_cast<int>((count + kReduceChunk - 1) / kReduceChunk);
  reduce_shard_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(*grads, n, shard_off, count, scale, out,
                                                                              partial);
  return launch_status();
}

extern "C" int nx_comm_norm_exchange(const double* partial, int nparts, const NxPeerTable* slots,
                                     const NxPeerTable* flags, int rank, int n, int* counter, NxOptState* state,
                                     int* status, nx_stream_t stream) {
  if (slots == nullptr || flags == nullptr || n < 1 || n > NX_MAX_PEERS || status == nullptr) return -1;
  norm_exchange_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(partial, nparts, *slots, *flags, rank, n, counter,
                                                                         state, status);
  return launch_status();
}

extern "C" int nx_comm_adamw_allgather(float* master, const float* grad, float* m, float* v,
                                       const NxPeerTable* shadows, const NxPeerTable* fp32_tails,
                                       int64_t tail_off, int n, int64_t shard_off, const NxAdamChunk* chunks,
                                       int nchunks, const NxOptState* state, nx_stream_t stream) {
  if (shadows == nullptr || n < 1 || n > NX_MAX_PEERS || nchunks <= 0) return -1;
  NxPeerTable none = {};
  adamw_shard_allgather_kernel<<<nchunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, grad, m, v, *shadows, fp32_tails ? *fp32_tails : none, fp32_tails ? tail_off : -1, n, shard_off, chunks,
      state);
  return launch_status();
}

extern "C" int nx_comm_allreduce_shard(const NxPeerTable* in, int in_dtype, int n_in, const NxPeerTable* out,
                                       int out_dtype, int n_out, int64_t shard_off, int64_t count, float scale,
                                       nx_stream_t stream) {
  if (in == nullptr || out == nullptr || n_in < 1 || n_in > NX_MAX_PEERS || n_out < 1 || n_out > NX_MAX_PEERS) return -1;
  if (count <= 0) return 0;
  if ((shard_off & 7) || (count & 7)) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = blocks_for(count / 8, 256, 148 * 8);
#define NX_AR(IT, OT) allreduce_shard_kernel<IT, OT><<<blocks, 256, 0, st>>>(*in, n_in, *out, n_out, shard_off, count, scale)
  if (in_dtype == NX_F32 && out_dtype == NX_F32) NX_AR(float, float);
  else if (in_dtype == NX_BF16 && out_dtype == NX_F32) NX_AR(__nv_bfloat16, float);
  else if (in_dtype == NX_BF16 && out_dtype == NX_BF16) NX_AR(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == NX_F32 && out_dtype == NX_BF16) NX_AR(float, __nv_bfloat16);
  else return -1;
#undef NX_AR
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// All-gather by peer loads: out[q * shard + i] = shards[q][i] for every rank q (16-byte vectors; `shard` counts
// vectors).  The FullShard engine gathers a unit's parameter shards with it before the unit's forward / backward.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_shards_kernel(NxPeerTable shards, int n, int64_t shard_vecs, uint4* __restrict__ out) {
  const int64_t total = shard_vecs * n;
  NX_GRID_STRIDE(i, total) {
    const int q = static_cast<int>(i / shard_vecs);
    out[i] = reinterpret_cast<const uint4*>(shards.ptr[q])[i - q * shard_vecs];
  }
}

extern "C" int nx_comm_gather_shards(const NxPeerTable* shards, int n, int64_t shard_bytes, void* out, nx_stream_t stream) {
  if (shards == nullptr || out == nullptr || n < 1 || n > NX_MAX_PEERS || shard_bytes < 0 || (shard_bytes & 15)) return -1;
  if (shard_bytes == 0) return 0;
  const int64_t vecs = shard_bytes / 16;
  gather_shards_kernel<<<blocks_for(vecs * n, 256, 148 * 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      *shards, n, vecs, static_cast<uint4*>(out));
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// In-switch all-reduce (NVLS): `mc` is the multicast address of a symmetric buffer, i.e. one address that stands for
// the same offset in every rank's copy.  `multimem.ld_reduce` makes NVSwitch read the 16 bytes from every rank and
// return their sum (FP32 accumulation), `multimem.st` writes the result into every rank's copy: a rank moves its
// slice over its own links once in each direction, whatever the number of ranks.
// ---------------------------------------------------------------------------------------------
template <bool BF16>
__device__ __forceinline__ void multimem_ld_reduce(uint64_t addr, uint32_t (&r)[4]) {
  if (BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "l"(addr)
                 : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "l"(addr)
                 : "memory");
}
template <bool BF16>
__device__ __forceinline__ void multimem_st(uint64_t addr, const uint32_t (&r)[4]) {
  if (BF16)
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3])
                 : "memory");
  else
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3])
                 : "memory");
}
template <bool BF16>
__device__ __forceinline__ void multimem_scale(uint32_t (&r)[4], float scale) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (BF16) {
      float lo, hi;
      nx::unpack_bf16x2(r[j], lo, hi);
      r[j] = nx::pack_bf16x2(lo * scale, hi * scale);
    } else {
      r[j] = __float_as_uint(__uint_as_float(r[j]) * scale);
    }
  }
}

template <bool BF16>
__global__ void __launch_bounds__(256) allreduce_multimem_kernel(uint8_t* mc, int64_t off_bytes, int64_t vecs, float scale) {
  constexpr int U = 4;  // reductions in flight per thread
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const uint64_t base = reinterpret_cast<uint64_t>(mc) + static_cast<uint64_t>(off_bytes);
  for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < vecs; i0 += stride * U) {
    uint32_t r[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < vecs) multimem_ld_reduce<BF16>(base + static_cast<uint64_t>(i0 + u * stride) * 16, r[u]);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i0 + u * stride < vecs) {
        if (scale != 1.0f) multimem_scale<BF16>(r[u], scale);
        multimem_st<BF16>(base + static_cast<uint64_t>(i0 + u * stride) * 16, r[u]);
      }
  }
  __threadfence_system();  // the stores are out before the barrier kernel that follows signals the peers
}

// ---------------------------------------------------------------------------------------------
// The sharded optimizer through NVSwitch.  Reduce-scatter: the owner asks the switch for the sum of its shard of the
// gradients (`multimem.ld_reduce` on the multicast address of the symmetric gradient buffer), so 1 / n of the buffer
// enters each GPU instead of (n - 1) / n; the square sum for the norm is formed in the same pass.  All-gather: the
// owner's AdamW writes every updated BF16 weight (and FP32 norm / bias value) once with `multimem.st`, which lands in
// every rank's copy, instead of once per peer.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
reduce_shard_multimem_kernel(const uint8_t* __restrict__ mc, int64_t shard_off, int64_t count, float scale,
                             float* __restrict__ out, double* __restrict__ partial) {
  __shared__ double s_scratch[32];
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kReduceChunk;
  const int64_t end = min(count, begin + kReduceChunk);
  const uint64_t base = reinterpret_cast<uint64_t>(mc) + static_cast<uint64_t>(shard_off) * 4;
  double sq = 0.0;
  for (int64_t i = begin + threadIdx.x * 4; i < end; i += blockDim.x * 4) {
    if (i + 4 <= end) {
      uint32_t r[4];
      multimem_ld_reduce<false>(base + static_cast<uint64_t>(i) * 4, r);
      float4 acc = make_float4(__uint_as_float(r[0]) * scale, __uint_as_float(r[1]) * scale, __uint_as_float(r[2]) * scale,
                               __uint_as_float(r[3]) * scale);
      *reinterpret_cast<float4*>(out + i) = acc;
      sq += static_cast<double>(acc.x) * acc.x + static_cast<double>(acc.y) * acc.y +
            static_cast<double>(acc.z) * acc.z + static_cast<double>(acc.w) * acc.w;
    } else {
      for (int64_t j = i; j < end; ++j) {
        float a;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f32 %0, [%1];" : "=f"(a) : "l"(base + static_cast<uint64_t>(j) * 4) : "memory");
        a *= scale;
        out[j] = a;
        sq += static_cast<double>(a) * a;
      }
    }
  }
  sq = block_sum<double>(sq, s_scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = sq;
}

// `adamw_shard_allgather_kernel` with the results stored through the multicast addresses of the BF16 shadow and the
// FP32 tail.  Eight parameters per thread where the global index allows a 16-byte store, one at a time at ragged ends.
__global__ void __launch_bounds__(256)
adamw_shard_multimem_kernel(float* __restrict__ master, const float* __restrict__ grad, float* __restrict__ m,
                            float* __restrict__ v, uint8_t* __restrict__ shadow_mc, uint8_t* __restrict__ tail_mc,
                            NxPeerTable shadows, int n, int64_t tail_off, int64_t shard_off,
                            const NxAdamChunk* __restrict__ chunks, const NxOptState* __restrict__ st) {
  if (st->found_inf) return;
  const NxAdamChunk ch = chunks[blockIdx.x];
  const float lr = __fmul_rn(st->lr, ch.lr_scale);
  const float wd = __fmul_rn(st->weight_decay, ch.wd_scale);
  const float b1 = st->beta1, b2 = st->beta2, omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  const float i1 = st->inv_bias1, i2 = st->inv_bias2, eps = st->eps, clip = st->clip_coef;
  const float lrwd = __fmul_rn(lr, wd);
  auto update = [&](int64_t gi) -> float {   // same operation order as adamw_kernel
    const int64_t i = gi - shard_off;
    const float g = __fmul_rn(grad[i], clip);
    float p = master[i];
    p = __fsub_rn(p, __fmul_rn(lrwd, p));
    const float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(omb1, g));
    const float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(omb2, __fmul_rn(g, g)));
    p = __fsub_rn(p, __fdiv_rn(__fmul_rn(lr, __fmul_rn(mi, i1)), __fadd_rn(__fsqrt_rn(__fmul_rn(vi, i2)), eps)));
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    return p;
  };
  auto store_one = [&](int64_t gi, float p) {   // a multicast store is at least 32 bits wide: single BF16 values go peer by peer
    const __nv_bfloat16 lp = __float2bfloat16_rn(p);
#pragma unroll 1
    for (int q = 0; q < n; ++q) reinterpret_cast<__nv_bfloat16*>(shadows.ptr[q])[gi] = lp;
    if (tail_off >= 0 && gi >= tail_off)
      asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(tail_mc) + static_cast<uint64_t>(gi - tail_off) * 4), "f"(p) : "memory");
  };
  const int64_t lo = ch.offset, hi = ch.offset + ch.count;
  const int64_t a0 = min(hi, (lo + 7) / 8 * 8), a1 = max(a0, hi / 8 * 8);   // [a0, a1): whole groups of 8 by global index
  for (int64_t gi = lo + threadIdx.x; gi < a0; gi += blockDim.x) store_one(gi, update(gi));
  for (int64_t gi = a1 + threadIdx.x; gi < hi; gi += blockDim.x) store_one(gi, update(gi));
  for (int64_t g8 = a0 + static_cast<int64_t>(threadIdx.x) * 8; g8 < a1; g8 += static_cast<int64_t>(blockDim.x) * 8) {
    float p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = update(g8 + j);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = nx::pack_bf16x2(p[2 * j], p[2 * j + 1]);
    multimem_st<false>(reinterpret_cast<uint64_t>(shadow_mc) + static_cast<uint64_t>(g8) * 2, w);
    if (tail_off >= 0 && g8 + 8 > tail_off) {
      const int64_t t = g8 - tail_off;
      if (t >= 0 && (t & 3) == 0) {
        uint32_t f0[4] = {__float_as_uint(p[0]), __float_as_uint(p[1]), __float_as_uint(p[2]), __float_as_uint(p[3])};
        uint32_t f1[4] = {__float_as_uint(p[4]), __float_as_uint(p[5]), __float_as_uint(p[6]), __float_as_uint(p[7])};
        multimem_st<false>(reinterpret_cast<uint64_t>(tail_mc) + static_cast<uint64_t>(t) * 4, f0);
        multimem_st<false>(reinterpret_cast<uint64_t>(tail_mc) + static_cast<uint64_t>(t + 4) * 4, f1);
      } else {   // the tail starts inside this group, or on an odd 16-byte phase
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (t + j >= 0)
            asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(tail_mc) + static_cast<uint64_t>(t + j) * 4), "f"(p[j]) : "memory");
      }
    }
  }
  __threadfence_system();
}

extern "C" int nx_comm_reduce_shard_multimem(void* grads_mc, int64_t shard_off, int64_t count, float scale, float* out,
                                             double* partial, nx_stream_t stream) {
  if (grads_mc == nullptr || count <= 0 || (shard_off & 3)) return -1;
  const int blocks = static_cast<int>((count + kReduceChunk - 1) / kReduceChunk);
  reduce_shard_multimem_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(grads_mc), shard_off, count, scale, out, partial);
  return launch_status();
}

extern "C" int nx_comm_adamw_allgather_multimem(float* master, const float* grad, float* m, float* v, void* shadow_mc,
                                                void* tail_mc, const NxPeerTable* shadows, int n, int64_t tail_off,
                                                int64_t shard_off, const NxAdamChunk* chunks, int nchunks,
                                                const NxOptState* state, nx_stream_t stream) {
  if (shadow_mc == nullptr || shadows == nullptr || n < 1 || n > NX_MAX_PEERS || nchunks <= 0 ||
      (tail_mc == nullptr && tail_off >= 0))
    return -1;
  adamw_shard_multimem_kernel<<<nchunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, grad, m, v, static_cast<uint8_t*>(shadow_mc), static_cast<uint8_t*>(tail_mc), *shadows, n, tail_off,
      shard_off, chunks, state);
  return launch_status();
}

extern "C" int nx_comm_allreduce_multimem(void* multicast_ptr, int dtype, int64_t shard_off, int64_t count, float scale,
                                          nx_stream_t stream) {
  if (multicast_ptr == nullptr || (dtype != NX_F32 && dtype != NX_BF16)) return -1;
  if (count <= 0) return 0;
  const int per_vec = dtype == NX_F32 ? 4 : 8;
  if ((shard_off % per_vec) || (count % per_vec)) return -1;
  const int64_t vecs = count / per_vec;
  const int64_t off_bytes = shard_off * (dtype == NX_F32 ? 4 : 2);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int blocks = blocks_for(vecs, 256, 148 * 4);
  if (dtype == NX_F32) allreduce_multimem_kernel<false><<<blocks, 256, 0, st>>>(static_cast<uint8_t*>(multicast_ptr), off_bytes, vecs, scale);
  else allreduce_multimem_kernel<true><<<blocks, 256, 0, st>>>(static_cast<uint8_t*>(multicast_ptr), off_bytes, vecs, scale);
  return launch_status();
}

extern "C" int nx_comm_a2a_heads(const void* x, const NxPeerTable* out, int B, int Tl, int H, int D, int rank, int n,
                                 int mode, nx_stream_t stream) {
  if (out == nullptr || n < 1 || n > NX_MAX_PEERS || H % n || (D & 7) || mode < 0 || mode > 1) return -1;
  const int64_t total = static_cast<int64_t>(B) * Tl * H * (D / 8);
  if (total <= 0) return 0;
  a2a_heads_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), *out, B, Tl, H, D, rank, n, mode);
  return launch_status();
}

extern "C" int nx_moe_dispatch(const void* x, const int32_t* token_of, const int32_t* expert_of, const int32_t* slot_of,
                               const NxPeerTable* bufs, int rows, int d, int local_experts, int capacity, int src_rank,
                               int n_ranks, const float* row_scale, int rows_per_token, nx_stream_t stream) {
  if (bufs == nullptr || rows < 0 || d <= 0 || (d & 7)) return -1;
  if (rows == 0) return 0;
  const int blocks = rows < 148 * 8 ? rows : 148 * 8;
  moe_dispatch_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), token_of, expert_of, slot_of, *bufs, rows, d, local_experts, capacity,
      src_rank, n_ranks, row_scale, rows_per_token < 1 ? 1 : rows_per_token);
  return launch_status();
}

extern "C" int nx_moe_combine(const NxPeerTable* bufs, const int32_t* expert, const int32_t* slot, const float* gate,
                              void* y, int tokens, int top_k, int d, int local_experts, int capacity,
                              nx_stream_t stream) {
  if (bufs == nullptr || tokens <= 0 || d <= 0 || (d & 7)) return -1;
  const int blocks = tokens < 148 * 8 ? tokens : 148 * 8;
  moe_combine_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      *bufs, expert, slot, gate, static_cast<__nv_bfloat16*>(y), tokens, top_k, d, local_experts, capacity);
  return launch_status();
}

extern "C" int nx_moe_gate_grad_peers(const void* dy, const NxPeerTable* bufs, const int32_t* expert, const int32_t* slot,
                                      float* dgate, int tokens, int top_k, int d, int local_experts, int capacity,
                                      nx_stream_t stream) {
  const int entries = tokens * top_k;
  if (entries <= 0) return 0;
  if (bufs == nullptr || (d & 7)) return -1;
  moe_gate_grad_peers_kernel<<<(entries + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), *bufs, expert, slot, dgate, entries, top_k, d, local_experts, capacity);
  return launch_status();
}

extern "C" int nx_vocab_ce_exchange(const float* local_stats, const NxPeerTable* tables, const NxPeerTable* flags,
                                    int rank, int n, int rows, int* counter, float* merged, int* status,
                                    nx_stream_t stream) {
  if (tables == nullptr || flags == nullptr || counter == nullptr || n < 1 || n > NX_MAX_PEERS || rows <= 0) return -1;
  vocab_ce_exchange_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(local_stats, *tables, *flags, rank, n,
                                                                              rows, counter, merged, status);
  return launch_status();
}
