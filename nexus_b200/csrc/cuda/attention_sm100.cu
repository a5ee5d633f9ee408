// Flash-style attention for sm_100a on tcgen05 tensor cores: forward, and a two-kernel
// deterministic backward (dQ kernel with the q block resident, which also forms rowsum(dO * O), then the
// dK/dV kernel with the kv block resident; no atomics, every gradient tile accumulates in TMEM).
//
// Shared design:
//   * Q/K/V/dO tiles arrive by TMA (4-D maps over [B, T, H, D] with arbitrary strides, so packed
//     QKV needs no split kernel) into 128B-swizzled shared memory;
//   * one elected thread issues tcgen05.mma; score tiles live in TMEM; each softmax thread owns one
//     TMEM lane (= one row), so row statistics need no shuffles;
//   * probabilities / dS are written back to swizzled shared memory as BF16 operands of the next MMA;
//   * the same shared-memory tile is consumed K-major or MN-major just by changing the descriptor,
//     which replaces every explicit transpose of a mma.sync implementation;
//   * every mbarrier wait is bounded and reports through the status word.
//
// Features: causal, sliding window, GQA (H % Hkv == 0), Tq != Tk (bottom-right aligned causal
// mask), head_dim 64 or 128, softmax scale.  Parity: src/cuda/flash_attention.cu:230-857 and
// include/nexus/attention/params.hpp:18-46 of the reference (which uses mma.sync m16n8k16).
#include "nx_api_attention.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"
#include <algorithm>
#include <cstdlib>
#include <type_traits>

namespace {
using namespace nx;

constexpr int kThreads = 192;  // warps 0-3: softmax / row math, warp 4: TMA, warp 5: MMA + TMEM
constexpr float kLog2e = 1.4426950408889634f;

struct AttnDev {
  void* out;        // fwd: O [B,Tq,H,D] bf16;   dq kernel: dQ;   dkdv kernel: dK
  void* out2;       // dkdv kernel: dV
  float* lse;       // [B,H,Tq] natural-log LSE (fwd: written; bwd: read)
  const float* dsum;  // [B,H,Tq] rowsum(dO * O) (bwd)
  int* status;
  int64_t o_row, o_head, o_batch;      // element strides of `out`
  int64_t o2_row, o2_head, o2_batch;   // element strides of `out2`
  int B, H, Hkv, Tq, Tk;
  int causal, window;  // window <= 0: unlimited
  int hfirst;          // TMA coordinate order, see load_tile
  float scale;
  int items, nqb;      // fwd (persistent): number of work items = nqb * H * B, q blocks per (head, batch)
  float* merge_o;      // fwd: FP32 [B,Tq,H,D] running output of earlier key/value chunks (in/out), or null
  float* merge_lse;    // fwd: FP32 [B,H,Tq] running log-sum-exp (in/out)
  float softcap;       // > 0: scores pass through softcap * tanh(scale * s / softcap)
  const float* alibi;  // [H] slopes or null: slope_h * (key position - query position) is added to the scaled score
  // dq kernel: forward output and its gradient as plain row views; the kernel forms dsum = rowsum(dO * O) itself
  // and leaves it in `dsum_out` for the dK/dV kernel that follows
  const __nv_bfloat16* o_in;
  const __nv_bfloat16* do_in;
  int64_t oi_row, oi_head, oi_batch, di_row, di_head, di_batch;
  float* dsum_out;
  float dropout_p;     // > 0: probabilities are dropped with this rate (the row sums are not)
  uint64_t drop_seed, drop_offset;  // Philox stream; element ((b*H + h)*Tq + q)*Tk + k of it decides P[b,h,q,k]
};

// Philox4x32-10, the generator of every dropout in this library: element i of a stream uses counter block
// offset + i / 4 and lane i % 4; u = top 24 bits / 2^24; an element is kept iff u >= p.
__device__ __forceinline__ void attn_philox4x32_10(uint32_t (&ctr)[4], uint32_t k0, uint32_t k1) {
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

// Soft-capping and ALiBi, folded into an "effective raw score" s' with scale * s' = cap * tanh(scale * s / cap) +
// slope * rel, so that the softmax code downstream stays as it is.  `dfac` receives d(scale * s')/d(scale * s).
struct ScoreExt {
  float scale, inv_scale, cap, inv_cap, slope;
  float drop_p, keep_inv;   // dropout rate and 1 / (1 - rate)
  uint32_t key0, key1;      // Philox key (the seed)
  uint64_t offset, head_base;  // stream offset; flat index of P[b, h, 0, 0]
  int Tk;
};
// 1 / (1 - p) when element `idx` of the stream is kept, 0 when it is dropped
__device__ __forceinline__ float drop_scale(const ScoreExt& e, uint64_t idx) {
  const uint64_t blk = e.offset + (idx >> 2);
  uint32_t ctr[4] = {static_cast<uint32_t>(blk), static_cast<uint32_t>(blk >> 32), 0u, 0u};
  attn_philox4x32_10(ctr, e.key0, e.key1);
  const uint32_t lane = static_cast<uint32_t>(idx) & 3u;
  const uint32_t x = lane == 0 ? ctr[0] : (lane == 1 ? ctr[1] : (lane == 2 ? ctr[2] : ctr[3]));
  const float u = static_cast<float>(x >> 8) * (1.0f / 16777216.0f);
  return u >= e.drop_p ? e.keep_inv : 0.0f;
}
// the same for the probability of query row q (inside its sequence) and key k
__device__ __forceinline__ float drop_scale_qk(const ScoreExt& e, int q, int k) {
  return drop_scale(e, e.head_base + static_cast<uint64_t>(q) * static_cast<uint64_t>(e.Tk) + static_cast<uint64_t>(k));
}
__device__ __forceinline__ ScoreExt make_ext(const AttnDev& p, int head, int batch) {
  ScoreExt e;
  e.drop_p = p.dropout_p;
  e.keep_inv = p.dropout_p > 0.0f ? 1.0f / (1.0f - p.dropout_p) : 1.0f;
  e.key0 = static_cast<uint32_t>(p.drop_seed);
  e.key1 = static_cast<uint32_t>(p.drop_seed >> 32);
  e.offset = p.drop_offset;
  e.head_base = (static_cast<uint64_t>(batch) * p.H + head) * static_cast<uint64_t>(p.Tq) * static_cast<uint64_t>(p.Tk);
  e.Tk = p.Tk;
  e.scale = p.scale;
  e.inv_scale = 1.0f / p.scale;
  e.cap = p.softcap;
  e.inv_cap = p.softcap > 0.0f ? 1.0f / p.softcap : 0.0f;
  e.slope = p.alibi != nullptr ? p.alibi[head] : 0.0f;
  return e;
}
__device__ __forceinline__ float score_ext(const ScoreExt& e, float s, int rel, float& dfac) {
  float z = s * e.scale;
  dfac = 1.0f;
  if (e.cap > 0.0f) {
    const float t = tanh_approx_f(z * e.inv_cap);
    z = e.cap * t;
    dfac = 1.0f - t * t;
  }
  return fmaf(e.slope, static_cast<float>(rel), z) * e.inv_scale;
}
__device__ __forceinline__ float score_ext(const ScoreExt& e, float s, int rel) {
  float d;
  return score_ext(e, s, rel, d);
}

// byte offset of the 16-byte chunk (8 bf16) `chunk` (0..7) of row `r` inside a [rows][64] swizzled slab
__device__ __forceinline__ uint32_t sw128_off(int r, int chunk) {
  return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}

// Load a [rows][HD] tile as HD/64 slabs of [rows][64].
// The map's dimension order follows the memory strides ({D,H,T,B} when heads are interleaved
// inside a token row, {D,T,H,B} when each head owns a contiguous [T, D] plane); `hfirst` selects it.
template <int HD>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int rows, int row0,
                                          int head, int batch, int hfirst) {
  // (debug builds check the tile coordinates at the call sites, where the tensor extents are known: NX_INDEX_OK)
#pragma unroll
  for (int s = 0; s < HD / 64; ++s) {
    if (hfirst)
      tma_load_4d(dst + s * rows * 128, tm, bar, 64 * s, head, row0, batch);
    else
      tma_load_4d(dst + s * rows * 128, tm, bar, 64 * s, row0, head, batch);
  }
}

// K-major operand: address of k-step `ks` (16 elements) in a tile of HD/64 (or cols/64) slabs of `rows` rows.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int rows, int ks) {
  const uint32_t a = tile_addr + static_cast<uint32_t>((ks >> 2) * rows * 128 + (ks & 3) * 32);
  return make_smem_desc_sw128(a, 16, 1024);
}
// MN-major view of a [k_rows][mn] tile stored as mn/64 slabs of [k_rows][64]: k-step `ks` = 16 rows.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int k_rows, int ks) {
  const uint32_t a = tile_addr + static_cast<uint32_t>(ks * 2048);
  return make_smem_desc_sw128(a, static_cast<uint32_t>(k_rows * 128), 1024);
}

// what k-step `ks` adds to the address field (bytes >> 4) of a K-major / MN-major descriptor built for k-step 0
__device__ __forceinline__ uint64_t kstep_kmajor(int rows, int ks) {
  return static_cast<uint64_t>((ks >> 2) * rows * 8 + (ks & 3) * 2);
}
__device__ __forceinline__ uint64_t kstep_mnmajor(int ks) { return static_cast<uint64_t>(ks * 128); }

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Per-row visible key range [lo, hi] (inclusive) under the causal / window / length masks.
__device__ __forceinline__ void row_limits(const AttnDev& p, int q, int& lo, int& hi) {
  const int off = p.Tk - p.Tq;
  hi = p.Tk - 1;
  lo = 0;
  if (p.causal) hi = min(hi, q + off);
  if (p.window > 0) lo = max(lo, q + off - p.window + 1);
}

// Forward softmax helpers.  A score row (128 keys) is shared by two threads of different warps: `c0` is
// the first of the 64 columns this thread owns (0 or 64).
template <bool kMask, bool kExt>
__device__ __forceinline__ float half_row_max(uint32_t taddr, int c0, int k0, int lo, int hi, const ScoreExt& ext,
                                              int qpos) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c0 + cc * 32, v);
    tmem_ld_wait();
    const int clo = lo - k0 - c0 - cc * 32, chi = hi - k0 - c0 - cc * 32;  // valid iff clo <= c <= chi
#pragma unroll
    for (int c = 0; c < 32; c += 4) {
      float s0 = __uint_as_float(v[c]), s1 = __uint_as_float(v[c + 1]), s2 = __uint_as_float(v[c + 2]),
            s3 = __uint_as_float(v[c + 3]);
      if (kExt) {
        const int rel = k0 + c0 + cc * 32 + c - qpos;
        s0 = score_ext(ext, s0, rel);
        s1 = score_ext(ext, s1, rel + 1);
        s2 = score_ext(ext, s2, rel + 2);
        s3 = score_ext(ext, s3, rel + 3);
      }
      if (kMask) {
        if (c < clo || c > chi) s0 = -INFINITY;
        if (c + 1 < clo || c + 1 > chi) s1 = -INFINITY;
        if (c + 2 < clo || c + 2 > chi) s2 = -INFINITY;
        if (c + 3 < clo || c + 3 > chi) s3 = -INFINITY;
      }
      m0 = fmaxf(m0, s0);
      m1 = fmaxf(m1, s1);
      m2 = fmaxf(m2, s2);
      m3 = fmaxf(m3, s3);
    }
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = exp2(S*sc - m) for this thread's 64 keys -> BF16 into slab `c0 / 64` of the swizzled [128][128] tile.
template <bool kMask, bool kExt>
__device__ __forceinline__ float half_softmax_store(uint32_t taddr, uint8_t* sP, int r, int c0, int k0, int lo, int hi,
                                                    float sc, float m_use, const ScoreExt& ext, int qpos, int qoff) {
  float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;
  uint8_t* slab = sP + (c0 >> 6) * (128 * 128);
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + c0 + cc * 32, v);
    tmem_ld_wait();
    const int clo = lo - k0 - c0 - cc * 32, chi = hi - k0 - c0 - cc * 32;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float e[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int c = 8 * g + j;
        float sv = __uint_as_float(v[c]);
        if (kExt) sv = score_ext(ext, sv, k0 + c0 + cc * 32 + c - qpos);
        float x = ex2f(fmaf(sv, sc, -m_use));
        if (kMask && (c < clo || c > chi)) x = 0.0f;
        e[j] = x;
      }
      r0 += e[0] + e[4];
      r1 += e[1] + e[5];
      r2 += e[2] + e[6];
      r3 += e[3] + e[7];
      if (kExt && ext.drop_p > 0.0f) {  // the row sum keeps every probability; the tile that meets V does not
#pragma unroll
        for (int j = 0; j < 8; ++j) e[j] *= drop_scale_qk(ext, qpos - qoff, k0 + c0 + cc * 32 + 8 * g + j);
      }
      uint4 w;
      w.x = pack_bf16x2(e[0], e[1]);
      w.y = pack_bf16x2(e[2], e[3]);
      w.z = pack_bf16x2(e[4], e[5]);
      w.w = pack_bf16x2(e[6], e[7]);
      *reinterpret_cast<uint4*>(slab + sw128_off(r, cc * 4 + g)) = w;
    }
  }
  return (r0 + r1) + (r2 + r3);
}

// barrier among the 256 softmax threads only (the TMA and MMA warps never join it)
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// first/last (exclusive) kv index that any row in [q0, q0+nq) can see
__device__ __forceinline__ void kv_range(const AttnDev& p, int q0, int nq, int& lo, int& hi) {
  const int off = p.Tk - p.Tq;
  hi = p.Tk;
  lo = 0;
  if (p.causal) hi = min(p.Tk, q0 + nq - 1 + off + 1);
  if (p.window > 0) lo = max(0, q0 + off - p.window + 1);
  if (hi < 0) hi = 0;
}

// ================================================================================================
// forward
// ================================================================================================
template <int HD>
struct FwdCfg {
  static constexpr int kQBytes = 128 * HD * 2;
  static constexpr int kKVBytes = 128 * HD * 2;
  static constexpr int kPBytes = 128 * 128 * 2;
  static constexpr int kXchgBytes = 128 * 4;  // row statistics exchanged between the two column halves (two CTAs
                                              // per SM leave no room for a second array)
  static constexpr int kSmem = kQBytes + 4 * kKVBytes + kPBytes + kXchgBytes + 128;
  static constexpr int kTmemCols = 256;  // S: 128, PV: HD
};

constexpr int kFwdThreads = 320;  // warps 0-7: softmax (row quarter = warp & 3, column half = warp >> 2), 8: TMA, 9: MMA

// Work item i of the persistent forward kernel -> (q block, head, batch).  Items are ordered by cost: under
// a causal mask the late q blocks see the most keys, so they come first and the CTAs (which take items
// i, i + grid, i + 2 grid, ...) finish together.
__device__ __forceinline__ void fwd_item(const AttnDev& p, int item, int& qb, int& h, int& b) {
  const int per = p.H * p.B;
  qb = p.nqb - 1 - item / per;
  const int rem = item % per;
  h = rem % p.H;
  b = rem / p.H;
}

template <int HD, bool EXT>  // EXT: soft-capping / ALiBi / dropout row math (a build of its own)
__global__ void __launch_bounds__(kFwdThreads, (HD == 64 ? 2 : 1))
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnDev p) {
  pdl_launch_dependents();
  using C = FwdCfg<HD>;
  constexpr int HH = HD / 2;  // output columns per softmax thread
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base; uniform early exit
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadArgument);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + C::kQBytes;               // 2 stages
  uint8_t* sV = sK + 2 * C::kKVBytes;          // 2 stages
  uint8_t* sP = sV + 2 * C::kKVBytes;          // [128][128] bf16 as 2 slabs
  float* sX = reinterpret_cast<float*>(sP + C::kPBytes);  // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sX + 128);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* p_full = bars + 6;
  uint64_t* o_full = bars + 7;
  uint64_t* q_empty = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 8);  // one arrival per softmax warp
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;

  // every role walks the same item list and keeps its own running counters of items and key tiles
  if (warp == 8) {
    if (lane == 0) {
      int n_item = 0, n_kv = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++n_item) {
        int qb, h, b;
        fwd_item(p, item, qb, h, b);
        const int hk = h / (p.H / p.Hkv);
        const int q0 = qb * 128;
        int kv_lo, kv_hi;
        kv_range(p, q0, min(128, p.Tq - q0), kv_lo, kv_hi);
        const int jb = kv_lo / 128, je = (kv_hi + 127) / 128;
        // debug builds: the item's tile coordinates lie inside the tensors (a tile may run past the end, never start there)
        if (!NX_INDEX_OK(q0 >= 0 && q0 < p.Tq && h >= 0 && h < p.H && hk < p.Hkv && b >= 0 && b < p.B && jb >= 0 &&
                         (je == jb || (je - 1) * 128 < p.Tk), p.status)) {
          *abort_flag = 1;
          break;
        }
        if (!mbar_wait_bounded(q_empty, (n_item & 1) ^ 1u, abort_flag)) {  // the previous item's QK^T are done
          atomicCAS(p.status, 0, kStatusTimeoutProducer);
          break;
        }
        mbar_arrive_expect_tx(q_full, C::kQBytes);
        load_tile<HD>(sQ, &tm_q, q_full, 128, q0, h, b, p.hfirst);
        for (int j = jb; j < je; ++j, ++n_kv) {
          const int s = n_kv & 1;
          if (!mbar_wait_bounded(&kv_empty[s], ((n_kv >> 1) & 1) ^ 1u, abort_flag)) {
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[s], 2 * C::kKVBytes);
          load_tile<HD>(sK + s * C::kKVBytes, &tm_k, &kv_full[s], 128, j * 128, hk, b, p.hfirst);
          load_tile<HD>(sV + s * C::kKVBytes, &tm_v, &kv_full[s], 128, j * 128, hk, b, p.hfirst);
        }
      }
    }
  } else if (warp == 9) {
    // the whole warp walks the loop (descriptors stay in uniform registers); one elected lane issues
    {
      const bool leader = elect_one();
      const uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, false, false, 128, 128);
      const uint32_t idesc_o = make_idesc(kFmtBF16, kFmtBF16, false, true, 128, HD);
      const uint64_t dQ = desc_kmajor(smem_u32(sQ), 128, 0), dP = desc_kmajor(smem_u32(sP), 128, 0);
      int n_item = 0, n_kv = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x, ++n_item) {
        int qb, h, b;
        fwd_item(p, item, qb, h, b);
        const int q0 = qb * 128;
        int kv_lo, kv_hi;
        kv_range(p, q0, min(128, p.Tq - q0), kv_lo, kv_hi);
        const int jb = kv_lo / 128, je = (kv_hi + 127) / 128;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(q_full, n_item & 1, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        for (int j = jb; j < je; ++j, ++n_kv) {
          const int s = n_kv & 1;
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&kv_full[s], (n_kv >> 1) & 1, abort_flag))) {
            if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t dK = desc_kmajor(smem_u32(sK + s * C::kKVBytes), 128, 0);
          const uint64_t dV = desc_mnmajor(smem_u32(sV + s * C::kKVBytes), 128, 0);
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
              umma_f16_ss(tmem_s, dQ + kstep_kmajor(128, ks), dK + kstep_kmajor(128, ks), idesc_s, ks > 0 ? 1u : 0u);
            umma_commit(s_full);
            if (j + 1 == je) umma_commit(q_empty);  // the Q tile may be replaced once these MMAs have read it
          }
          __syncwarp();
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(p_full, n_kv & 1, abort_flag))) {
            if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_f16_ss(tmem_o, dP + kstep_kmajor(128, ks), dV + kstep_mnmajor(ks), idesc_o, ks > 0 ? 1u : 0u);
            umma_commit(o_full);
            umma_commit(&kv_empty[s]);
          }
          __syncwarp();
        }
        if (jb >= je && leader) umma_commit(q_empty);  // nothing visible: release Q at once
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows
    // Two threads (warps w and w + 4) share a row: each owns 64 of the 128 score columns and half of the
    // output columns; they exchange the row maximum through shared memory once per key tile.
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // row inside the q block == TMEM lane
    const int c0 = half * 64;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float sc = p.scale * kLog2e;
    int n_kv = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < p.items && ok; item += gridDim.x) {
      int qb, h, b;
      fwd_item(p, item, qb, h, b);
      const int q0 = qb * 128;
      const int q = q0 + r;
      int kv_lo, kv_hi;
      kv_range(p, q0, min(128, p.Tq - q0), kv_lo, kv_hi);
      const int jb = kv_lo / 128, je = (kv_hi + 127) / 128;
      float m_run = -INFINITY, l_run = 0.0f;  // l_run: partial sum over this thread's columns
      int row_lo, row_hi;
      row_limits(p, q, row_lo, row_hi);
      constexpr bool ext_on = EXT;
      const ScoreExt ext = EXT ? make_ext(p, h, b) : ScoreExt{};
      float o_acc[HH];
#pragma unroll
      for (int c = 0; c < HH; ++c) o_acc[c] = 0.0f;
      for (int j = jb; j < je; ++j, ++n_kv) {
        const int k0 = j * 128;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(s_full, n_kv & 1, abort_flag));
        if (!ok) {
          if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          break;
        }
        tc_fence_after_sync();
        // does this tile need per-element masking?  (uniform over the CTA by construction of the bounds)
        const int off = p.Tk - p.Tq;
        const bool need_mask = (k0 + 128 > p.Tk) || (p.causal && (k0 + 127 > q0 + off)) ||
                               (p.window > 0 && (k0 < q0 + 127 + off - p.window + 1));
        float mx, rs;
        const int qpos = q + off;
        if (ext_on) {
          if (need_mask) mx = half_row_max<true, true>(tmem_s + lane_addr, c0, k0, row_lo, row_hi, ext, qpos);
          else mx = half_row_max<false, true>(tmem_s + lane_addr, c0, k0, row_lo, row_hi, ext, qpos);
        } else {
          if (need_mask) mx = half_row_max<true, false>(tmem_s + lane_addr, c0, k0, row_lo, row_hi, ext, qpos);
          else mx = half_row_max<false, false>(tmem_s + lane_addr, c0, k0, row_lo, row_hi, ext, qpos);
        }
        // second half publishes, first half combines and publishes the row maximum
        if (half == 1) sX[r] = mx;
        softmax_bar();
        if (half == 0) {
          mx = fmaxf(mx, sX[r]);
          sX[r] = mx;
        }
        softmax_bar();
        if (half == 1) mx = sX[r];
        const float m_new = fmaxf(m_run, mx * sc);
        const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;
        const float alpha = ex2f(m_run - m_use);  // m_run == -inf -> 0
        if (ext_on) {
          if (need_mask) rs = half_softmax_store<true, true>(tmem_s + lane_addr, sP, r, c0, k0, row_lo, row_hi, sc, m_use, ext, qpos, off);
          else rs = half_softmax_store<false, true>(tmem_s + lane_addr, sP, r, c0, k0, row_lo, row_hi, sc, m_use, ext, qpos, off);
        } else {
          if (need_mask) rs = half_softmax_store<true, false>(tmem_s + lane_addr, sP, r, c0, k0, row_lo, row_hi, sc, m_use, ext, qpos, off);
          else rs = half_softmax_store<false, false>(tmem_s + lane_addr, sP, r, c0, k0, row_lo, row_hi, sc, m_use, ext, qpos, off);
        }
        l_run = l_run * alpha + rs;
        m_run = m_new;
        fence_proxy_async_smem();  // generic-proxy writes of P -> visible to the tensor core's async proxy
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(o_full, n_kv & 1, abort_flag));
        if (!ok) {
          if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int cc = 0; cc < HH / 32; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_o + lane_addr + half * HH + cc * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) o_acc[cc * 32 + c] = o_acc[cc * 32 + c] * alpha + __uint_as_float(v[c]);
        }
        tc_fence_before_sync();
        softmax_bar();  // the exchanged maxima have been read before the next tile overwrites them
      }
      // the two halves of a row add their partial sums
      if (!ok) l_run = 0.0f;
      if (half == 1) sX[r] = l_run;
      softmax_bar();
      if (half == 0) {
        l_run += sX[r];
        sX[r] = l_run;
      }
      softmax_bar();
      if (half == 1) l_run = sX[r];
      if (ok && q < p.Tq && p.merge_o != nullptr) {
        // merge with the result of earlier key/value chunks: softmax over the union of the key sets
        const int64_t li = (static_cast<int64_t>(b) * p.H + h) * p.Tq + q;
        float* mo = p.merge_o + ((static_cast<int64_t>(b) * p.Tq + q) * p.H + h) * HD + half * HH;
        const float lse_new = l_run > 0.0f ? (m_run / kLog2e + logf(l_run)) : -INFINITY;
        const float lse_old = p.merge_lse[li];
        const float mm = fmaxf(lse_new, lse_old);
        const float w_new = (lse_new == -INFINITY) ? 0.0f : __expf(lse_new - mm);
        const float w_old = (lse_old == -INFINITY) ? 0.0f : __expf(lse_old - mm);
        const float den = w_new + w_old;
        const float c_new = den > 0.0f ? w_new / den / (l_run > 0.0f ? l_run : 1.0f) : 0.0f;
        const float c_old = den > 0.0f ? w_old / den : 0.0f;
#pragma unroll
        for (int g = 0; g < HH / 4; ++g) {
          float4 prev = reinterpret_cast<const float4*>(mo)[g];
          prev.x = prev.x * c_old + o_acc[4 * g + 0] * c_new;
          prev.y = prev.y * c_old + o_acc[4 * g + 1] * c_new;
          prev.z = prev.z * c_old + o_acc[4 * g + 2] * c_new;
          prev.w = prev.w * c_old + o_acc[4 * g + 3] * c_new;
          reinterpret_cast<float4*>(mo)[g] = prev;
          o_acc[4 * g + 0] = prev.x;
          o_acc[4 * g + 1] = prev.y;
          o_acc[4 * g + 2] = prev.z;
          o_acc[4 * g + 3] = prev.w;
        }
        l_run = den > 0.0f ? 1.0f : 0.0f;  // o_acc now holds the normalised merged output
        m_run = (den > 0.0f ? mm + logf(den) : -INFINITY) * kLog2e;
      }
      softmax_bar();  // every thread has read merge_lse / sX before they are written again
      if (ok && q < p.Tq) {
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(b) * p.o_batch +
                              static_cast<int64_t>(q) * p.o_row + static_cast<int64_t>(h) * p.o_head + half * HH;
#pragma unroll
        for (int g = 0; g < HH / 8; ++g) {
          uint4 w;
          w.x = pack_bf16x2(o_acc[8 * g + 0] * inv, o_acc[8 * g + 1] * inv);
          w.y = pack_bf16x2(o_acc[8 * g + 2] * inv, o_acc[8 * g + 3] * inv);
          w.z = pack_bf16x2(o_acc[8 * g + 4] * inv, o_acc[8 * g + 5] * inv);
          w.w = pack_bf16x2(o_acc[8 * g + 6] * inv, o_acc[8 * g + 7] * inv);
          reinterpret_cast<uint4*>(orow)[g] = w;
        }
        if (half == 0) {
          const int64_t li = (static_cast<int64_t>(b) * p.H + h) * p.Tq + q;
          const float lse = l_run > 0.0f ? (m_run / kLog2e + logf(l_run)) : -INFINITY;
          if (p.lse) p.lse[li] = lse;
          if (p.merge_lse) p.merge_lse[li] = lse;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================================================================================
// forward with two q tiles in flight.  One persistent CTA per SM works on 256 query rows of one
// (head, batch) at a time: softmax group A (warps 0-3) owns rows 0-127, group B (warps 4-7) rows
// 128-255, and both walk the same key/value tiles, which are loaded once.  The MMA warp interleaves
//   PV_A(j-1), QK_A(j), PV_B(j-1), QK_B(j)
// so the tensor core works on one tile while the other tile's exponentials run.  Each softmax thread
// owns a whole score row (its TMEM lane), so no row statistic crosses threads.  The output tile
// accumulates in TMEM across key tiles; it is rescaled (by the row's own thread) only when the running
// maximum has grown by more than 2^8, otherwise the stale maximum stays the reference of the
// exponentials, and the last step divides by the matching row sum.
// TMEM (512 columns): S_A 0-127, S_B 128-255, O_A 256.., O_B 384..
// Probabilities go back as BF16 into the first 64 columns of the score tile itself, two per column, and the
// P V MMA reads them from TMEM as its A operand, so they never touch shared memory.  (A variant that wrote P
// to swizzled shared memory and issued the next Q K^T as soon as the scores were in registers measured slower,
// 105 us against 93 us on 16 x 12 x 1024 x 64, as did four softmax warps more per tile, 118 us.)
// ================================================================================================
template <int HD>
struct Fwd2Cfg {
  static constexpr int kStages = (HD == 64) ? 3 : 2;
  static constexpr int kQBytes = 128 * HD * 2;
  static constexpr int kKVBytes = 128 * HD * 2;
  static constexpr int kSmem = 2 * kQBytes + kStages * 2 * kKVBytes + 256;
  static constexpr int kTmemCols = 512;
};
constexpr int kFwd2Threads = 320;  // warps 0-3: softmax A, 4-7: softmax B, 8: TMA, 9: MMA
constexpr float kRescaleStep = 8.0f;  // log2 of the growth of the row maximum that forces a rescale

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (128 rows on the lanes, two BF16 per column along K) is read from TMEM
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Work of one round of the persistent loop: CTA c takes item round * grid + c in even rounds and
// round * grid + (grid - 1 - c) in odd ones, and the items are sorted by cost (late q blocks first under a causal
// mask), so that the CTAs' totals stay close.  Key tile ranges [jb, je) are per q tile; an absent tile has jb == je.
struct PairWork {
  int q0, h, b;
  int jbA, jeA, jbB, jeB, jb, je;
};
__device__ __forceinline__ bool pair_work(const AttnDev& p, int round, PairWork& w) {
  const int G = static_cast<int>(gridDim.x), c = static_cast<int>(blockIdx.x);
  const int item = round * G + ((round & 1) ? (G - 1 - c) : c);
  if (item >= p.items) return false;
  const int per = p.H * p.B;
  const int qb = p.nqb - 1 - item / per;
  const int rem = item % per;
  w.h = rem % p.H;
  w.b = rem / p.H;
  w.q0 = qb * 256;
  int lo, hi;
  kv_range(p, w.q0, min(128, p.Tq - w.q0), lo, hi);
  w.jbA = lo / 128;
  w.jeA = (hi + 127) / 128;
  if (w.jeA <= w.jbA) w.jbA = w.jeA = 0;
  w.jbB = w.jeB = 0;
  if (w.q0 + 128 < p.Tq) {
    kv_range(p, w.q0 + 128, min(128, p.Tq - w.q0 - 128), lo, hi);
    w.jbB = lo / 128;
    w.jeB = (hi + 127) / 128;
    if (w.jeB <= w.jbB) w.jbB = w.jeB = 0;
  }
  const bool a = w.jeA > w.jbA, bb = w.jeB > w.jbB;
  w.jb = a ? (bb ? min(w.jbA, w.jbB) : w.jbA) : w.jbB;
  w.je = a ? (bb ? max(w.jeA, w.jeB) : w.jeA) : w.jeB;
  if (!a && !bb) w.jb = w.je = 0;
  return true;
}

template <int HD>
__global__ void __launch_bounds__(kFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnDev p) {
  pdl_launch_dependents();
  using C = Fwd2Cfg<HD>;
  constexpr int S = C::kStages;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base; uniform early exit
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadArgument);
    return;
  }
  uint8_t* sQ = smem;                             // [2] q tiles
  uint8_t* sK = sQ + 2 * C::kQBytes;              // [S]
  uint8_t* sV = sK + S * C::kKVBytes;             // [S]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + S * C::kKVBytes);
  uint64_t* q_full = bars;         // [2]
  uint64_t* q_empty = bars + 2;    // [2]
  uint64_t* kv_full = bars + 4;    // [S]
  uint64_t* kv_empty = bars + 7;   // [S]
  uint64_t* s_full = bars + 10;    // [2]
  uint64_t* p_full = bars + 12;    // [2]
  uint64_t* o_done = bars + 14;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int x = 0; x < 2; ++x) {
      mbar_init(&q_full[x], 1);
      mbar_init(&q_empty[x], 1);
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x], 4);  // one arrival per softmax warp of the group
      mbar_init(&o_done[x], 1);
    }
    for (int s = 0; s < S; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      int nq[2] = {0, 0}, n_kv = 0;
      bool ok = true;
      PairWork w;
      for (int round = 0; ok && pair_work(p, round, w); ++round) {
        const int hk = w.h / (p.H / p.Hkv);
        if (!NX_INDEX_OK(w.q0 >= 0 && w.q0 < p.Tq && w.h < p.H && hk < p.Hkv && w.b < p.B && w.jb >= 0 &&
                         (w.je == w.jb || (w.je - 1) * 128 < p.Tk), p.status)) {
          *abort_flag = 1;
          break;
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const bool active = x == 0 ? (w.jeA > w.jbA) : (w.jeB > w.jbB);
          if (!active) continue;
          if (!mbar_wait_bounded(&q_empty[x], (nq[x] & 1) ^ 1u, abort_flag)) {  // the previous item's QK^T are done
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          ++nq[x];
          mbar_arrive_expect_tx(&q_full[x], C::kQBytes);
          load_tile<HD>(sQ + x * C::kQBytes, &tm_q, &q_full[x], 128, w.q0 + x * 128, w.h, w.b, p.hfirst);
        }
        for (int j = w.jb; ok && j < w.je; ++j, ++n_kv) {
          const int s = n_kv % S;
          if (!mbar_wait_bounded(&kv_empty[s], ((n_kv / S) & 1) ^ 1u, abort_flag)) {
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&kv_full[s], 2 * C::kKVBytes);
          load_tile<HD>(sK + s * C::kKVBytes, &tm_k, &kv_full[s], 128, j * 128, hk, w.b, p.hfirst);
          load_tile<HD>(sV + s * C::kKVBytes, &tm_v, &kv_full[s], 128, j * 128, hk, w.b, p.hfirst);
        }
      }
    }
  } else if (warp == 9) {
    // Every lane walks the loop (uniform control flow keeps the descriptors in uniform registers); one elected lane
    // issues the MMAs and commits.
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, false, false, 128, 128);
    const uint32_t idesc_o = make_idesc(kFmtBF16, kFmtBF16, false, true, 128, HD);
    int nqA = 0, nqB = 0, npA = 0, npB = 0, n_kv = 0;
    bool ok = true;
    PairWork w;
    for (int round = 0; ok && pair_work(p, round, w); ++round) {
      if (w.jeA > w.jbA) {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&q_full[0], nqA & 1, abort_flag));
        ++nqA;
      }
      if (ok && w.jeB > w.jbB) {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&q_full[1], nqB & 1, abort_flag));
        ++nqB;
      }
      if (!ok) {
        if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
        break;
      }
      const int kv0 = n_kv;  // key tile j of this item sits in stage (kv0 + j - jb) % S
      for (int j = w.jb; ok && j <= w.je; ++j) {
        if (j < w.je) {
          const int n = kv0 + (j - w.jb);
          ok = __all_sync(0xffffffffu, mbar_wait_bounded(&kv_full[n % S], (n / S) & 1, abort_flag));
          if (!ok) {
            if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
            break;
          }
        }
        const int sj = (kv0 + (j - w.jb)) % S, sjm = (kv0 + (j - w.jb) + S - 1) % S;
        const uint64_t dK = desc_kmajor(smem_u32(sK + sj * C::kKVBytes), 128, 0);
        const uint64_t dV = desc_mnmajor(smem_u32(sV + sjm * C::kKVBytes), 128, 0);
        // P aliases S, so per tile the order is P V (j-1), then Q K^T (j); the two tiles alternate
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int jbx = x == 0 ? w.jbA : w.jbB, jex = x == 0 ? w.jeA : w.jeB;
          const uint32_t tmem_s = tmem_base + x * 128, tmem_o = tmem_base + 256 + x * 128;
          if (ok && j - 1 >= jbx && j - 1 < jex) {  // P_x(j-1) @ V(j-1)
            const int np = x == 0 ? npA : npB;
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&p_full[x], np & 1, abort_flag));
            if (!ok) {
              if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
            } else {
              if (x == 0) ++npA;
              else ++npB;
              tc_fence_after_sync();
              const uint32_t acc0 = (j - 1 > jbx) ? 1u : 0u;
              if (leader) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)  // one k-step = 16 keys = 8 TMEM columns of packed P, 2 KiB of the V tile
                  umma_f16_ts(tmem_o, tmem_s + ks * 8, dV + kstep_mnmajor(ks), idesc_o, (ks > 0) ? 1u : acc0);
                umma_commit(&o_done[x]);
              }
            }
          }
          if (ok && j >= jbx && j < jex) {  // S_x(j) = Q_x K(j)^T
            tc_fence_after_sync();
            const uint64_t dQ = desc_kmajor(smem_u32(sQ + x * C::kQBytes), 128, 0);
            if (leader) {
#pragma unroll
              for (int ks = 0; ks < HD / 16; ++ks)
                umma_f16_ss(tmem_s, dQ + kstep_kmajor(128, ks), dK + kstep_kmajor(128, ks), idesc_s, ks > 0 ? 1u : 0u);
              umma_commit(&s_full[x]);
              if (j + 1 == jex) umma_commit(&q_empty[x]);  // the Q tile may be replaced once these MMAs have read it
            }
          }
        }
        if (ok && j > w.jb && leader) umma_commit(&kv_empty[sjm]);  // both tiles are done with key tile j - 1
        __syncwarp();
      }
      n_kv = kv0 + (w.je - w.jb);
    }
  } else {
    // ------------------------------------------------------------------ softmax + output rows
    const int x = warp >> 2;                      // q tile of this group
    const int r = (warp & 3) * 32 + lane;         // row inside the q tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + x * 128 + lane_addr, tmem_o = tmem_base + 256 + x * 128 + lane_addr;
    const float sc = p.scale * kLog2e;
    const int off = p.Tk - p.Tq;
    int cnt = 0;  // key tiles this group has processed: phase counter of s_full / o_done
    bool ok = true;
    PairWork w;
    for (int round = 0; ok && pair_work(p, round, w); ++round) {
      const int jbx = x == 0 ? w.jbA : w.jbB, jex = x == 0 ? w.jeA : w.jeB;
      if (jex <= jbx) {
        // no visible key for any row of this tile: rows that exist get zeros and -inf (nothing to merge either)
        const int q0x = w.q0 + x * 128, q = q0x + r;
        if (q < p.Tq && q0x < p.Tq) {
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(w.b) * p.o_batch +
                                static_cast<int64_t>(q) * p.o_row + static_cast<int64_t>(w.h) * p.o_head;
          const int64_t li = (static_cast<int64_t>(w.b) * p.H + w.h) * p.Tq + q;
          if (p.merge_o == nullptr) {
#pragma unroll
            for (int g = 0; g < HD / 8; ++g) reinterpret_cast<uint4*>(orow)[g] = make_uint4(0u, 0u, 0u, 0u);
            if (p.lse) p.lse[li] = -INFINITY;
          } else {
            const float* mo = p.merge_o + ((static_cast<int64_t>(w.b) * p.Tq + q) * p.H + w.h) * HD;
#pragma unroll
            for (int g = 0; g < HD / 8; ++g) {
              const float4 u0 = reinterpret_cast<const float4*>(mo)[2 * g], u1 = reinterpret_cast<const float4*>(mo)[2 * g + 1];
              uint4 wv;
              wv.x = pack_bf16x2(u0.x, u0.y);
              wv.y = pack_bf16x2(u0.z, u0.w);
              wv.z = pack_bf16x2(u1.x, u1.y);
              wv.w = pack_bf16x2(u1.z, u1.w);
              reinterpret_cast<uint4*>(orow)[g] = wv;
            }
            if (p.lse) p.lse[li] = p.merge_lse[li];
          }
        }
        continue;
      }
      const int q0 = w.q0 + x * 128;
      const int q = q0 + r;
      int row_lo, row_hi;
      row_limits(p, q, row_lo, row_hi);
      float m_ref = -INFINITY, l_run = 0.0f;
      for (int j = jbx; j < jex; ++j, ++cnt) {
        const int k0 = j * 128;
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&s_full[x], cnt & 1, abort_flag));
        if (!ok) {
          if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          break;
        }
        tc_fence_after_sync();
        // the whole row in registers with one wait: a TMEM load takes several hundred cycles to come back, so the
        // row is read once
        uint32_t sv[4][32];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32b_x32(tmem_s + cc * 32, sv[cc]);
        tmem_ld_wait();
        const bool need_mask = (k0 + 128 > p.Tk) || (p.causal && (k0 + 127 > q0 + off)) ||
                               (p.window > 0 && (k0 < q0 + 127 + off - p.window + 1));
        const int clo = row_lo - k0, chi = row_hi - k0;  // column c is visible iff clo <= c <= chi
        if (need_mask) {
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (cc * 32 + c < clo || cc * 32 + c > chi) sv[cc][c] = 0xff800000u;  // -inf
        }
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            m0 = fmaxf(m0, __uint_as_float(sv[cc][c]));
            m1 = fmaxf(m1, __uint_as_float(sv[cc][c + 1]));
            m2 = fmaxf(m2, __uint_as_float(sv[cc][c + 2]));
            m3 = fmaxf(m3, __uint_as_float(sv[cc][c + 3]));
          }
        const float m_new = fmaxf(m_ref, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * sc);
        // rescale only when the maximum has moved far: a warp-uniform decision, every lane uses its own factor
        const bool grow = m_new - kRescaleStep > m_ref;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? ex2f(m_ref - m_new) : 1.0f;  // m_ref == -inf -> 0
          if (grow) {
            l_run *= alpha;
            m_ref = m_new;
          }
          if (j > jbx) {  // the output tile holds the sums of the earlier key tiles
            ok = __all_sync(0xffffffffu, mbar_wait_bounded(&o_done[x], (cnt - 1) & 1, abort_flag));
            if (!ok) {
              if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
              break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (int cc = 0; cc < HD / 32; ++cc) {
              uint32_t ov[32];
              tmem_ld_32x32b_x32(tmem_o + cc * 32, ov);
              tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * alpha);
              tmem_st_32x32b_x32(tmem_o + cc * 32, ov);
            }
            tmem_st_wait();
          }
        }
        const float m_use = (m_ref == -INFINITY) ? 0.0f : m_ref;
        float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = ex2f(fmaf(__uint_as_float(sv[cc][8 * g + i]), sc, -m_use));  // -inf -> 0
            r0 += e[0] + e[4];
            r1 += e[1] + e[5];
            r2 += e[2] + e[6];
            r3 += e[3] + e[7];
            pk[4 * g + 0] = pack_bf16x2(e[0], e[1]);
            pk[4 * g + 1] = pack_bf16x2(e[2], e[3]);
            pk[4 * g + 2] = pack_bf16x2(e[4], e[5]);
            pk[4 * g + 3] = pack_bf16x2(e[6], e[7]);
          }
          tmem_st_32x32b_x16(tmem_s + cc * 16, pk);  // two probabilities per column
        }
        l_run += (r0 + r1) + (r2 + r3);
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[x]);
      }
      if (!ok) break;
      // ---- the last P V has retired: normalise (and merge) the output rows
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(&o_done[x], (cnt - 1) & 1, abort_flag));
      if (!ok) {
        if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      float o_acc[HD];
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t ov[32];
        tmem_ld_32x32b_x32(tmem_o + cc * 32, ov);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) o_acc[cc * 32 + c] = __uint_as_float(ov[c]);
      }
      tc_fence_before_sync();
      if (q < p.Tq) {
        const int64_t li = (static_cast<int64_t>(w.b) * p.H + w.h) * p.Tq + q;
        float m_fin = m_ref;
        if (p.merge_o != nullptr) {
          // merge with the result of earlier key/value chunks: softmax over the union of the key sets
          float* mo = p.merge_o + ((static_cast<int64_t>(w.b) * p.Tq + q) * p.H + w.h) * HD;
          const float lse_new = l_run > 0.0f ? (m_ref / kLog2e + logf(l_run)) : -INFINITY;
          const float lse_old = p.merge_lse[li];
          const float mm = fmaxf(lse_new, lse_old);
          const float w_new = (lse_new == -INFINITY) ? 0.0f : __expf(lse_new - mm);
          const float w_old = (lse_old == -INFINITY) ? 0.0f : __expf(lse_old - mm);
          const float den = w_new + w_old;
          const float c_new = den > 0.0f ? w_new / den / (l_run > 0.0f ? l_run : 1.0f) : 0.0f;
          const float c_old = den > 0.0f ? w_old / den : 0.0f;
#pragma unroll
          for (int g = 0; g < HD / 4; ++g) {
            float4 prev = reinterpret_cast<const float4*>(mo)[g];
            prev.x = prev.x * c_old + o_acc[4 * g + 0] * c_new;
            prev.y = prev.y * c_old + o_acc[4 * g + 1] * c_new;
            prev.z = prev.z * c_old + o_acc[4 * g + 2] * c_new;
            prev.w = prev.w * c_old + o_acc[4 * g + 3] * c_new;
            reinterpret_cast<float4*>(mo)[g] = prev;
            o_acc[4 * g + 0] = prev.x;
            o_acc[4 * g + 1] = prev.y;
            o_acc[4 * g + 2] = prev.z;
            o_acc[4 * g + 3] = prev.w;
          }
          l_run = den > 0.0f ? 1.0f : 0.0f;  // o_acc now holds the normalised merged output
          m_fin = (den > 0.0f ? mm + logf(den) : -INFINITY) * kLog2e;
        }
        const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(w.b) * p.o_batch +
                              static_cast<int64_t>(q) * p.o_row + static_cast<int64_t>(w.h) * p.o_head;
#pragma unroll
        for (int g = 0; g < HD / 8; ++g) {
          uint4 wv;
          wv.x = pack_bf16x2(o_acc[8 * g + 0] * inv, o_acc[8 * g + 1] * inv);
          wv.y = pack_bf16x2(o_acc[8 * g + 2] * inv, o_acc[8 * g + 3] * inv);
          wv.z = pack_bf16x2(o_acc[8 * g + 4] * inv, o_acc[8 * g + 5] * inv);
          wv.w = pack_bf16x2(o_acc[8 * g + 6] * inv, o_acc[8 * g + 7] * inv);
          reinterpret_cast<uint4*>(orow)[g] = wv;
        }
        const float lse = l_run > 0.0f ? (m_fin / kLog2e + logf(l_run)) : -INFINITY;
        if (p.lse) p.lse[li] = lse;
        if (p.merge_lse) p.merge_lse[li] = lse;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 9) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================================================================================
// backward, part 1: dK / dV.  One CTA per (kv block of 128, kv head, batch); loops over the q heads
// of the group and over q chunks of 64 rows.  TMEM: S^T [128 kv][64 q], dP^T [128][64], dV [128][HD],
// dK [128][HD].  Thread r owns kv row r.
// ================================================================================================
template <int HD>
struct DkvCfg {
  static constexpr int kKVBytes = 128 * HD * 2;   // K and V tiles (resident)
  static constexpr int kQBytes = 64 * HD * 2;     // Q / dO chunk
  static constexpr int kPBytes = 128 * 64 * 2;    // P^T and dS^T
  static constexpr int kSmem = 2 * kKVBytes + 4 * kQBytes + 2 * kPBytes + 2 * 2 * 64 * 4 + 128;
  static constexpr int kTmemCols = (HD == 64) ? 256 : 512;  // 64 + 64 + 2*HD
};

template <int HD, bool EXT>  // EXT: soft-capping / ALiBi / dropout row math (a build of its own)
__global__ void __launch_bounds__(kThreads, (HD == 64 ? 2 : 1))
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                     const AttnDev p) {
  pdl_launch_dependents();
  using C = DkvCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base; uniform early exit
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadArgument);
    return;
  }
  uint8_t* sK = smem;
  uint8_t* sV = sK + C::kKVBytes;
  uint8_t* sQ = sV + C::kKVBytes;        // 2 stages
  uint8_t* sDO = sQ + 2 * C::kQBytes;    // 2 stages
  uint8_t* sPT = sDO + 2 * C::kQBytes;   // [128 kv][64 q] bf16
  uint8_t* sDST = sPT + C::kPBytes;      // [128 kv][64 q] bf16
  float* sLse = reinterpret_cast<float*>(sDST + C::kPBytes);  // [2][64] (log2 domain)
  float* sDsum = sLse + 2 * 64;                               // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDsum + 2 * 64);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;    // [2]
  uint64_t* q_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;    // S^T and dP^T ready
  uint64_t* p_full = bars + 6;    // P^T and dS^T written
  uint64_t* acc_done = bars + 7;  // dV/dK MMAs of this chunk retired (P^T/dS^T reusable)
  uint64_t* stat_full = bars + 8;  // per-q statistics of the chunk staged in shared memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid in cost order: under a causal mask the early kv blocks are seen by the most queries, and
  // CTAs are handed out in block-index order, so the long ones start first
  const int per_blk = p.Hkv * p.B;
  const int kb = blockIdx.x / per_blk, hk = (blockIdx.x % per_blk) % p.Hkv, b = (blockIdx.x % per_blk) / p.Hkv;
  const int k0 = kb * 128;
  const int group = p.H / p.Hkv;
  const int off = p.Tk - p.Tq;

  // q rows that can see this kv block: q >= k0 - off (causal), q <= k0 + 127 - off + window - 1 (window)
  int q_lo = 0, q_hi = p.Tq;
  if (p.causal) q_lo = max(0, k0 - off);
  if (p.window > 0) q_hi = min(p.Tq, k0 + 127 - off + p.window);
  const int cb = q_lo / 64;
  const int ce = q_hi > q_lo ? (q_hi + 63) / 64 : cb;
  const int nchunk = ce - cb;
  const int iters = nchunk * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);  // one arrival per math warp
    mbar_init(acc_done, 1);
    mbar_init(stat_full, 2);  // warps 0 and 1 stage the statistics
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_st = tmem_base;         // S^T   64 cols
  const uint32_t tmem_dpt = tmem_base + 64;   // dP^T  64 cols
  const uint32_t tmem_dv = tmem_base + 128;   // dV    HD cols
  const uint32_t tmem_dk = tmem_base + 128 + HD;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(kv_full, 2 * C::kKVBytes);
      load_tile<HD>(sK, &tm_k, kv_full, 128, k0, hk, b, p.hfirst);
      load_tile<HD>(sV, &tm_v, kv_full, 128, k0, hk, b, p.hfirst);
      for (int it = 0; it < iters; ++it) {
        const int s = it & 1;
        const int hq = hk * group + it / nchunk;
        const int c0 = (cb + it % nchunk) * 64;
        if (!mbar_wait_bounded(&q_empty[s], ((it >> 1) & 1) ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, kStatusTimeoutProducer);
          break;
        }
        mbar_arrive_expect_tx(&q_full[s], 2 * C::kQBytes);
        load_tile<HD>(sQ + s * C::kQBytes, &tm_q, &q_full[s], 64, c0, hq, b, p.hfirst);
        load_tile<HD>(sDO + s * C::kQBytes, &tm_do, &q_full[s], 64, c0, hq, b, p.hfirst);
      }
    }
  } else if (warp == 5) {
    // the whole warp walks the loop (descriptors stay in uniform registers); one elected lane issues
    {
      const bool leader = elect_one();
      const uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, false, false, 128, 64);   // K Q^T, V dO^T
      const uint32_t idesc_g = make_idesc(kFmtBF16, kFmtBF16, false, true, 128, HD);    // P^T dO, dS^T Q
      bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(kv_full, 0, abort_flag));
      if (!ok && leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
      const uint64_t dK = desc_kmajor(smem_u32(sK), 128, 0), dV = desc_kmajor(smem_u32(sV), 128, 0);
      const uint64_t dPT = desc_kmajor(smem_u32(sPT), 128, 0), dDST = desc_kmajor(smem_u32(sDST), 128, 0);
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it & 1;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&q_full[s], (it >> 1) & 1, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        const uint32_t aQ = smem_u32(sQ + s * C::kQBytes), aDO = smem_u32(sDO + s * C::kQBytes);
        const uint64_t dQk = desc_kmajor(aQ, 64, 0), dDOk = desc_kmajor(aDO, 64, 0);
        const uint64_t dQm = desc_mnmajor(aQ, 64, 0), dDOm = desc_mnmajor(aDO, 64, 0);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            umma_f16_ss(tmem_st, dK + kstep_kmajor(128, ks), dQk + kstep_kmajor(64, ks), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            umma_f16_ss(tmem_dpt, dV + kstep_kmajor(128, ks), dDOk + kstep_kmajor(64, ks), idesc_s, ks > 0 ? 1u : 0u);
          umma_commit(s_full);
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(p_full, it & 1, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        // dV += P^T dO ; dK += dS^T Q   (reduction over the 64 q rows of the chunk: 4 k-steps)
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_dv, dPT + kstep_kmajor(128, ks), dDOm + kstep_mnmajor(ks), idesc_g,
                        (it > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_dk, dDST + kstep_kmajor(128, ks), dQm + kstep_mnmajor(ks), idesc_g,
                        (it > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&q_empty[s]);
          umma_commit(acc_done);
        }
        __syncwarp();
      }
    }
  } else {
    const int r = warp * 32 + lane;  // kv row inside the block == TMEM lane
    const int k = k0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sc = p.scale * kLog2e;
    // queries that may attend to key k:  k - off <= q (causal),  q <= k - off + window - 1 (window)
    int q_row_lo = p.causal ? k - off : 0;
    int q_row_hi = p.Tq - 1;
    if (p.window > 0) q_row_hi = min(q_row_hi, k - off + p.window - 1);
    if (k >= p.Tk) q_row_lo = 0x3fffffff;  // key out of range: nothing valid
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const int hq = hk * group + it / nchunk;
      const int c0 = (cb + it % nchunk) * 64;
      // stage the per-q statistics of this chunk (double-buffered by iteration parity)
      float* lse_s = sLse + (it & 1) * 64;
      float* ds_s = sDsum + (it & 1) * 64;
      if (r < 64) {
        const int q = c0 + r;
        const int64_t idx = (static_cast<int64_t>(b) * p.H + hq) * p.Tq + q;
        float l = q < p.Tq ? p.lse[idx] : INFINITY;
        if (l == -INFINITY) l = INFINITY;  // row that saw no key: probabilities are zero
        lse_s[r] = l * kLog2e;
        ds_s[r] = q < p.Tq ? p.dsum[idx] : 0.0f;
        __syncwarp();
        if (lane == 0) mbar_arrive(stat_full);
      }
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(stat_full, it & 1, abort_flag));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_bounded(s_full, it & 1, abort_flag));
      if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_done, (it - 1) & 1, abort_flag));
      if (!ok) {
        if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const bool need_mask = (k0 + 128 > p.Tk) || (c0 + 64 > p.Tq) || (p.causal && (k0 + 127 > c0 + off)) ||
                             (p.window > 0 && (k0 < c0 + 63 + off - p.window + 1));
      constexpr bool ext_on = EXT;
      const ScoreExt ext = EXT ? make_ext(p, hq, b) : ScoreExt{};
      auto body = [&](auto mask_tag, auto ext_tag) {
        constexpr bool kMask = decltype(mask_tag)::value;
        constexpr bool kExt = decltype(ext_tag)::value;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32b_x32(tmem_st + lane_addr + cc * 32, sv);
          tmem_ld_32x32b_x32(tmem_dpt + lane_addr + cc * 32, dv);
          tmem_ld_wait();
          const int clo = q_row_lo - c0 - cc * 32, chi = q_row_hi - c0 - cc * 32;  // valid iff clo <= c <= chi
          float pr[32], dsv[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int qi = cc * 32 + c;
            float sraw = __uint_as_float(sv[c]), dfac = 1.0f;
            if (kExt) sraw = score_ext(ext, sraw, k - (c0 + qi + off), dfac);
            float e = ex2f(fmaf(sraw, sc, -lse_s[qi]));
            if (kMask && (c < clo || c > chi)) e = 0.0f;
            float dp = __uint_as_float(dv[c]), keep = 1.0f;
            if (kExt && ext.drop_p > 0.0f) {
              keep = drop_scale_qk(ext, c0 + qi, k);
              dp *= keep;
            }
            pr[c] = e * keep;  // what met V in the forward pass
            dsv[c] = e * (dp - ds_s[qi]) * p.scale;
            if (kExt) dsv[c] *= dfac;
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w, z;
            w.x = pack_bf16x2(pr[8 * g + 0], pr[8 * g + 1]);
            w.y = pack_bf16x2(pr[8 * g + 2], pr[8 * g + 3]);
            w.z = pack_bf16x2(pr[8 * g + 4], pr[8 * g + 5]);
            w.w = pack_bf16x2(pr[8 * g + 6], pr[8 * g + 7]);
            z.x = pack_bf16x2(dsv[8 * g + 0], dsv[8 * g + 1]);
            z.y = pack_bf16x2(dsv[8 * g + 2], dsv[8 * g + 3]);
            z.z = pack_bf16x2(dsv[8 * g + 4], dsv[8 * g + 5]);
            z.w = pack_bf16x2(dsv[8 * g + 6], dsv[8 * g + 7]);
            const uint32_t o = sw128_off(r, cc * 4 + g);
            *reinterpret_cast<uint4*>(sPT + o) = w;
            *reinterpret_cast<uint4*>(sDST + o) = z;
          }
        }
      };
      if (ext_on) {
        if (need_mask) body(std::true_type{}, std::true_type{});
        else body(std::false_type{}, std::true_type{});
      } else {
        if (need_mask) body(std::true_type{}, std::false_type{});
        else body(std::false_type{}, std::false_type{});
      }
      fence_proxy_async_smem();  // this thread's tile writes -> visible to the tensor core's reads
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // drain: wait for the last accumulation, then write dK / dV rows
    if (ok && iters > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_done, (iters - 1) & 1, abort_flag));
      if (!ok && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
    }
    if (ok) {  // warp-uniform: the TMEM loads below are warp-collective, only the stores are per row
      tc_fence_after_sync();
      const bool row_ok = k < p.Tk;
      __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(b) * p.o_batch +
                          static_cast<int64_t>(k) * p.o_row + static_cast<int64_t>(hk) * p.o_head;
      __nv_bfloat16* dvp = reinterpret_cast<__nv_bfloat16*>(p.out2) + static_cast<int64_t>(b) * p.o2_batch +
                           static_cast<int64_t>(k) * p.o2_row + static_cast<int64_t>(hk) * p.o2_head;
#pragma unroll 1
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t a[32], c[32];
        if (iters > 0) {
          tmem_ld_32x32b_x32(tmem_dk + lane_addr + cc * 32, a);
          tmem_ld_32x32b_x32(tmem_dv + lane_addr + cc * 32, c);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = c[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w, z;
          w.x = pack_bf16x2(__uint_as_float(a[8 * g + 0]), __uint_as_float(a[8 * g + 1]));
          w.y = pack_bf16x2(__uint_as_float(a[8 * g + 2]), __uint_as_float(a[8 * g + 3]));
          w.z = pack_bf16x2(__uint_as_float(a[8 * g + 4]), __uint_as_float(a[8 * g + 5]));
          w.w = pack_bf16x2(__uint_as_float(a[8 * g + 6]), __uint_as_float(a[8 * g + 7]));
          z.x = pack_bf16x2(__uint_as_float(c[8 * g + 0]), __uint_as_float(c[8 * g + 1]));
          z.y = pack_bf16x2(__uint_as_float(c[8 * g + 2]), __uint_as_float(c[8 * g + 3]));
          z.z = pack_bf16x2(__uint_as_float(c[8 * g + 4]), __uint_as_float(c[8 * g + 5]));
          z.w = pack_bf16x2(__uint_as_float(c[8 * g + 6]), __uint_as_float(c[8 * g + 7]));
          if (row_ok) {
            reinterpret_cast<uint4*>(dk + cc * 32)[g] = w;
            reinterpret_cast<uint4*>(dvp + cc * 32)[g] = z;
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ================================================================================================
// backward, part 2: dQ.  One CTA per (q block of 128, head, batch); loops over kv chunks of 64.
// TMEM: S [128 q][64 kv], dP [128][64], dQ [128][HD].  Thread r owns q row r.
// ================================================================================================
template <int HD>
struct DqCfg {
  static constexpr int kQBytes = 128 * HD * 2;   // Q and dO tiles (resident)
  static constexpr int kKVBytes = 64 * HD * 2;   // K / V chunk
  static constexpr int kPBytes = 128 * 64 * 2;   // dS
#ifndef NX_DQ_STAGES
#define NX_DQ_STAGES 2
#endif
  static constexpr int kStages = (HD == 64) ? NX_DQ_STAGES : 2;  // K / V chunk stages (a third one measured no faster)
  static constexpr int kSmem = 2 * kQBytes + 2 * kStages * kKVBytes + kPBytes + 256;
  static constexpr int kTmemCols = 256;  // 64 + 64 + HD
};

template <int HD, bool EXT>  // EXT: soft-capping / ALiBi / dropout row math (a build of its own)
__global__ void __launch_bounds__(kThreads, (HD == 64 ? 2 : 1))
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const AttnDev p) {
  using C = DqCfg<HD>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // the swizzled tiles need a 1 KiB aligned base; uniform early exit
    if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadArgument);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + C::kQBytes;
  constexpr int NS = C::kStages;
  uint8_t* sK = sDO + C::kQBytes;        // NS stages
  uint8_t* sV = sK + NS * C::kKVBytes;   // NS stages
  uint8_t* sDS = sV + NS * C::kKVBytes;  // [128 q][64 kv] bf16
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDS + C::kPBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;        // [NS]
  uint64_t* kv_empty = kv_full + NS;   // [NS]
  uint64_t* s_full = kv_empty + NS;
  uint64_t* p_full = s_full + 1;
  uint64_t* acc_done = p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid in cost order (late q blocks see the most keys under a causal mask)
  const int per_blk = p.H * p.B;
  const int qb = p.nqb - 1 - blockIdx.x / per_blk;
  const int h = (blockIdx.x % per_blk) % p.H, b = (blockIdx.x % per_blk) / p.H;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * 128;

  int kv_lo, kv_hi;
  kv_range(p, q0, min(128, p.Tq - q0), kv_lo, kv_hi);
  const int jb = kv_lo / 64;
  const int je = kv_hi > kv_lo ? (kv_hi + 63) / 64 : jb;
  const int iters = je - jb;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NS; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);  // one arrival per math warp
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_dp = tmem_base + 64;
  const uint32_t tmem_dq = tmem_base + 128;

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, 2 * C::kQBytes);
      load_tile<HD>(sQ, &tm_q, q_full, 128, q0, h, b, p.hfirst);
      load_tile<HD>(sDO, &tm_do, q_full, 128, q0, h, b, p.hfirst);
      for (int it = 0; it < iters; ++it) {
        const int s = it % NS;
        if (!mbar_wait_bounded(&kv_empty[s], ((it / NS) & 1) ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, kStatusTimeoutProducer);
          break;
        }
        mbar_arrive_expect_tx(&kv_full[s], 2 * C::kKVBytes);
        load_tile<HD>(sK + s * C::kKVBytes, &tm_k, &kv_full[s], 64, (jb + it) * 64, hk, b, p.hfirst);
        load_tile<HD>(sV + s * C::kKVBytes, &tm_v, &kv_full[s], 64, (jb + it) * 64, hk, b, p.hfirst);
      }
    }
  } else if (warp == 5) {
    // the whole warp walks the loop (descriptors stay in uniform registers); one elected lane issues
    {
      const bool leader = elect_one();
      const uint32_t idesc_s = make_idesc(kFmtBF16, kFmtBF16, false, false, 128, 64);  // Q K^T, dO V^T
      const uint32_t idesc_g = make_idesc(kFmtBF16, kFmtBF16, false, true, 128, HD);   // dS K
      bool ok = __all_sync(0xffffffffu, mbar_wait_bounded(q_full, 0, abort_flag));
      if (!ok && leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
      const uint64_t dQ = desc_kmajor(smem_u32(sQ), 128, 0), dDO = desc_kmajor(smem_u32(sDO), 128, 0);
      const uint64_t dDS = desc_kmajor(smem_u32(sDS), 128, 0);
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % NS;
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&kv_full[s], (it / NS) & 1, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        const uint32_t aK = smem_u32(sK + s * C::kKVBytes), aV = smem_u32(sV + s * C::kKVBytes);
        const uint64_t dKk = desc_kmajor(aK, 64, 0), dVk = desc_kmajor(aV, 64, 0), dKm = desc_mnmajor(aK, 64, 0);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            umma_f16_ss(tmem_s, dQ + kstep_kmajor(128, ks), dKk + kstep_kmajor(64, ks), idesc_s, ks > 0 ? 1u : 0u);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks)
            umma_f16_ss(tmem_dp, dDO + kstep_kmajor(128, ks), dVk + kstep_kmajor(64, ks), idesc_s, ks > 0 ? 1u : 0u);
          umma_commit(s_full);
        }
        __syncwarp();
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(p_full, it & 1, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem_dq, dDS + kstep_kmajor(128, ks), dKm + kstep_mnmajor(ks), idesc_g,
                        (it > 0 || ks > 0) ? 1u : 0u);
          umma_commit(&kv_empty[s]);
          umma_commit(acc_done);
        }
        __syncwarp();
      }
    }
  } else {
    const int r = warp * 32 + lane;
    const int q = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const float sc = p.scale * kLog2e;
    const int off = p.Tk - p.Tq;
    const int64_t sidx = (static_cast<int64_t>(b) * p.H + h) * p.Tq + q;
    float lse_n = q < p.Tq ? p.lse[sidx] : INFINITY;
    if (lse_n == -INFINITY) lse_n = INFINITY;  // row that saw no key: probabilities are zero
    const float lse2 = lse_n * kLog2e;
    // dsum = rowsum(dO * O) of this thread's row, straight from global memory (the loads overlap the first tiles'
    // TMA traffic); published for the dK/dV kernel
    float dsum = 0.0f;
    if (q < p.Tq) {
      const uint4* orow = reinterpret_cast<const uint4*>(p.o_in + static_cast<int64_t>(b) * p.oi_batch +
                                                         static_cast<int64_t>(q) * p.oi_row + static_cast<int64_t>(h) * p.oi_head);
      const uint4* grow = reinterpret_cast<const uint4*>(p.do_in + static_cast<int64_t>(b) * p.di_batch +
                                                         static_cast<int64_t>(q) * p.di_row + static_cast<int64_t>(h) * p.di_head);
      float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        const uint4 ov = orow[i], gv = grow[i];
        const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float x0, x1, y0, y1;
          unpack_bf16x2(ow[j], x0, x1);
          unpack_bf16x2(gw[j], y0, y1);
          a0 = fmaf(x0, y0, a0);
          a1 = fmaf(x1, y1, a1);
        }
      }
      dsum = a0 + a1;
      p.dsum_out[sidx] = dsum;
    }
    int row_lo, row_hi;
    row_limits(p, q, row_lo, row_hi);
    if (q >= p.Tq) row_lo = 0x3fffffff;
    constexpr bool ext_on = EXT;
    const ScoreExt ext = EXT ? make_ext(p, h, b) : ScoreExt{};
    bool ok = true;
    for (int it = 0; it < iters; ++it) {
      const int k0 = (jb + it) * 64;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(s_full, it & 1, abort_flag));
      if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_done, (it - 1) & 1, abort_flag));
      if (!ok) {
        if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const bool need_mask = (k0 + 64 > p.Tk) || (q0 + 128 > p.Tq) || (p.causal && (k0 + 63 > q0 + off)) ||
                             (p.window > 0 && (k0 < q0 + 127 + off - p.window + 1));
      auto body = [&](auto mask_tag, auto ext_tag) {
        constexpr bool kMask = decltype(mask_tag)::value;
        constexpr bool kExt = decltype(ext_tag)::value;
#pragma unroll 1
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t sv[32], dv[32];
          tmem_ld_32x32b_x32(tmem_s + lane_addr + cc * 32, sv);
          tmem_ld_32x32b_x32(tmem_dp + lane_addr + cc * 32, dv);
          tmem_ld_wait();
          const int clo = row_lo - k0 - cc * 32, chi = row_hi - k0 - cc * 32;
          float dsv[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            float sraw = __uint_as_float(sv[c]), dfac = 1.0f;
            if (kExt) sraw = score_ext(ext, sraw, k0 + cc * 32 + c - (q + off), dfac);
            float e = ex2f(fmaf(sraw, sc, -lse2));
            if (kMask && (c < clo || c > chi)) e = 0.0f;
            float dp = __uint_as_float(dv[c]);
            if (kExt && ext.drop_p > 0.0f) dp *= drop_scale_qk(ext, q, k0 + cc * 32 + c);
            dsv[c] = e * (dp - dsum) * p.scale;
            if (kExt) dsv[c] *= dfac;
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 z;
            z.x = pack_bf16x2(dsv[8 * g + 0], dsv[8 * g + 1]);
            z.y = pack_bf16x2(dsv[8 * g + 2], dsv[8 * g + 3]);
            z.z = pack_bf16x2(dsv[8 * g + 4], dsv[8 * g + 5]);
            z.w = pack_bf16x2(dsv[8 * g + 6], dsv[8 * g + 7]);
            *reinterpret_cast<uint4*>(sDS + sw128_off(r, cc * 4 + g)) = z;
          }
        }
      };
      if (ext_on) {
        if (need_mask) body(std::true_type{}, std::true_type{});
        else body(std::false_type{}, std::true_type{});
      } else {
        if (need_mask) body(std::true_type{}, std::false_type{});
        else body(std::false_type{}, std::false_type{});
      }
      fence_proxy_async_smem();  // this thread's tile writes -> visible to the tensor core's reads
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && iters > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_done, (iters - 1) & 1, abort_flag));
      if (!ok && lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
    }
    if (ok) {  // warp-uniform: the TMEM loads below are warp-collective, only the stores are per row
      tc_fence_after_sync();
      const bool row_ok = q < p.Tq;
      __nv_bfloat16* dq = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(b) * p.o_batch +
                          static_cast<int64_t>(q) * p.o_row + static_cast<int64_t>(h) * p.o_head;
#pragma unroll 1
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t a[32];
        if (iters > 0) {
          tmem_ld_32x32b_x32(tmem_dq + lane_addr + cc * 32, a);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = 0u;
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(a[8 * g + 0]), __uint_as_float(a[8 * g + 1]));
          w.y = pack_bf16x2(__uint_as_float(a[8 * g + 2]), __uint_as_float(a[8 * g + 3]));
          w.z = pack_bf16x2(__uint_as_float(a[8 * g + 4]), __uint_as_float(a[8 * g + 5]));
          w.w = pack_bf16x2(__uint_as_float(a[8 * g + 6]), __uint_as_float(a[8 * g + 7]));
          if (row_ok) reinterpret_cast<uint4*>(dq + cc * 32)[g] = w;
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
int check_view(const NxAttnView& v) {
  if (v.ptr == nullptr) return -1;
  if (reinterpret_cast<uintptr_t>(v.ptr) & 15) return -1;
  if ((v.row_stride & 7) || (v.head_stride & 7) || (v.batch_stride & 7)) return -1;
  return 0;
}

bool head_first(const NxAttnView& v) { return v.head_stride <= v.row_stride; }

int make_map(CUtensorMap* m, const NxAttnView& v, int T, int H, int B, int HD, int box_rows) {
  if (head_first(v))
    return nx::make_tensor_map_4d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v.ptr, HD, H, T, B, v.head_stride,
                                  v.row_stride, v.batch_stride, 64, 1, box_rows);
  return nx::make_tensor_map_4d(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v.ptr, HD, T, H, B, v.row_stride,
                                v.head_stride, v.batch_stride, 64, box_rows, 1);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess ? 0 : -2;
}

AttnDev base_params(const NxAttnArgs* a) {
  AttnDev p{};
  p.lse = a->lse;
  p.merge_o = a->merge_o;
  p.merge_lse = a->merge_lse;
  p.dsum = a->dsum;
  p.status = a->status;
  p.B = a->batch;
  p.H = a->heads;
  p.Hkv = a->kv_heads;
  p.Tq = a->tq;
  p.Tk = a->tk;
  p.causal = a->causal;
  p.window = a->window;
  p.scale = a->scale;
  p.softcap = a->softcap;
  p.alibi = a->alibi_slopes;
  p.dropout_p = a->dropout_p;
  p.drop_seed = a->dropout_seed;
  p.drop_offset = a->dropout_offset;
  p.hfirst = head_first(a->q) ? 1 : 0;
  return p;
}

int check_args(const NxAttnArgs* a) {
  if (a == nullptr || a->status == nullptr) return -1;
  if (a->head_dim != 64 && a->head_dim != 128) return -1;
  if (a->batch <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads) return -1;
  if (a->tq <= 0 || a->tk <= 0) return -1;
  if (!(a->dropout_p >= 0.0f && a->dropout_p < 1.0f) || a->softcap < 0.0f) return -1;
  // every TMA-read view must share one coordinate order
  const bool hf = head_first(a->q);
  if (head_first(a->k) != hf || head_first(a->v) != hf) return -1;
  if (a->d_o.ptr != nullptr && head_first(a->d_o) != hf) return -1;
  return 0;
}

}  // namespace

extern "C" int nx_attention_fwd(const NxAttnArgs* a, nx_stream_t stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (check_args(a) || check_view(a->q) || check_view(a->k) || check_view(a->v) || check_view(a->o)) return -1;
  const int HD = a->head_dim;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, a->q, a->tq, a->heads, a->batch, HD, 128))) return rc;
  if ((rc = make_map(&tk, a->k, a->tk, a->kv_heads, a->batch, HD, 128))) return rc;
  if ((rc = make_map(&tv, a->v, a->tk, a->kv_heads, a->batch, HD, 128))) return rc;
  AttnDev p = base_params(a);
  p.out = a->o.ptr;
  p.o_row = a->o.row_stride;
  p.o_head = a->o.head_stride;
  p.o_batch = a->o.batch_stride;
  p.nqb = (a->tq + 127) / 128;
  p.items = p.nqb * a->heads * a->batch;
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return -2;
  // one persistent CTA per slot: two per SM for head_dim 64 (registers / shared memory allow it), one otherwise
  const int grid = std::min(p.items, sms * (HD == 64 ? 2 : 1));
  const bool ext = p.softcap > 0.0f || p.alibi != nullptr || p.dropout_p > 0.0f;
  // The two-tile kernel serves the plain softmax (no soft-capping / ALiBi / dropout).  It is the default for
  // head_dim 128 (369 us against 499 us on 2 x 32 x 4096 x 128, causal); at head_dim 64 the two forms time alike
  // and the one-tile kernel below stays.  NEXUS_B200_ATTN_FWD=1 / =2 forces the one-tile / two-tile form.
  static const int fwd_mode = [] {
    const char* e = std::getenv("NEXUS_B200_ATTN_FWD");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (!ext && (fwd_mode == 2 || (fwd_mode == 0 && HD == 128))) {
    p.nqb = (a->tq + 255) / 256;
    p.items = p.nqb * a->heads * a->batch;
    const int grid2 = std::min(p.items, sms);
#define NX_FWD2(HD_)                                                                                \
  do {                                                                                              \
    static bool once = false;                                                                       \
    if (!once) {                                                                                    \
      if (set_smem(attn_fwd2_kernel<HD_>, Fwd2Cfg<HD_>::kSmem)) return -2;                          \
      once = true;                                                                                  \
    }                                                                                               \
    attn_fwd2_kernel<HD_><<<grid2, kFwd2Threads, Fwd2Cfg<HD_>::kSmem, st>>>(tq, tk, tv, p);         \
  } while (0)
    if (HD == 64) NX_FWD2(64);
    else NX_FWD2(128);
#undef NX_FWD2
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
#define NX_FWD(HD_, EXT_)                                                                           \
  do {                                                                                              \
    static bool once = false;                                                                       \
    if (!once) {                                                                                    \
      if (set_smem(attn_fwd_kernel<HD_, EXT_>, FwdCfg<HD_>::kSmem)) return -2;                      \
      once = true;                                                                                  \
    }                                                                                               \
    attn_fwd_kernel<HD_, EXT_><<<grid, kFwdThreads, FwdCfg<HD_>::kSmem, st>>>(tq, tk, tv, p);       \
  } while (0)
  if (HD == 64) {
    if (ext) NX_FWD(64, true);
    else NX_FWD(64, false);
  } else {
    if (ext) NX_FWD(128, true);
    else NX_FWD(128, false);
  }
#undef NX_FWD
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int nx_attention_bwd(const NxAttnArgs* a, nx_stream_t stream_) {
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  if (check_args(a) || check_view(a->q) || check_view(a->k) || check_view(a->v) || check_view(a->o) ||
      check_view(a->d_o) || check_view(a->dq) || check_view(a->dk) || check_view(a->dv))
    return -1;
  if (a->lse == nullptr || a->dsum == nullptr) return -1;
  const int HD = a->head_dim;
  const bool ext = a->softcap > 0.0f || a->alibi_slopes != nullptr || a->dropout_p > 0.0f;
  int rc;
#define NX_BWD(KERN_, CFG_, HD_, EXT_)                                                              \
  do {                                                                                              \
    static bool once = false;                                                                       \
    if (!once) {                                                                                    \
      if (set_smem(KERN_<HD_, EXT_>, CFG_<HD_>::kSmem)) return -2;                                  \
      once = true;                                                                                  \
    }                                                                                               \
    KERN_<HD_, EXT_><<<grid, kThreads, CFG_<HD_>::kSmem, st>>>(tq, tk, tv, tdo, p);                 \
  } while (0)
  // part 1: dQ (also forms dsum = rowsum(dO * O) and leaves it for part 2)
  {
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_map(&tq, a->q, a->tq, a->heads, a->batch, HD, 128))) return rc;
    if ((rc = make_map(&tdo, a->d_o, a->tq, a->heads, a->batch, HD, 128))) return rc;
    if ((rc = make_map(&tk, a->k, a->tk, a->kv_heads, a->batch, HD, 64))) return rc;
    if ((rc = make_map(&tv, a->v, a->tk, a->kv_heads, a->batch, HD, 64))) return rc;
    AttnDev p = base_params(a);
    p.out = a->dq.ptr;
    p.o_row = a->dq.row_stride;
    p.o_head = a->dq.head_stride;
    p.o_batch = a->dq.batch_stride;
    p.nqb = (a->tq + 127) / 128;
    p.o_in = static_cast<const __nv_bfloat16*>(a->o.ptr);
    p.oi_row = a->o.row_stride;
    p.oi_head = a->o.head_stride;
    p.oi_batch = a->o.batch_stride;
    p.do_in = static_cast<const __nv_bfloat16*>(a->d_o.ptr);
    p.di_row = a->d_o.row_stride;
    p.di_head = a->d_o.head_stride;
    p.di_batch = a->d_o.batch_stride;
    p.dsum_out = a->dsum;
    const unsigned grid = static_cast<unsigned>(p.nqb * a->heads * a->batch);
    if (HD == 64) {
      if (ext) NX_BWD(attn_bwd_dq_kernel, DqCfg, 64, true);
      else NX_BWD(attn_bwd_dq_kernel, DqCfg, 64, false);
    } else {
      if (ext) NX_BWD(attn_bwd_dq_kernel, DqCfg, 128, true);
      else NX_BWD(attn_bwd_dq_kernel, DqCfg, 128, false);
    }
  }
  // part 2: dK, dV (reads the dsum that part 1 wrote)
  {
    CUtensorMap tq, tk, tv, tdo;
    if ((rc = make_map(&tq, a->q, a->tq, a->heads, a->batch, HD, 64))) return rc;
    if ((rc = make_map(&tdo, a->d_o, a->tq, a->heads, a->batch, HD, 64))) return rc;
    if ((rc = make_map(&tk, a->k, a->tk, a->kv_heads, a->batch, HD, 128))) return rc;
    if ((rc = make_map(&tv, a->v, a->tk, a->kv_heads, a->batch, HD, 128))) return rc;
    AttnDev p = base_params(a);
    p.out = a->dk.ptr;
    p.o_row = a->dk.row_stride;
    p.o_head = a->dk.head_stride;
    p.o_batch = a->dk.batch_stride;
    p.out2 = a->dv.ptr;
    p.o2_row = a->dv.row_stride;
    p.o2_head = a->dv.head_stride;
    p.o2_batch = a->dv.batch_stride;
    const unsigned grid = static_cast<unsigned>(((a->tk + 127) / 128) * a->kv_heads * a->batch);
    if (HD == 64) {
      if (ext) NX_BWD(attn_bwd_dkdv_kernel, DkvCfg, 64, true);
      else NX_BWD(attn_bwd_dkdv_kernel, DkvCfg, 64, false);
    } else {
      if (ext) NX_BWD(attn_bwd_dkdv_kernel, DkvCfg, 128, true);
      else NX_BWD(attn_bwd_dkdv_kernel, DkvCfg, 128, false);
    }
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
#undef NX_BWD
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
