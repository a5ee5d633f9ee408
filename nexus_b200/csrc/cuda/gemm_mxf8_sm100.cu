// Block-scaled FP8 (MX) GEMM for sm_100a and the quantiser that feeds it.
//
// Operands are FP8 codes (E4M3 / E5M2) with one E8M0 scale (a power of two) per 32 elements along K.  The
// tensor core applies the scales itself: tcgen05.mma kind::mxf8f6f4.block_scale reads them from tensor memory,
// where tcgen05.cp puts them straight from the shared-memory stage that a bulk copy filled - the scale bytes are
// stored in global memory in the order the hardware wants (512-byte atoms of 128 rows x 4 blocks), so no thread
// ever touches them on the way.
//
//   warp 0      : producer - two tiled TMA loads (A, B: 128 rows x 128 bytes, 128-byte swizzle) and two 512-byte
//                 bulk copies (scale atoms) per k-block
//   warp 1      : TMEM owner and MMA issuer - per k-block two tcgen05.cp (scales -> TMEM) and four MMAs (K = 32
//                 each, scale-factor id = position of the 32-block inside the atom)
//   warps 2..5  : epilogue - tcgen05.ld, alpha / bias / activation, then BF16 / FP32 values or, for an 8-bit
//                 output, MX codes plus scale atoms of the result (each thread holds one 32-block of its row, which
//                 is exactly one block of the next GEMM's K dimension)
//
// Persistent CTAs (one per SM) walk 128 x 128 tiles; two accumulators in TMEM let the epilogue of a tile overlap
// the MMAs of the next.  Every wait is bounded and reports through the status word.
//
// Replaces the reference's emulated FP8 linear (src/cuda/kernels_fp8.cu, include/nexus/cuda/fp8.hpp: per-tensor
// scales, dequantise + BF16 GEMM) with per-block scales applied inside the MMA.
#include "common.cuh"
#include "nx_api_lowp.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

#include <algorithm>
#include <cstdlib>
#include <cuda_fp8.h>

namespace {
using namespace nx;

constexpr int kBM = 128, kBN = 128, kBK = 128;  // kBK: FP8 elements = bytes of one swizzle row
constexpr int kTileBytes = kBM * kBK;           // 16 KiB per operand tile
constexpr int kAtomBytes = 512;
constexpr int kStageBytes = 2 * kTileBytes + 2 * kAtomBytes;
constexpr int kStages = 6;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;  // 2 x 128 accumulator columns + 4 + 4 scale columns, rounded up to a power of two
constexpr int kSfaCol = 256, kSfbCol = 260;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;

__device__ __forceinline__ uint8_t enc8(float x, int fmt) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, fmt == NX_E4M3 ? __NV_E4M3 : __NV_E5M2));
}
__device__ __forceinline__ float dec8(uint8_t b, int fmt) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), fmt == NX_E4M3 ? __NV_E4M3 : __NV_E5M2);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// E8M0 byte of the smallest power of two s with amax / s <= fmax (127 for an all-zero block), kept inside [1, 253]
// so that both 2^(byte-127) and its reciprocal are normal floats.
__device__ __forceinline__ uint32_t mx_scale_byte(float amax, int fmt) {
  if (!(amax > 0.0f)) return 127u;
  const float v = amax * (fmt == NX_E4M3 ? (1.0f / 448.0f) : (1.0f / 57344.0f));
  const uint32_t bits = __float_as_uint(v);
  uint32_t e = (bits >> 23) & 0xFFu;
  if ((bits & 0x7FFFFFu) != 0u) e += 1u;
  return min(max(e, 1u), 253u);
}
__device__ __forceinline__ float mx_inv_scale(uint32_t byte) { return __uint_as_float((254u - byte) << 23); }
__device__ __forceinline__ float mx_scale(uint32_t byte) { return __uint_as_float(byte << 23); }

// byte offset of the scale of (row r, 32-block j) of a matrix with `kb128` column blocks of 128
__host__ __device__ __forceinline__ size_t mx_scale_offset(int r, int j, int kb128) {
  return (static_cast<size_t>(r >> 7) * kb128 + (j >> 2)) * kAtomBytes + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (j & 3);
}

// One thread per (row of the codes, 32-block).  The grid covers the padded scale domain (rows up to a multiple of 128,
// blocks up to a multiple of 4) so that every byte of every atom is written: padding gets the scale 1.
template <bool TRANSPOSE>
__global__ void mx_quantize_kernel(const void* __restrict__ src, int src_dtype, int64_t ld, int rows, int cols,
                                   uint8_t* __restrict__ codes, uint8_t* __restrict__ scales, int fmt) {
  // code matrix: R x Kc (blocks along Kc)
  const int R = TRANSPOSE ? cols : rows, Kc = TRANSPOSE ? rows : cols;
  const int kb128 = (Kc + 127) >> 7, nblk = kb128 * 4, rpad = (R + 127) & ~127;
  const int64_t total = static_cast<int64_t>(rpad) * nblk;
  NX_GRID_STRIDE(i, total) {
    // TRANSPOSE: consecutive threads take consecutive code rows (= source columns): coalesced source reads.
    const int r = TRANSPOSE ? static_cast<int>(i % rpad) : static_cast<int>(i / nblk);
    const int j = TRANSPOSE ? static_cast<int>(i / rpad) : static_cast<int>(i % nblk);
    uint8_t* sp = scales + mx_scale_offset(r, j, kb128);
    const int k0 = j * 32;
    if (r >= R || k0 >= Kc) {
      *sp = 127;
      continue;
    }
    float v[32];
    float am = 0.0f;
    bool loaded = false;
    if constexpr (!TRANSPOSE) {
      // a whole block of a BF16 row in four 16-byte loads
      if (src_dtype == NX_BF16 && k0 + 32 <= Kc && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const uint4* sp4 = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src) +
                                                          static_cast<int64_t>(r) * ld + k0);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 u = sp4[q];
          unpack_bf16x2(u.x, v[8 * q + 0], v[8 * q + 1]);
          unpack_bf16x2(u.y, v[8 * q + 2], v[8 * q + 3]);
          unpack_bf16x2(u.z, v[8 * q + 4], v[8 * q + 5]);
          unpack_bf16x2(u.w, v[8 * q + 6], v[8 * q + 7]);
        }
#pragma unroll
        for (int t = 0; t < 32; ++t) am = fmaxf(am, fabsf(v[t]));
        loaded = true;
      }
    }
    if (!loaded) {
#pragma unroll
      for (int t = 0; t < 32; ++t) {
        const int k = k0 + t;
        float x = 0.0f;
        if (k < Kc) x = TRANSPOSE ? load_as_float(src, src_dtype, static_cast<int64_t>(k) * ld + r)
                                  : load_as_float(src, src_dtype, static_cast<int64_t>(r) * ld + k);
        v[t] = x;
        am = fmaxf(am, fabsf(x));
      }
    }
    const uint32_t sb = mx_scale_byte(am, fmt);
    const float inv = mx_inv_scale(sb);
    *sp = static_cast<uint8_t>(sb);
    uint8_t* cp = codes + static_cast<int64_t>(r) * Kc + k0;
    if (k0 + 32 <= Kc && (Kc & 15) == 0) {
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        w[q] = enc8(v[4 * q] * inv, fmt) | (enc8(v[4 * q + 1] * inv, fmt) << 8) | (enc8(v[4 * q + 2] * inv, fmt) << 16) |
               (enc8(v[4 * q + 3] * inv, fmt) << 24);
      reinterpret_cast<uint4*>(cp)[0] = make_uint4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<uint4*>(cp)[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
      for (int t = 0; t < 32 && k0 + t < Kc; ++t) cp[t] = enc8(v[t] * inv, fmt);
    }
  }
}

__global__ void mx_dequantize_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, int fmt,
                                     int rows, int cols, void* __restrict__ dst, int dst_dtype) {
  const int kb128 = (cols + 127) >> 7;
  const int64_t total = static_cast<int64_t>(rows) * cols;
  NX_GRID_STRIDE(i, total) {
    const int r = static_cast<int>(i / cols), k = static_cast<int>(i % cols);
    const uint32_t sb = scales[mx_scale_offset(r, k >> 5, kb128)];
    store_from_float(dst, dst_dtype, i, dec8(codes[i], fmt) * mx_scale(sb));
  }
}

// ------------------------------------------------------------------------------------------------
// PTX used only by this kernel
// ------------------------------------------------------------------------------------------------
// Untiled bulk copy global -> shared (no multicast); both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Shared-memory descriptor of one scale atom: 32 rows of 16 bytes, no swizzle (8-row groups 128 bytes apart).
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128u >> 4) << 32;  // stride between 8-row groups
  d |= 1ull << 46;                              // descriptor version
  return d;
}
// 32 rows x 128 bits of shared memory -> 4 TMEM columns, repeated in all four lane quarters.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mxf8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of the block-scaled kinds: operand formats, K-major operands, E8M0 scales, M x N; the
// scale-factor ids (which byte of each 4-byte TMEM scale column this MMA uses) are or-ed in per instruction.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n) {
  return (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_with_sf_id(uint32_t idesc, uint32_t id) { return idesc | (id << 4) | (id << 29); }

struct MxParams {
  void* out;
  uint8_t* out_scales;
  const void* bias;
  unsigned int* amax_out;
  int* status;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int64_t ldo;
  int m, n, k;
  int out_dtype, bias_dtype, act;
  int tiles_m, tiles_n, kb_total, num_tiles;
  int out_fmt_kb128;  // column blocks of 128 of the result's scale atoms
  float alpha;
};

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == NX_ACT_GELU) return gelu_tanh_f(v);
  if (act == NX_ACT_RELU) return fmaxf(v, 0.0f);
  if (act == NX_ACT_SILU) return silu_f(v);
  return v;
}

// One 32-column chunk of one accumulator row: alpha, bias, activation, running |max|, then the store - values as
// BF16 / FP32, or, for an 8-bit output, the chunk as one block of the result's block-scaled form (its own power-of-two
// scale, 32 codes, and the scale byte at its place in the atom order).
__device__ __forceinline__ void mx_epilogue_chunk(const MxParams& p, const uint32_t (&raw)[32], int row, int col0, bool out8,
                                                  float& tmax) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]) * p.alpha;
  if (p.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.n) v[j] += load_as_float(p.bias, p.bias_dtype, col0 + j);
  }
  if (p.act != NX_ACT_NONE) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.act);
  }
  const bool row_ok = row < p.m;
  const int valid = min(32, p.n - col0);  // <= 0: the whole chunk is past N
  if (p.amax_out != nullptr && row_ok) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) tmax = fmaxf(tmax, fabsf(v[j]));
  }
  if (out8) {
    // one 32-block of the result's row: its own power-of-two scale, codes, and the scale byte in atom order
    if ((col0 >> 5) < p.out_fmt_kb128 * 4) {
      uint32_t sbyte = 127u;
      if (row_ok && valid > 0) {
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) am = fmaxf(am, fabsf(v[j]));
        sbyte = mx_scale_byte(am, p.out_dtype);
        const float inv = mx_inv_scale(sbyte);
        uint32_t w[8];
#pragma unroll
        for (int q = 0; q < 8; ++q)
          w[q] = enc8(v[4 * q] * inv, p.out_dtype) | (enc8(v[4 * q + 1] * inv, p.out_dtype) << 8) |
                 (enc8(v[4 * q + 2] * inv, p.out_dtype) << 16) | (enc8(v[4 * q + 3] * inv, p.out_dtype) << 24);
        uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0);
        op[0] = make_uint4(w[0], w[1], w[2], w[3]);
        op[1] = make_uint4(w[4], w[5], w[6], w[7]);
      }
      p.out_scales[mx_scale_offset(row, col0 >> 5, p.out_fmt_kb128)] = static_cast<uint8_t>(sbyte);
    }
  } else if (row_ok && valid > 0) {
    if (p.out_dtype == NX_F32) {
      float* op = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
      if (valid == 32 && (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          reinterpret_cast<float4*>(op)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      } else {
        for (int j = 0; j < valid; ++j) op[j] = v[j];
      }
    } else {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
      if (valid == 32 && (p.ldo & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          reinterpret_cast<uint4*>(op)[q] =
              make_uint4(pack_bf16x2(v[8 * q], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                         pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
      } else {
        for (int j = 0; j < valid; ++j) op[j] = __float2bfloat16_rn(v[j]);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mxf8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const MxParams p,
                 const uint32_t idesc) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                  // [kStages]
  uint64_t* empty_bar = bars + kStages;       // [kStages]
  uint64_t* tfull_bar = bars + 2 * kStages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // stage layout: A tile | B tile | A scale atom | B scale atom  (the tiles stay 1 KiB aligned: stage size is 33 KiB)
  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const int m0 = tm * kBM, n0 = tn * kBN;
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kTileBytes;
          uint8_t* ssa = sb + kTileBytes;
          uint8_t* ssb = ssa + kAtomBytes;
          mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_3d(sa, &tmap_a, &full_bar[stage], kb * kBK, m0, 0);
          tma_load_3d(sb, &tmap_b, &full_bar[stage], kb * kBK, n0, 0);
          bulk_load(ssa, p.sfa + (static_cast<size_t>(tm) * p.kb_total + kb) * kAtomBytes, kAtomBytes, &full_bar[stage]);
          bulk_load(ssb, p.sfb + (static_cast<size_t>(tn) * p.kb_total + kb) * kAtomBytes, kAtomBytes, &full_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kBN);
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutMma);
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint32_t sb = sa + kTileBytes;
          // scales of this k-block: shared memory -> TMEM; the tensor-core pipe runs them before the MMAs below
          tmem_cp_32x128b_warpx4(tmem_base + kSfaCol, make_sf_desc(sb + kTileBytes));
          tmem_cp_32x128b_warpx4(tmem_base + kSfbCol, make_sf_desc(sb + kTileBytes + kAtomBytes));
#pragma unroll
          for (int ks = 0; ks < kBK / 32; ++ks) {
            const uint64_t da = make_smem_desc_sw128(sa + ks * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + ks * 32, 16, 1024);
            umma_mxf8_ss(tmem_d, da, db, idesc_with_sf_id(idesc, ks), tmem_base + kSfaCol, tmem_base + kSfbCol,
                         (kb > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once the copies and MMAs above have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    float tmax = 0.0f;
    const bool out8 = p.out_dtype == NX_E4M3 || p.out_dtype == NX_E5M2;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const int row = tm * kBM + quarter * 32 + lane;
      const int n0 = tn * kBN;
      if (!mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag)) {
        atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * kBN);
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32b_x32(taddr + c * 32, raw);
        tmem_ld_wait();
        mx_epilogue_chunk(p, raw, row, n0 + c * 32, out8, tmax);
      }
      // this warp has read its part of the accumulator: hand it back to the MMA issuer
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (p.amax_out != nullptr) {
      tmax = warp_max(tmax);
      if (lane == 0 && tmax > 0.0f) atomicMax(p.amax_out, __float_as_uint(tmax));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}


// ------------------------------------------------------------------------------------------------
// CTA-pair variant: one 256 x 256 tile per cluster of two (tcgen05 cta_group::2).  Each CTA stages its own 128 rows
// of A, half (128 rows) of the B tile, the scale atom of its A rows and both scale atoms of the B tile, so a tile's
// operands cross L2 -> shared memory once per 256 x 256 outputs instead of once per 128 x 128.  The accumulator takes
// 256 of the 512 TMEM columns and the scales 12 more, so there is one accumulator: the epilogue (eight warps per CTA)
// drains it before the next tile's MMAs start, while the producer keeps filling stages.
// ------------------------------------------------------------------------------------------------
constexpr int kPairBN = 256;
constexpr int kPairStages = 6;
constexpr int kPairSfBytes = 3 * kAtomBytes;  // per stage: A atom, B atom (columns 0..127), B atom (columns 128..255)
constexpr int kPairThreads = 320;             // warp 0 producer, warp 1 MMA, warps 2..9 epilogue
constexpr int kPairSfaCol = 256, kPairSfbCol = 260;
constexpr int kPairSmemBytes = kPairStages * (2 * kTileBytes + kPairSfBytes) + 1024 + 256;

__device__ __forceinline__ void tmem_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_mxf8_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t"
      "}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kPairThreads, 1)
gemm_mxf8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                      const MxParams p, const uint32_t idesc) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_base = smem + kPairStages * 2 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sf_base + kPairStages * kPairSfBytes);
  uint64_t* full_bar = bars;                   // [stages]  used in the even CTA: bytes of both CTAs
  uint64_t* empty_bar = bars + kPairStages;    // [stages]  in both CTAs
  uint64_t* tfull_bar = bars + 2 * kPairStages;  // in both CTAs
  uint64_t* tempty_bar = tfull_bar + 1;          // used in the even CTA: 16 epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const int tile_first = static_cast<int>(blockIdx.x >> 1), tile_step = static_cast<int>(gridDim.x >> 1);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);
    *abort_flag = 0;
    fence_mbar_init();
  }
  cluster_sync_all();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kCtaStageBytes = 2 * kTileBytes + kPairSfBytes;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (one lane in each CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = tile_first; t < p.num_tiles && ok; t += tile_step) {
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const int m0 = tm * 256 + static_cast<int>(cta_rank) * kBM;
        const int n0 = tn * kPairBN;
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            break;
          }
          uint8_t* sa = smem + stage * 2 * kTileBytes;
          uint8_t* sb = sa + kTileBytes;
          uint8_t* ss = sf_base + stage * kPairSfBytes;
          if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * kCtaStageBytes);
          const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
          tma_load_3d_pair(sa, &tmap_a, bar, kb * kBK, m0, 0);
          tma_load_3d_pair(sb, &tmap_b, bar, kb * kBK, n0 + static_cast<int>(cta_rank) * 128, 0);
          // scale atoms as rows of 256 bytes: atom index * 2 is the row
          tma_load_3d_pair(ss, &tmap_sfa, bar, 0, 2 * ((2 * tm + static_cast<int>(cta_rank)) * p.kb_total + kb), 0);
          tma_load_3d_pair(ss + kAtomBytes, &tmap_sfb, bar, 0, 2 * ((2 * tn) * p.kb_total + kb), 0);
          tma_load_3d_pair(ss + 2 * kAtomBytes, &tmap_sfb, bar, 0, 2 * ((2 * tn + 1) * p.kb_total + kb), 0);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      // the even CTA's commits also arrive on this CTA's barriers: leave only after every filled stage was released
      for (int s = 0; s < kPairStages && ok; ++s) {
        ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag);
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = tile_first; t < p.num_tiles && ok; t += tile_step) {
        if (!mbar_wait_bounded(tempty_bar, acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        tc_fence_after_sync();
        for (int kb = 0; kb < p.kb_total; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutMma);
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * 2 * kTileBytes);
          const uint32_t sb = sa + kTileBytes;
          const uint32_t ss = smem_u32(sf_base + stage * kPairSfBytes);
          // each CTA's atoms (same shared-memory offsets) -> its own TMEM
          tmem_cp_32x128b_warpx4_pair(tmem_base + kPairSfaCol, make_sf_desc(ss));
          tmem_cp_32x128b_warpx4_pair(tmem_base + kPairSfbCol, make_sf_desc(ss + kAtomBytes));
          tmem_cp_32x128b_warpx4_pair(tmem_base + kPairSfbCol + 4, make_sf_desc(ss + 2 * kAtomBytes));
#pragma unroll
          for (int ks = 0; ks < kBK / 32; ++ks) {
            const uint64_t da = make_smem_desc_sw128(sa + ks * 32, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sb + ks * 32, 16, 1024);
            umma_mxf8_ss_pair(tmem_base, da, db, idesc_with_sf_id(idesc, ks), tmem_base + kPairSfaCol,
                              tmem_base + kPairSfbCol, (kb > 0 || ks > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(tfull_bar, 3);
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;  // columns [128 * half, 128 * half + 128) of the tile
    uint32_t acc_phase = 0;
    float tmax = 0.0f;
    const bool out8 = p.out_dtype == NX_E4M3 || p.out_dtype == NX_E5M2;
    for (int t = tile_first; t < p.num_tiles; t += tile_step) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const int row = tm * 256 + static_cast<int>(cta_rank) * kBM + quarter * 32 + lane;
      const int n0 = tn * kPairBN + half * 128;
      if (!mbar_wait_bounded(tfull_bar, acc_phase, abort_flag)) {
        atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(half * 128);
      // The warp's whole share of the accumulator (32 rows x 128 columns) moves to registers first, so that the
      // accumulator goes back to the MMA issuer after four TMEM loads; bias, activation, conversion and the global
      // stores then run under the next tile's MMAs.
      uint32_t raw[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(taddr + c * 32, raw[c]);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(tempty_bar), 0));
#pragma unroll
      for (int c = 0; c < 4; ++c) mx_epilogue_chunk(p, raw[c], row, n0 + c * 32, out8, tmax);
      acc_phase ^= 1u;
    }
    if (p.amax_out != nullptr) {
      tmax = warp_max(tmax);
      if (lane == 0 && tmax > 0.0f) atomicMax(p.amax_out, __float_as_uint(tmax));
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or leaves while the other may still use the pair
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

extern "C" size_t nx_mx_scale_bytes(int rows, int cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>((cols + 127) / 128) * kAtomBytes;
}

extern "C" int nx_mx_quantize(const void* src, int src_dtype, int64_t ld, int rows, int cols, void* codes, void* scales,
                              int fmt, int transpose, nx_stream_t stream_) {
  if (src == nullptr || codes == nullptr || scales == nullptr || rows <= 0 || cols <= 0) return -1;
  if (fmt != NX_E4M3 && fmt != NX_E5M2) return -1;
  if (src_dtype != NX_BF16 && src_dtype != NX_F32 && src_dtype != NX_F16) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int R = transpose ? cols : rows, Kc = transpose ? rows : cols;
  const int64_t total = static_cast<int64_t>((R + 127) & ~127) * (((Kc + 127) >> 7) * 4);
  const int threads = 128;
  const int blocks = blocks_for(total, threads, kNumSmsB200 * 32);
  if (transpose)
    mx_quantize_kernel<true><<<blocks, threads, 0, stream>>>(src, src_dtype, ld, rows, cols, static_cast<uint8_t*>(codes),
                                                             static_cast<uint8_t*>(scales), fmt);
  else
    mx_quantize_kernel<false><<<blocks, threads, 0, stream>>>(src, src_dtype, ld, rows, cols, static_cast<uint8_t*>(codes),
                                                              static_cast<uint8_t*>(scales), fmt);
  return launch_status();
}

extern "C" int nx_mx_dequantize(const void* codes, const void* scales, int fmt, int rows, int cols, void* dst,
                                int dst_dtype, nx_stream_t stream_) {
  if (codes == nullptr || scales == nullptr || dst == nullptr || rows <= 0 || cols <= 0) return -1;
  if (fmt != NX_E4M3 && fmt != NX_E5M2) return -1;
  const int64_t total = static_cast<int64_t>(rows) * cols;
  mx_dequantize_kernel<<<blocks_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(codes), static_cast<const uint8_t*>(scales), fmt, rows, cols, dst, dst_dtype);
  return launch_status();
}

namespace {
// -3: clusters of two cannot be placed on this device (the caller falls back to single-CTA tiles)
int launch_mx_pair(const NxMxGemmArgs* a, MxParams p, const CUtensorMap& ta, cudaStream_t stream) {
  static int max_clusters = 0;  // 0: not asked yet, < 0: unavailable
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(gemm_mxf8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) !=
        cudaSuccess)
      return -2;
    cfg.gridDim = dim3(2 * 74);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_mxf8_pair_kernel, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      max_clusters = -1;
    } else {
      max_clusters = n;
    }
  }
  if (max_clusters < 0) return -3;
  p.tiles_m = (a->m + 255) / 256;
  p.tiles_n = (a->n + kPairBN - 1) / kPairBN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  // B: 128 rows per CTA; the scale atoms seen as rows of 256 bytes (two rows per atom)
  CUtensorMap tb, tsa, tsb;
  int rc = nx::make_tensor_map_3d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->b, a->k, a->n, 1, a->ldb, 0, kBK, 128);
  if (rc != 0) return rc;
  const uint64_t kb128 = static_cast<uint64_t>(p.kb_total);
  rc = nx::make_tensor_map_3d(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->sfa, 256, 2 * ((a->m + 127) / 128) * kb128, 1, 256, 0,
                              256, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != 0) return rc;
  rc = nx::make_tensor_map_3d(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->sfb, 256, 2 * ((a->n + 127) / 128) * kb128, 1, 256, 0,
                              256, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != 0) return rc;
  int clusters = std::min(p.num_tiles, max_clusters);
  if (a->max_ctas > 1) clusters = std::min(clusters, a->max_ctas / 2);
  cfg.gridDim = dim3(2 * clusters);
  const uint32_t idesc = make_idesc_mx(a->a_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2,
                                       a->b_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2, 256, kPairBN);
  if (cudaLaunchKernelEx(&cfg, gemm_mxf8_pair_kernel, ta, tb, tsa, tsb, p, idesc) != cudaSuccess) {
    (void)cudaGetLastError();
    return -2;
  }
  return 0;
}
}  // namespace

extern "C" int nx_gemm_mxf8(const NxMxGemmArgs* a, nx_stream_t stream_) {
  if (a == nullptr || a->a == nullptr || a->b == nullptr || a->sfa == nullptr || a->sfb == nullptr || a->out == nullptr ||
      a->status == nullptr)
    return -1;
  if (a->m <= 0 || a->n <= 0 || a->k <= 0) return -1;
  const auto is8 = [](int d) { return d == NX_E4M3 || d == NX_E5M2; };
  if (!is8(a->a_dtype) || !is8(a->b_dtype)) return -1;
  // TMA: 16-byte aligned bases and pitches; the scale atoms are fetched with 16-byte bulk copies
  if ((a->lda & 15) != 0 || (a->ldb & 15) != 0 || (a->k & 15) != 0) return -1;
  if (((reinterpret_cast<uintptr_t>(a->a) | reinterpret_cast<uintptr_t>(a->b) | reinterpret_cast<uintptr_t>(a->sfa) |
        reinterpret_cast<uintptr_t>(a->sfb)) & 15) != 0)
    return -1;
  const bool out8 = is8(a->out_dtype);
  if (!out8 && a->out_dtype != NX_BF16 && a->out_dtype != NX_F32) return -1;
  if (out8 && (a->out_scales == nullptr || (a->n & 31) != 0 || (a->ldo & 15) != 0 ||
               (reinterpret_cast<uintptr_t>(a->out) & 15) != 0))
    return -1;
  if (a->act != NX_ACT_NONE && a->act != NX_ACT_GELU && a->act != NX_ACT_RELU && a->act != NX_ACT_SILU) return -1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);

  MxParams p{};
  p.out = a->out;
  p.out_scales = static_cast<uint8_t*>(a->out_scales);
  p.bias = a->bias;
  p.amax_out = reinterpret_cast<unsigned int*>(a->amax_out);
  p.status = a->status;
  p.sfa = static_cast<const uint8_t*>(a->sfa);
  p.sfb = static_cast<const uint8_t*>(a->sfb);
  p.ldo = a->ldo;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  p.out_dtype = a->out_dtype;
  p.bias_dtype = a->bias_dtype;
  p.act = a->act;
  p.tiles_m = (a->m + kBM - 1) / kBM;
  p.tiles_n = (a->n + kBN - 1) / kBN;
  p.kb_total = (a->k + kBK - 1) / kBK;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.out_fmt_kb128 = (a->n + 127) / 128;
  p.alpha = a->alpha;

  CUtensorMap ta, tb;
  int rc = nx::make_tensor_map_3d(&ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->a, a->k, a->m, 1, a->lda, 0, kBK, kBM);
  if (rc != 0) return rc;
  rc = nx::make_tensor_map_3d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->b, a->k, a->n, 1, a->ldb, 0, kBK, kBN);
  if (rc != 0) return rc;

  // CTA pairs (256 x 256 tiles) when the problem fills them; otherwise, or where clusters of two cannot be placed,
  // single-CTA 128 x 128 tiles
  static const bool single_only = std::getenv("NX_MX_SINGLE") != nullptr;  // measurement switch
  if (a->m >= 256 && a->n >= 256 && !single_only && (a->max_ctas <= 0 || a->max_ctas >= 2)) {
    const int rc_pair = launch_mx_pair(a, p, ta, stream);
    if (rc_pair != -3) return rc_pair;
  }

  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_mxf8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return -2;
  if (a->max_ctas > 0 && a->max_ctas < sms) sms = a->max_ctas;
  const int grid = p.num_tiles < sms ? p.num_tiles : sms;
  const uint32_t idesc = make_idesc_mx(a->a_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2,
                                       a->b_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2, kBM, kBN);
  gemm_mxf8_kernel<<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p, idesc);
  return launch_status();
}
