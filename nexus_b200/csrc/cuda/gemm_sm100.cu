// Persistent, warp-specialised BF16/FP16 GEMM for sm_100a.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor into 128B-swizzled shared-memory stages)
//   warp 1      : TMEM owner + UMMA issuer (tcgen05.mma, one elected lane; accumulators in TMEM)
//   warps 2..9  : epilogue (tcgen05.ld -> registers -> bias / GELU / dGELU / residual / accumulate -> global);
//                 two warps share each TMEM lane quarter and split the tile's columns
//
// One CTA per SM walks over (tile, k-slice) work units; two TMEM accumulator buffers let the
// epilogue of unit i overlap the main loop of unit i+1.  Operands may be K-major or MN-major, so
// forward (x W^T), dgrad (dy W) and wgrad (dy^T x) all run without a transpose pass.
//
// Replaces the reference's cuBLASLt layer and its epilogues Bias / BiasGelu(+aux) / DGelu /
// beta=1 accumulate (include/nexus/cuda/gemm.hpp:38-121, src/cuda/gemm_lt.cpp:260-360).
#include "nx_api_comm.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"
#include <algorithm>
#include <cstdlib>

namespace {

using namespace nx;

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kThreads = 320;  // warp 0: TMA, warp 1: MMA, warps 2..9: epilogue (two per TMEM lane quarter)
constexpr int kSmemBudget = 200 * 1024;

template <int BN>
struct Cfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kSmemBudget / kStageBytes;  // 4 for BN=256, 6 for BN=128
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kStoreBytes = 8 * 2 * 2048;  // per epilogue warp: [32 rows][32 bf16] for out and for aux_out
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct DevParams {
  void* out;
  const void* bias;
  const void* aux_in;
  void* aux_out;
  const void* residual;
  float* workspace;
  int* status;
  int64_t ldo, ld_aux, ld_res, stride_o;
  int m, n, k, batch;
  int out_dtype, bias_dtype, res_dtype, act, accumulate, split_k;
  int tiles_m, tiles_n, kb_total, kb_per_slice;
  int num_units;
  float alpha;
  // 8-bit float inputs: 128 elements per 128-byte swizzle row, kind::f8f6f4 MMA (K = 32 per instruction)
  int fp8, bk_elems;
  const float* scale_a;   // [m] per-row scale of A (may be null)
  const float* scale_b;   // [n] per-row scale of B (may be null)
  unsigned int* amax_out;  // max |out| as float bits (may be null)
  int tma_store;           // BF16 out (and aux_out) leave through shared memory and tiled TMA stores
};

struct Unit {
  int m0, n0, batch, slice, kb_begin, kb_end;
};

// Operands / output spread over the ranks of a group (peer-mapped memory).  Tiles never straddle a
// rank boundary (rows per rank are multiples of the tile height).
template <bool DIST>
struct DistParam {
  char unused;
};
template <>
struct alignas(64) DistParam<true> {
  CUtensorMap a[NX_MAX_PEERS];
  CUtensorMap b[NX_MAX_PEERS];
  float* out[NX_MAX_PEERS];
  int a_rows, b_rows, out_rows;  // rows per rank
  int a_sharded, b_sharded, out_scatter;
};

__device__ __forceinline__ Unit decode_unit(const DevParams& p, int u) {
  Unit w;
  int tm = u % p.tiles_m;
  u /= p.tiles_m;
  w.slice = u % p.split_k;
  u /= p.split_k;
  int tn = u % p.tiles_n;
  w.batch = u / p.tiles_n;
  w.m0 = tm * kBM;
  w.n0 = tn;  // multiplied by BN by the caller
  w.kb_begin = w.slice * p.kb_per_slice;
  w.kb_end = min(p.kb_total, w.kb_begin + p.kb_per_slice);
  return w;
}

template <typename T>
__device__ __forceinline__ void load_row32(const T* __restrict__ ptr, bool vec_ok, int valid, float (&v)[32]);

template <>
__device__ __forceinline__ void load_row32<__nv_bfloat16>(const __nv_bfloat16* __restrict__ ptr, bool vec_ok,
                                                          int valid, float (&v)[32]) {
  if (vec_ok) {
    const uint4* p4 = reinterpret_cast<const uint4*>(ptr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q = p4[i];
      unpack_bf16x2(q.x, v[8 * i + 0], v[8 * i + 1]);
      unpack_bf16x2(q.y, v[8 * i + 2], v[8 * i + 3]);
      unpack_bf16x2(q.z, v[8 * i + 4], v[8 * i + 5]);
      unpack_bf16x2(q.w, v[8 * i + 6], v[8 * i + 7]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? __bfloat162float(ptr[j]) : 0.0f;
  }
}
template <>
__device__ __forceinline__ void load_row32<float>(const float* __restrict__ ptr, bool vec_ok, int valid,
                                                  float (&v)[32]) {
  if (vec_ok) {
    const float4* p4 = reinterpret_cast<const float4*>(ptr);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float4 q = p4[i];
      v[4 * i + 0] = q.x;
      v[4 * i + 1] = q.y;
      v[4 * i + 2] = q.z;
      v[4 * i + 3] = q.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < valid) ? ptr[j] : 0.0f;
  }
}

__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16* ptr, bool vec_ok, int valid, const float (&v)[32]) {
  if (vec_ok) {
    uint4* p4 = reinterpret_cast<uint4*>(ptr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 q;
      q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
      q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
      q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
      q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      p4[i] = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) ptr[j] = __float2bfloat16_rn(v[j]);
  }
}
__device__ __forceinline__ void store_row32_f32(float* ptr, bool vec_ok, int valid, const float (&v)[32]) {
  if (vec_ok) {
    float4* p4 = reinterpret_cast<float4*>(ptr);
#pragma unroll
    for (int i = 0; i < 8; ++i) p4[i] = make_float4(v[4 * i + 0], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid) ptr[j] = v[j];
  }
}

// One row (32 BF16 = 64 bytes) of a [32 rows][32 cols] staging tile in the 64-byte swizzle of its tensor map:
// 16-byte chunk c of row r lives at chunk c ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage_row32_bf16(uint8_t* buf, int r, const float (&v)[32]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 q;
    q.x = pack_bf16x2(v[8 * i + 0], v[8 * i + 1]);
    q.y = pack_bf16x2(v[8 * i + 2], v[8 * i + 3]);
    q.z = pack_bf16x2(v[8 * i + 4], v[8 * i + 5]);
    q.w = pack_bf16x2(v[8 * i + 6], v[8 * i + 7]);
    *reinterpret_cast<uint4*>(buf + r * 64 + ((i ^ ((r >> 1) & 3)) << 4)) = q;
  }
}

__device__ __forceinline__ void load_any32(const void* base, int dtype, int64_t elem_off, bool vec_ok, int valid,
                                           float (&v)[32]) {
  if (dtype == NX_F32)
    load_row32<float>(reinterpret_cast<const float*>(base) + elem_off, vec_ok, valid, v);
  else
    load_row32<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(base) + elem_off, vec_ok, valid, v);
}

#ifdef NX_PROFILE_MMA
// Profiling build only (-DNX_PROFILE_MMA): per CTA, cycles the MMA-issuing thread spent in total, waiting for a
// free accumulator, waiting for TMA data, and between a stage's arrival and the commit of its MMAs (which blocks
// while the tensor-core queue is full), plus k-block and tile counts.  Read back with nx_gemm_prof_read.
__device__ long long g_mma_prof[148 * 8];
#define NX_PROF(x) x
#else
#define NX_PROF(x)
#endif

template <int BN, bool A_MN, bool B_MN, bool DIST>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const DevParams p, const uint32_t idesc, const __grid_constant__ DistParam<DIST> dist,
            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_aux) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128B swizzle pattern (descriptor base_offset = 0).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* store_base = smem + C::kStages * C::kStageBytes;  // 1 KiB aligned (stage sizes are multiples of it)
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_base + C::kStoreBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + C::kStages;      // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        Unit w = decode_unit(p, u);
        const int n0 = w.n0 * BN;
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            break;
          }
          uint8_t* sa = stage_base + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          const int k0 = kb * p.bk_elems;
          const CUtensorMap* ma = &tmap_a;
          const CUtensorMap* mb = &tmap_b;
          int am0 = w.m0, bn0 = n0;
          if constexpr (DIST) {
            // the tile's rows live in the memory of the rank that owns them: plain (non-multicast) TMA
            if (dist.a_sharded) {
              const int q = w.m0 / dist.a_rows;
              ma = &dist.a[q];
              am0 = w.m0 - q * dist.a_rows;
            }
            if (dist.b_sharded) {
              const int q = n0 / dist.b_rows;
              mb = &dist.b[q];
              bn0 = n0 - q * dist.b_rows;
            }
          }
          if (!A_MN) {
            tma_load_3d(sa, ma, &full_bar[stage], k0, am0, w.batch);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_3d(sa + j * (64 * kBK * 2), ma, &full_bar[stage], am0 + 64 * j, k0, w.batch);
          }
          if (!B_MN) {
            tma_load_3d(sb, mb, &full_bar[stage], k0, bn0, w.batch);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * kBK * 2), mb, &full_bar[stage], bn0 + 64 * j, k0, w.batch);
          }
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      NX_PROF(long long t_acc = 0; long long t_tma = 0; long long t_issue = 0; long long n_kb = 0; long long n_tiles = 0;
              const long long t_begin = clock64();)
      for (int u = blockIdx.x; u < p.num_units && ok; u += gridDim.x) {
        Unit w = decode_unit(p, u);
        NX_PROF(const long long c0 = clock64();)
        if (!mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag)) {
          atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        NX_PROF(t_acc += clock64() - c0; ++n_tiles;)
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          NX_PROF(const long long c1 = clock64();)
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutMma);
            break;
          }
          NX_PROF(const long long c2 = clock64(); t_tma += c2 - c1; ++n_kb;)
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stage_base + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int ks = 0; ks < kBK / 16; ++ks) {
            // K-major: 16 elements = 32 bytes inside the swizzled row.  MN-major: 16 k-rows = 2 KiB.
            const uint32_t a_addr = A_MN ? sa + ks * 2048 : sa + ks * 32;
            const uint32_t b_addr = B_MN ? sb + ks * 2048 : sb + ks * 32;
            const uint64_t da = make_smem_desc_sw128(a_addr, A_MN ? 64 * kBK * 2 : 16, 1024);
            const uint64_t db = make_smem_desc_sw128(b_addr, B_MN ? 64 * kBK * 2 : 16, 1024);
            if (p.fp8)
              umma_f8_ss(tmem_d, da, db, idesc, (kb > w.kb_begin || ks > 0) ? 1u : 0u);
            else
              umma_f16_ss(tmem_d, da, db, idesc, (kb > w.kb_begin || ks > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          NX_PROF(t_issue += clock64() - c2;)
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      NX_PROF(if (blockIdx.x < 148) {
        long long* o = g_mma_prof + blockIdx.x * 8;
        o[0] = clock64() - t_begin; o[1] = t_acc; o[2] = t_tma; o[3] = t_issue; o[4] = n_kb; o[5] = n_tiles;
      })
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;     // which half of the tile's columns this warp handles
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int u = blockIdx.x; u < p.num_units; u += gridDim.x) {
      Unit w = decode_unit(p, u);
      const int n0 = w.n0 * BN;
      const bool got = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {  // warp-uniform exit: the TMEM loads below need the whole warp
        if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const int row = w.m0 + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
#pragma unroll 1
      for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (p.tma_store) {
          // the staging tiles may be rewritten once the previous stores have read them; every lane stays in the
          // loop (rows past M carry garbage that the tiled store clips)
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        } else if (!row_ok) {
          continue;
        }
        const int valid = min(32, p.n - col0);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        if (p.scale_a != nullptr && row_ok) {
          const float sa_row = p.scale_a[row];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= sa_row;
        }
        if (p.scale_b != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= (j < valid) ? p.scale_b[col0 + j] : 0.0f;
        }

        if constexpr (DIST) {
          if (dist.out_scatter) {
            // GEMM -> reduce-scatter: add the tile into the FP32 buffer of the rank that owns these rows
            const int owner = row / dist.out_rows;
            float* op = dist.out[owner] + static_cast<int64_t>(row - owner * dist.out_rows) * p.ldo + col0;
            if ((valid == 32) && ((p.ldo & 3) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(op + j), "f"(v[j]), "f"(v[j + 1]),
                             "f"(v[j + 2]), "f"(v[j + 3])
                             : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) atomicAdd(op + j, v[j]);
            }
            continue;
          }
        }
        if (p.split_k > 1) {
          if (p.accumulate == 2) {
            // split-K slices add straight into the FP32 output (vector reductions in L2)
            float* op = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(row) * p.ldo + col0;
            if ((valid == 32) && ((p.ldo & 3) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(op + j), "f"(v[j]), "f"(v[j + 1]),
                             "f"(v[j + 2]), "f"(v[j + 3])
                             : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < valid) atomicAdd(op + j, v[j]);
            }
            continue;
          }
          float* wp = p.workspace + (static_cast<int64_t>(w.slice) * p.m + row) * p.n + col0;
          const bool vec = (valid == 32) && ((p.n & 3) == 0);
          store_row32_f32(wp, vec, valid, v);
          continue;
        }
        if (p.bias != nullptr) {
          float b[32];
          const bool vec = (valid == 32) && ((col0 & 7) == 0);
          load_any32(p.bias, p.bias_dtype, col0, vec, valid, b);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += b[j];
        }
        const int64_t aux_off = static_cast<int64_t>(row) * p.ld_aux + col0;
        const bool aux_vec = (valid == 32) && ((p.ld_aux & 7) == 0);
        if (p.act == NX_ACT_DGELU && p.aux_in != nullptr && row_ok) {
          float a[32];
          load_row32<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + aux_off, aux_vec, valid, a);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh_f(a[j]);
        }
        uint8_t* st_out = store_base + (warp - 2) * 4096;
        if (p.aux_out != nullptr) {
          if (p.tma_store) stage_row32_bf16(st_out + 2048, lane, v);
          else store_row32_bf16(reinterpret_cast<__nv_bfloat16*>(p.aux_out) + aux_off, aux_vec, valid, v);
        }
        if (p.act == NX_ACT_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_f(v[j]);
        } else if (p.act == NX_ACT_RELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = fmaxf(v[j], 0.0f);
        } else if (p.act == NX_ACT_SILU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = silu_f(v[j]);
        }
        if (p.residual != nullptr && row_ok) {
          float q[32];
          const bool vec = (valid == 32) && ((p.ld_res & 7) == 0);
          load_any32(p.residual, p.res_dtype, static_cast<int64_t>(row) * p.ld_res + col0, vec, valid, q);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += q[j];
        }
        const int64_t out_off = static_cast<int64_t>(w.batch) * p.stride_o + static_cast<int64_t>(row) * p.ldo + col0;
        const bool out_vec = (valid == 32) && ((p.ldo & 7) == 0) && ((p.stride_o & 7) == 0);
        if (p.accumulate) {
          float q[32];
          load_any32(p.out, p.out_dtype, out_off, out_vec, valid, q);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += q[j];
        }
        if (p.amax_out != nullptr && row_ok) {  // non-negative floats order like their bit patterns
          float am = 0.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < valid) am = fmaxf(am, fabsf(v[j]));
          if (am > 0.0f) atomicMax(p.amax_out, __float_as_uint(am));
        }
        if (p.tma_store) {
          stage_row32_bf16(st_out, lane, v);
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
          __syncwarp();
          const int row0 = w.m0 + quarter * 32;
          if (lane == 0 && row0 < p.m) {
            if (p.aux_out != nullptr) tma_store_3d(&tmap_aux, st_out + 2048, col0, row0, w.batch);
            tma_store_3d(&tmap_out, st_out, col0, row0, w.batch);
            tma_store_commit();
          }
        } else if (p.out_dtype == NX_F32) {
          store_row32_f32(reinterpret_cast<float*>(p.out) + out_off, out_vec, valid, v);
        } else {
          store_row32_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + out_off, out_vec, valid, v);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (p.tma_store && lane == 0) tma_store_wait_all();  // the staging tiles die with the CTA
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    // A wait ran out: give copies that are still in flight time to land before the CTA's shared
    // memory and TMEM go away.
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, bool A_MN, bool B_MN, bool DIST = false>
int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const DevParams& p, uint32_t in_fmt, int grid,
                   cudaStream_t stream, const DistParam<DIST>& dist = DistParam<DIST>{}, int fmt_b = -1,
                   const CUtensorMap* t_out = nullptr, const CUtensorMap* t_aux = nullptr) {
  using C = Cfg<BN>;
  static bool attr_set = false;
  auto kern = gemm_kernel<BN, A_MN, B_MN, DIST>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return -2;
    attr_set = true;
  }
  const uint32_t idesc = make_idesc(in_fmt, fmt_b < 0 ? in_fmt : static_cast<uint32_t>(fmt_b), A_MN, B_MN, kBM, BN);
  // unused store maps are passed as copies of an operand map: never dereferenced unless p.tma_store is set
  kern<<<grid, kThreads, C::kSmemBytes, stream>>>(ta, tb, p, idesc, dist, t_out ? *t_out : ta, t_aux ? *t_aux : ta);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* out, int out_dtype, int64_t ldo, int m,
                                     int n, int split_k, int accumulate) {
  const int64_t total = static_cast<int64_t>(m) * n;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < split_k; ++k) s += ws[static_cast<int64_t>(k) * total + i];
    const int r = static_cast<int>(i / n), c = static_cast<int>(i % n);
    const int64_t off = static_cast<int64_t>(r) * ldo + c;
    if (out_dtype == NX_F32) {
      float* o = reinterpret_cast<float*>(out);
      o[off] = accumulate ? o[off] + s : s;
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
      o[off] = __float2bfloat16_rn(accumulate ? __bfloat162float(o[off]) + s : s);
    }
  }
}

}  // namespace

extern "C" int nx_sm_count(void) {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  }
  return count;
}

extern "C" size_t nx_gemm_workspace_bytes(int m, int n, int split_k) {
  return split_k > 1 ? static_cast<size_t>(split_k) * m * n * sizeof(float) : 0;
}

extern "C" int nx_splitk_reduce(const float* workspace, void* out, int out_dtype, int64_t ldo, int m, int n,
                                int split_k, int accumulate, nx_stream_t stream) {
  const int64_t total = static_cast<int64_t>(m) * n;
  if (total == 0) return 0;
  int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 8));
  splitk_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(workspace, out, out_dtype, ldo, m, n,
                                                                              split_k, accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int nx_gemm(const NxGemmArgs* a, nx_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->m <= 0 || a->n <= 0 || a->k <= 0 || a->batch <= 0) return -1;
  const bool fp8 = a->in_dtype == NX_E4M3 || a->in_dtype == NX_E5M2;
  if (a->in_dtype != NX_BF16 && a->in_dtype != NX_F16 && !fp8) return -1;
  if (a->out_dtype != NX_BF16 && a->out_dtype != NX_F32) return -1;
  if (a->status == nullptr) return -1;
  const int b_dtype = a->b_dtype_plus1 > 0 ? a->b_dtype_plus1 - 1 : a->in_dtype;
  if (fp8 && (a->a_mn_major || a->b_mn_major || (b_dtype != NX_E4M3 && b_dtype != NX_E5M2))) return -1;
  if (!fp8 && b_dtype != a->in_dtype) return -1;
  // TMA: base 16-byte aligned, every non-innermost stride a multiple of 16 bytes.
  const int pitch_mask = fp8 ? 15 : 7;
  if ((reinterpret_cast<uintptr_t>(a->a) & 15) || (reinterpret_cast<uintptr_t>(a->b) & 15)) return -1;
  if ((a->lda & pitch_mask) || (a->ldb & pitch_mask)) return -1;
  if (a->batch > 1 && ((a->stride_a & pitch_mask) || (a->stride_b & pitch_mask))) return -1;
  int split = a->split_k < 1 ? 1 : a->split_k;
  if (split > 1 && a->batch != 1) return -1;
  if (split > 1 && a->accumulate == 2 && a->out_dtype != NX_F32) return -1;
  if (split > 1 && a->accumulate != 2 && a->workspace == nullptr) return -1;

  int bn = a->block_n;
  if (bn != 128 && bn != 256) bn = (a->n >= 256) ? 256 : 128;

  const int bk = fp8 ? 2 * kBK : kBK;  // elements per 128-byte swizzle row
  const int kb_total = (a->k + bk - 1) / bk;
  if (split > kb_total) split = kb_total;
  int kb_per = (kb_total + split - 1) / split;
  split = (kb_total + kb_per - 1) / kb_per;

  DevParams p{};
  p.out = a->out;
  p.bias = a->bias;
  p.aux_in = a->aux_in;
  p.aux_out = a->aux_out;
  p.residual = a->residual;
  p.workspace = a->workspace;
  p.status = a->status;
  p.ldo = a->ldo;
  p.ld_aux = a->ld_aux;
  p.ld_res = a->ld_res;
  p.stride_o = a->batch > 1 ? a->stride_o : 0;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  p.batch = a->batch;
  p.out_dtype = a->out_dtype;
  p.bias_dtype = a->bias_dtype;
  p.res_dtype = a->res_dtype;
  p.act = a->act;
  p.accumulate = a->accumulate;
  p.split_k = split;
  p.tiles_m = (a->m + kBM - 1) / kBM;
  p.tiles_n = (a->n + bn - 1) / bn;
  p.kb_total = kb_total;
  p.kb_per_slice = kb_per;
  p.num_units = p.tiles_m * p.tiles_n * split * a->batch;
  p.alpha = a->alpha;
  p.fp8 = fp8 ? 1 : 0;
  p.bk_elems = bk;
  p.scale_a = a->scale_a;
  p.scale_b = a->scale_b;
  p.amax_out = reinterpret_cast<unsigned int*>(a->amax_out);

  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (a->in_dtype == NX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const int eb = fp8 ? 1 : 2;
  CUtensorMap ta, tb;
  const uint64_t sa = a->batch > 1 ? static_cast<uint64_t>(a->stride_a) : 0;
  const uint64_t sb = a->batch > 1 ? static_cast<uint64_t>(a->stride_b) : 0;
  int rc;
  if (!a->a_mn_major)
    rc = nx::make_tensor_map_3d(&ta, dt, eb, a->a, a->k, a->m, a->batch, a->lda, sa, bk, kBM);
  else
    rc = nx::make_tensor_map_3d(&ta, dt, 2, a->a, a->m, a->k, a->batch, a->lda, sa, 64, kBK);
  if (rc != 0) return rc;
  if (!a->b_mn_major)
    rc = nx::make_tensor_map_3d(&tb, dt, eb, a->b, a->k, a->n, a->batch, a->ldb, sb, bk, bn);
  else
    rc = nx::make_tensor_map_3d(&tb, dt, 2, a->b, a->n, a->k, a->batch, a->ldb, sb, 64, kBK);
  if (rc != 0) return rc;

  // BF16 results leave through shared memory and tiled stores (full-line writes) when the layout allows a map
  CUtensorMap to, tx;
  const bool can_tma_out = a->out_dtype == NX_BF16 && split == 1 && a->accumulate == 0 && (a->ldo & 7) == 0 &&
                           (reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && (a->batch == 1 || (a->stride_o & 7) == 0) &&
                           (a->aux_out == nullptr || ((a->ld_aux & 7) == 0 && (reinterpret_cast<uintptr_t>(a->aux_out) & 15) == 0 &&
                                                      a->batch == 1));
  p.tma_store = 0;
  static const bool direct_only = std::getenv("NX_GEMM_DIRECT_STORE") != nullptr;  // measurement switch
  if (can_tma_out && !direct_only) {
    const uint64_t so = a->batch > 1 ? static_cast<uint64_t>(a->stride_o) : 0;
    rc = nx::make_tensor_map_3d(&to, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->out, a->n, a->m, a->batch, a->ldo, so, 32, 32,
                                CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc == 0 && a->aux_out != nullptr)
      rc = nx::make_tensor_map_3d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->aux_out, a->n, a->m, 1, a->ld_aux, 0, 32, 32,
                                  CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc == 0) p.tma_store = 1;
  }

  int sms = nx_sm_count();
  if (sms <= 0) return -2;
  if (a->max_ctas > 0 && a->max_ctas < sms) sms = a->max_ctas;
  const int grid = p.num_units < sms ? p.num_units : sms;
  const uint32_t fmt = fp8 ? (a->in_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2) : (a->in_dtype == NX_BF16 ? kFmtBF16 : kFmtF16);
  const int fmt_b = fp8 ? static_cast<int>(b_dtype == NX_E4M3 ? kFmtE4M3 : kFmtE5M2) : -1;

#define NX_LAUNCH(BN_, AM_, BM_) \
  rc = launch_variant<BN_, AM_, BM_>(ta, tb, p, fmt, grid, stream, DistParam<false>{}, fmt_b, p.tma_store ? &to : nullptr, \
                                     (p.tma_store && a->aux_out) ? &tx : nullptr)
  if (bn == 256) {
    if (!a->a_mn_major && !a->b_mn_major) NX_LAUNCH(256, false, false);
    else if (!a->a_mn_major && a->b_mn_major) NX_LAUNCH(256, false, true);
    else if (a->a_mn_major && !a->b_mn_major) NX_LAUNCH(256, true, false);
    else NX_LAUNCH(256, true, true);
  } else {
    if (!a->a_mn_major && !a->b_mn_major) NX_LAUNCH(128, false, false);
    else if (!a->a_mn_major && a->b_mn_major) NX_LAUNCH(128, false, true);
    else if (a->a_mn_major && !a->b_mn_major) NX_LAUNCH(128, true, false);
    else NX_LAUNCH(128, true, true);
  }
#undef NX_LAUNCH
  return rc;
}

// K-major operands only; batch 1; no split-K.  Rows per rank must be multiples of the tile size.
extern "C" int nx_gemm_dist(const NxGemmArgs* a, const NxGemmDist* d, nx_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || d == nullptr || a->m <= 0 || a->n <= 0 || a->k <= 0 || a->status == nullptr) return -1;
  if (a->batch != 1 || a->a_mn_major || a->b_mn_major || a->in_dtype != NX_BF16) return -1;
  const int n = d->n_ranks;
  if (n < 1 || n > NX_MAX_PEERS || (a->lda & 7) || (a->ldb & 7)) return -1;
  if (d->a_sharded && (a->m % n || (a->m / n) % kBM)) return -1;
  int bn = (a->n >= 256) ? 256 : 128;
  if (d->b_sharded) {
    if (a->n % n) return -1;
    const int per = a->n / n;
    if (per % 256 == 0) bn = 256;
    else if (per % 128 == 0) bn = 128;
    else return -1;
  }
  if (d->out_scatter && (a->m % n || (a->m / n) % kBM || a->out_dtype != NX_F32)) return -1;

  DevParams p{};
  p.out = a->out;
  p.bias = a->bias;
  p.aux_in = a->aux_in;
  p.aux_out = a->aux_out;
  p.residual = a->residual;
  p.status = a->status;
  p.ldo = a->ldo;
  p.ld_aux = a->ld_aux;
  p.ld_res = a->ld_res;
  p.m = a->m;
  p.n = a->n;
  p.k = a->k;
  p.batch = 1;
  p.out_dtype = a->out_dtype;
  p.bias_dtype = a->bias_dtype;
  p.res_dtype = a->res_dtype;
  p.act = a->act;
  p.accumulate = a->accumulate;
  p.split_k = 1;
  p.tiles_m = (a->m + kBM - 1) / kBM;
  p.tiles_n = (a->n + bn - 1) / bn;
  p.kb_total = (a->k + kBK - 1) / kBK;
  p.kb_per_slice = p.kb_total;
  p.fp8 = 0;
  p.bk_elems = kBK;
  p.scale_a = nullptr;
  p.scale_b = nullptr;
  p.amax_out = nullptr;
  p.num_units = p.tiles_m * p.tiles_n;
  p.alpha = a->alpha;

  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  DistParam<true> dist{};
  dist.a_sharded = d->a_sharded;
  dist.b_sharded = d->b_sharded;
  dist.out_scatter = d->out_scatter;
  dist.a_rows = d->a_sharded ? a->m / n : a->m;
  dist.b_rows = d->b_sharded ? a->n / n : a->n;
  dist.out_rows = d->out_scatter ? a->m / n : a->m;
  CUtensorMap ta, tb;
  int rc;
  for (int q = 0; q < n; ++q) {
    if (d->a_sharded) {
      if (reinterpret_cast<uintptr_t>(d->a_ptrs[q]) & 15) return -1;
      if ((rc = nx::make_tensor_map_3d(&dist.a[q], dt, 2, d->a_ptrs[q], a->k, dist.a_rows, 1, a->lda, 0, kBK, kBM))) return rc;
    }
    if (d->b_sharded) {
      if (reinterpret_cast<uintptr_t>(d->b_ptrs[q]) & 15) return -1;
      if ((rc = nx::make_tensor_map_3d(&dist.b[q], dt, 2, d->b_ptrs[q], a->k, dist.b_rows, 1, a->ldb, 0, kBK, bn))) return rc;
    }
    dist.out[q] = static_cast<float*>(d->out_ptrs[q]);
  }
  const void* a0 = d->a_sharded ? d->a_ptrs[d->rank] : a->a;
  const void* b0 = d->b_sharded ? d->b_ptrs[d->rank] : a->b;
  if ((rc = nx::make_tensor_map_3d(&ta, dt, 2, a0, a->k, d->a_sharded ? dist.a_rows : a->m, 1, a->lda, 0, kBK, kBM))) return rc;
  if ((rc = nx::make_tensor_map_3d(&tb, dt, 2, b0, a->k, d->b_sharded ? dist.b_rows : a->n, 1, a->ldb, 0, kBK, bn))) return rc;
  int sms = nx_sm_count();
  if (sms <= 0) return -2;
  const int grid = p.num_units < sms ? p.num_units : sms;
  if (bn == 256) return launch_variant<256, false, false, true>(ta, tb, p, kFmtBF16, grid, stream, dist);
  return launch_variant<128, false, false, true>(ta, tb, p, kFmtBF16, grid, stream, dist);
}

#ifdef NX_PROFILE_MMA
extern "C" int nx_gemm_prof_read(long long* out) {
  return cudaMemcpyFromSymbol(out, g_mma_prof, sizeof(long long) * 148 * 8) == cudaSuccess ? 0 : -1;
}
#endif
