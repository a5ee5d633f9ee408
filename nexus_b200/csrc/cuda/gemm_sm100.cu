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
// The pair kernel is launched with programmatic stream serialization: its set-up (barriers, TMEM, cluster sync) runs
// while the previous kernel of the stream drains, and `griddepcontrol.wait` orders everything that touches global
// memory after that kernel.  The kernels that precede GEMMs in a training step issue `griddepcontrol.launch_dependents`.
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

// PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2); each stages its own 128 A rows
// and half of the B rows, so a k-block costs each SM 32 KiB of shared-memory traffic instead of 48 KiB.
template <int BN, bool PAIR = false>
struct Cfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;  // B rows staged by one CTA
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // per epilogue warp: a ring of [32 rows][32 bf16] staging tiles for the tiled stores (the pair's smaller stages
  // leave room for four, so stores of out AND aux_out are double-buffered)
#ifndef NX_PAIR_SLOTS
#define NX_PAIR_SLOTS 4
#endif
  static constexpr int kStoreSlots = PAIR ? NX_PAIR_SLOTS : 2;
  static constexpr int kStoreBytes = 8 * kStoreSlots * 2048;
  // 4 stages (BN=256), 6 (BN=128); the pair: 5 with four staging tiles per warp, 6 with two
  static constexpr int kStages = (PAIR ? kSmemBudget + 32 * 1024 - kStoreBytes : kSmemBudget) / kStageBytes;
  static constexpr int kTmemCols = 2 * BN;
  // the pair's bias strips: [tile parity][column half][128 floats]; its buffer is declared 1 KiB-aligned, the
  // single-CTA kernel rounds its base up inside a 1 KiB slack
  static constexpr int kBiasBytes = PAIR ? 2 * 2 * 128 * 4 : 0;
  static constexpr int kSlackBytes = PAIR ? 0 : 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kBiasBytes + kSlackBytes + 256 /*barriers*/;
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
  int n_fastest;           // consecutive work units walk along N (A tile reused from L2) instead of along M
  // All-gather fused into the GEMM (nx_gemm_ag): A is this rank's [M][lda] gather buffer; the last `ag_copiers`
  // CTAs of the grid push this rank's row block into every peer's buffer and raise per-chunk flags there, while
  // the GEMM CTAs start with the local rows and take the other ranks' rows in ring order as their flags come up.
  int ag_ranks, ag_rank, ag_rows, ag_copiers;  // ag_ranks <= 1: plain GEMM
  int64_t ag_ld_bytes;                        // bytes between rows of the gather buffers
  int ag_row_bytes;                           // bytes of one row that are copied (K * 2)
  const int* ag_counter;                      // generation of this call = *ag_counter + 1
  void* ag_gather[NX_MAX_PEERS];
  int* ag_flags[NX_MAX_PEERS];                // per rank: int[ag_ranks][ag_rows / 128]
  int rot_rows;                               // work units start at this row and wrap around (ring order)
  // GEMM fused with a reduce-scatter (nx_gemm_rs): `out` is a local BF16 [M][ldo] buffer of partial sums; every
  // epilogue warp counts a finished tile on rs_done[row block], and the last `rs_copiers` CTAs store each complete
  // 256-row block into slot `rs_rank` of the buffer of the rank that owns those rows.
  int rs_ranks, rs_rank, rs_rows, rs_copiers;  // rs_ranks <= 1: plain GEMM
  int rs_expected;                            // arrivals that complete one row block (16 per column tile)
  int rs_copy_own;                            // 0: the rows this rank owns stay in `out` only (the caller sums them from there)
  int* rs_done;                               // [M / 256], zeroed by the caller before the launch
  void* rs_slots[NX_MAX_PEERS];               // per rank: BF16 [rs_ranks][rs_rows][ldo]
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
  int k_rows;                    // K rows per rank when an MN-major operand is sharded along K
  int a_sharded, b_sharded, out_scatter, rank;
};

template <int TILE_M = kBM>
__device__ __forceinline__ Unit decode_unit(const DevParams& p, int u) {
  Unit w;
  int tm, tn;
  if (p.n_fastest) {
    tn = u % p.tiles_n;
    u /= p.tiles_n;
    w.slice = u % p.split_k;
    u /= p.split_k;
    tm = u % p.tiles_m;
    w.batch = u / p.tiles_m;
  } else {
    tm = u % p.tiles_m;
    u /= p.tiles_m;
    w.slice = u % p.split_k;
    u /= p.split_k;
    tn = u % p.tiles_n;
    w.batch = u / p.tiles_n;
  }
  w.m0 = tm * TILE_M;
  if (p.rot_rows > 0) {  // ring order: all-gather starts with the local rows, reduce-scatter ends with them
    w.m0 += p.rot_rows;
    if (w.m0 >= p.m) w.m0 -= p.m;
  }
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
// counters of the profiling build: one row of 8 per CTA (or CTA pair), for grids of up to kProfRows CTAs
constexpr int kProfRows = 256;
__device__ long long g_mma_prof[kProfRows * 8];
__device__ long long g_epi_prof[kProfRows * 8];  // first epilogue warp: busy cycles per tile, TMEM-load wait, store-slot wait, tiles
#define NX_PROF(x) x
#else
#define NX_PROF(x)
#endif

// FAST (pair only): the epilogue of the training GEMMs and nothing else - BF16 result through tiled stores,
// optional bias, GELU with saved pre-activation, or dGELU of a saved pre-activation - with the bias staged once
// per tile in shared memory and one proxy fence / store group per tile (two with aux_out).
// Copier CTAs move contiguous byte ranges from this GPU's memory into a peer's (or its own) memory.  Loads are
// untiled bulk copies (TMA engine) from LOCAL global memory into the CTA's shared memory, two stages of kCopyStage
// bytes in flight so that the load latency hides behind the previous stage's stores; the stores are plain 16-byte
// stores by all threads (posted writes, coalesced), so nothing but this GPU's own memory is ever bulk-loaded.
constexpr int kCopyPiece = 16 * 1024;
constexpr int kCopyPieces = 6;
constexpr int kCopyStage = kCopyPiece * kCopyPieces;  // 96 KiB per stage, two stages

struct CopierSmem {
  uint64_t* bars;      // [2]
  volatile int* flag;  // scratch int for CTA-wide decisions
  uint8_t* buf;        // 2 * kCopyStage bytes, 128-byte aligned
  uint32_t phase[2];
};

__device__ __forceinline__ CopierSmem copier_smem_init(uint8_t* smem_raw) {
  CopierSmem cs;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  cs.bars = reinterpret_cast<uint64_t*>(base);
  cs.flag = reinterpret_cast<volatile int*>(base + 16);
  cs.buf = base + 128;
  cs.phase[0] = cs.phase[1] = 0;
  if (threadIdx.x == 0) {
    mbar_init(&cs.bars[0], 1);
    mbar_init(&cs.bars[1], 1);
    *cs.flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  return cs;
}

// All threads of the CTA call this with the same arguments.  Returns false when a wait ran out (status is set).
__device__ __forceinline__ bool copier_copy(CopierSmem& cs, const char* __restrict__ src, char* __restrict__ dst, int64_t bytes,
                                            int* status) {
  const int rounds = static_cast<int>((bytes + kCopyStage - 1) / kCopyStage);
  auto issue = [&](int r) {  // thread 0 only
    const int s = r & 1;
    const int64_t off = static_cast<int64_t>(r) * kCopyStage;
    const int len = static_cast<int>(min(static_cast<int64_t>(kCopyStage), bytes - off));
    mbar_arrive_expect_tx(&cs.bars[s], static_cast<uint32_t>(len));
    for (int o = 0; o < len; o += kCopyPiece)
      bulk_load(cs.buf + s * kCopyStage + o, src + off + o, static_cast<uint32_t>(min(kCopyPiece, len - o)), &cs.bars[s]);
  };
  if (threadIdx.x == 0) issue(0);
  for (int r = 0; r < rounds; ++r) {
    const int s = r & 1;
    if (threadIdx.x == 0 && r + 1 < rounds) issue(r + 1);  // the other stage was drained before the last barrier
    if (!mbar_wait_bounded(&cs.bars[s], cs.phase[s], cs.flag)) {
      atomicCAS(status, 0, kStatusTimeoutProducer);
      return false;  // every thread sees the same barrier and the shared abort flag: the exit is CTA-wide
    }
    cs.phase[s] ^= 1u;
    const int64_t off = static_cast<int64_t>(r) * kCopyStage;
    const int len = static_cast<int>(min(static_cast<int64_t>(kCopyStage), bytes - off));
    const uint8_t* sb = cs.buf + s * kCopyStage;
    for (int i = threadIdx.x * 16; i < len; i += blockDim.x * 16)
      *reinterpret_cast<uint4*>(dst + off + i) = *reinterpret_cast<const uint4*>(sb + i);
    __syncthreads();  // the stage may be refilled
  }
  return true;
}

// Copier CTA of the all-gather GEMM: pushes chunk after chunk (128 rows) of this rank's row block into the gather
// buffer of one peer after the other (the peer that needs it soonest first), then raises that chunk's flag on the peer.
// Plain stores to peer memory; the release store of the flag follows a system-scope fence by every storing thread.
__device__ __forceinline__ void ag_copier_run(const DevParams& p, int cid, uint8_t* smem_raw) {
  const int n = p.ag_ranks, r = p.ag_rank;
  const int chunks = p.ag_rows / kBM;
  const int epoch = *reinterpret_cast<const volatile int*>(p.ag_counter) + 1;
  CopierSmem cs = copier_smem_init(smem_raw);
  const bool contiguous = p.ag_ld_bytes == p.ag_row_bytes;
  const char* src_base = reinterpret_cast<const char*>(p.ag_gather[r]) + static_cast<int64_t>(r) * p.ag_rows * p.ag_ld_bytes;
  for (int s = 1; s < n; ++s) {
    const int dest = (r - s + n) % n;
    char* dst_base = reinterpret_cast<char*>(p.ag_gather[dest]) + static_cast<int64_t>(r) * p.ag_rows * p.ag_ld_bytes;
    for (int j = cid; j < chunks; j += p.ag_copiers) {
      const char* src = src_base + static_cast<int64_t>(j) * kBM * p.ag_ld_bytes;
      char* dst = dst_base + static_cast<int64_t>(j) * kBM * p.ag_ld_bytes;
      if (contiguous) {
        if (!copier_copy(cs, src, dst, static_cast<int64_t>(kBM) * p.ag_row_bytes, p.status)) return;
      } else {
        for (int row = 0; row < kBM; ++row)
          if (!copier_copy(cs, src + row * p.ag_ld_bytes, dst + row * p.ag_ld_bytes, p.ag_row_bytes, p.status)) return;
      }
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x == 0)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.ag_flags[dest] + r * chunks + j), "r"(epoch) : "memory");
    }
  }
}

// Copier CTA of the reduce-scatter GEMM: takes finished 256-row blocks (in the order the GEMM CTAs finish them) and
// copies them from the local buffer of partial sums into slot `rs_rank` of the owner's buffer.
__device__ __forceinline__ void rs_copier_run(const DevParams& p, int cid, uint8_t* smem_raw) {
  const int blocks = p.m / (2 * kBM);
  const int64_t ld_bytes = p.ldo * 2;
  const int row_bytes = p.n * 2;
  const bool contiguous = ld_bytes == row_bytes;
  const int first = p.rot_rows / (2 * kBM);
  CopierSmem cs = copier_smem_init(smem_raw);
  // copier `cid` takes every rs_copiers-th block of the ring order: the copiers work on different blocks at once
  for (int i = cid; i < blocks; i += p.rs_copiers) {
    int rb = first + i;
    if (rb >= blocks) rb -= blocks;
    const int row0 = rb * 2 * kBM;
    const int owner = row0 / p.rs_rows;
    if (owner == p.rs_rank && !p.rs_copy_own) continue;  // stays in `out`; nothing to wait for
    if (threadIdx.x == 0) {
      *cs.flag = 0;
      const uint64_t t0 = globaltimer_ns();
      for (;;) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p.rs_done + rb) : "memory");
        if (v >= p.rs_expected) break;
        if (globaltimer_ns() - t0 > NX_WAIT_LIMIT_NS) {
          atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          *cs.flag = 1;
          break;
        }
        __nanosleep(200);
      }
      asm volatile("fence.proxy.async;" ::: "memory");  // the block was written by TMA stores and is read by bulk loads
    }
    __syncthreads();
    if (*cs.flag) return;
    const char* src = reinterpret_cast<const char*>(p.out) + static_cast<int64_t>(row0) * ld_bytes;
    char* dst = reinterpret_cast<char*>(p.rs_slots[owner]) +
                (static_cast<int64_t>(p.rs_rank) * p.rs_rows + (row0 - owner * p.rs_rows)) * ld_bytes;
    if (contiguous) {
      if (!copier_copy(cs, src, dst, static_cast<int64_t>(2 * kBM) * row_bytes, p.status)) return;
    } else {
      for (int row = 0; row < 2 * kBM; ++row)
        if (!copier_copy(cs, src + row * ld_bytes, dst + row * ld_bytes, row_bytes, p.status)) return;
    }
  }
  __threadfence_system();  // the partial sums are in the owners' memory before this grid counts as complete
}

// Producer side of the all-gather GEMM: rows [row0, row0 + 128) belong to rank row0 / ag_rows; unless they are this
// rank's own, wait (bounded) until their owner's copier has raised the chunk's flag for this call.
__device__ __forceinline__ bool ag_wait_rows(const DevParams& p, int row0, int epoch, volatile int* abort_flag) {
  const int q = row0 / p.ag_rows;
  if (q == p.ag_rank) return true;
  const int chunks = p.ag_rows / kBM;
  const int* flag = p.ag_flags[p.ag_rank] + q * chunks + (row0 - q * p.ag_rows) / kBM;
  const uint64_t t0 = globaltimer_ns();
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= epoch) break;
    if (*abort_flag != 0 || globaltimer_ns() - t0 > NX_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      atomicCAS(p.status, 0, kStatusTimeoutPeer);
      return false;
    }
    __nanosleep(100);
  }
  asm volatile("fence.proxy.async;" ::: "memory");  // the rows were written through the generic proxy; TMA reads them
  return true;
}

template <int BN, bool A_MN, bool B_MN, bool DIST, bool PAIR = false, bool FAST = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const DevParams p, const uint32_t idesc, const __grid_constant__ DistParam<DIST> dist,
            const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_aux) {
  using C = Cfg<BN, PAIR>;
  static_assert(!(PAIR && DIST), "the CTA-pair tile is for single-GPU operands");
  static_assert(!FAST || PAIR, "the lean epilogue is built for the pair kernel");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // all-gather GEMM: the last ag_copiers CTAs (whole clusters) only move data and never touch barriers or TMEM
  const int gemm_ctas = static_cast<int>(gridDim.x) - (p.ag_ranks > 1 ? p.ag_copiers : 0) - (p.rs_ranks > 1 ? p.rs_copiers : 0);
  if (static_cast<int>(blockIdx.x) >= gemm_ctas) {
    pdl_wait();  // this rank's rows come from the previous kernel of the stream
    if (p.ag_ranks > 1) ag_copier_run(p, static_cast<int>(blockIdx.x) - gemm_ctas, smem_raw);
    else rs_copier_run(p, static_cast<int>(blockIdx.x) - gemm_ctas, smem_raw);
    return;
  }
  if constexpr (PAIR) {
    // no slack to round the base up in: refuse to run on a base that is not 1 KiB-aligned (same in every CTA)
    if ((smem_u32(smem_raw) & 1023u) != 0u) {
      if (threadIdx.x == 0) atomicCAS(p.status, 0, kStatusBadArgument);
      return;
    }
  }
  // 1024-byte alignment: required by the 128B swizzle pattern (descriptor base_offset = 0).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* store_base = smem + C::kStages * C::kStageBytes;  // 1 KiB aligned (stage sizes are multiples of it)
  float* bias_strip = reinterpret_cast<float*>(store_base + C::kStoreBytes);  // pair only
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_base + C::kStoreBytes + C::kBiasBytes);
  uint64_t* full_bar = bars;                    // [kStages]
  uint64_t* empty_bar = bars + C::kStages;      // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;  // [2]
  uint64_t* tempty_bar = tfull_bar + 2;         // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // pair: consecutive CTAs form a cluster; the even one issues the MMAs and owns the barriers both wait on
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int unit_first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int unit_step = PAIR ? (gemm_ctas >> 1) : gemm_ctas;
  constexpr int kTileM = PAIR ? 2 * kBM : kBM;
  const int m_off = static_cast<int>(cta_rank) * kBM;  // this CTA's rows inside the pair's tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], PAIR ? 16 : 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before anything may signal them
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(tmem_slot, C::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, C::kTmemCols);
      tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this CTA's own state: when the launch allows it, it ran while the previous kernel
  // of the stream was still finishing.  From here on operands, bias, residual and outputs are read and written.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int ag_epoch = p.ag_ranks > 1 ? *reinterpret_cast<const volatile int*>(p.ag_counter) + 1 : 0;
      for (int u = unit_first; u < p.num_units && ok; u += unit_step) {
        Unit w = decode_unit<kTileM>(p, u);
        w.m0 += m_off;
        const int n0 = w.n0 * BN;
        if (p.ag_ranks > 1 && !ag_wait_rows(p, w.m0, ag_epoch, abort_flag)) {
          ok = false;
          break;
        }
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            atomicCAS(p.status, 0, kStatusTimeoutProducer);
            break;
          }
          uint8_t* sa = stage_base + stage * C::kStageBytes;
          uint8_t* sb = sa + C::kABytes;
          const int k0 = kb * p.bk_elems;
          // debug builds: the tile must start inside the operands (partial tiles are zero-filled by TMA, but a tile
          // that starts outside means the unit decoding went wrong) and x must be 16-byte aligned
          if (!NX_INDEX_OK(w.m0 - m_off >= 0 && w.m0 - m_off < p.m && n0 >= 0 && n0 < p.n && k0 >= 0 && k0 < p.k &&
                           (k0 & 7) == 0 && w.batch >= 0 && w.batch < p.batch, p.status)) {
            ok = false;
            *abort_flag = 1;
            break;
          }
          if constexpr (PAIR) {
            // both CTAs' bytes are counted on the even CTA's barrier, which that CTA arms for the pair
            if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2 * C::kStageBytes);
            const uint32_t bar = mapa_shared(smem_u32(&full_bar[stage]), 0);
            const int bn0 = n0 + static_cast<int>(cta_rank) * C::kBRows;
            if (!A_MN) {
              tma_load_3d_pair(sa, &tmap_a, bar, k0, w.m0, w.batch);
            } else {
#pragma unroll
              for (int j = 0; j < kBM / 64; ++j)
                tma_load_3d_pair(sa + j * (64 * kBK * 2), &tmap_a, bar, w.m0 + 64 * j, k0, w.batch);
            }
            if (!B_MN) {
              tma_load_3d_pair(sb, &tmap_b, bar, k0, bn0, w.batch);
            } else {
#pragma unroll
              for (int j = 0; j < C::kBRows / 64; ++j)
                tma_load_3d_pair(sb + j * (64 * kBK * 2), &tmap_b, bar, bn0 + 64 * j, k0, w.batch);
            }
            if (++stage == C::kStages) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
          }
          mbar_arrive_expect_tx(&full_bar[stage], C::kStageBytes);
          const CUtensorMap* ma = &tmap_a;
          const CUtensorMap* mb = &tmap_b;
          int am0 = w.m0, bn0 = n0, ak0 = k0, bk0 = k0;
          if constexpr (DIST) {
            // the tile lives in the memory of the rank that owns it: plain (non-multicast) TMA from peer memory
            if (dist.a_sharded == NX_DIST_ROWS) {
              const int q = w.m0 / dist.a_rows;
              ma = &dist.a[q];
              am0 = w.m0 - q * dist.a_rows;
            } else if (dist.a_sharded == NX_DIST_K) {
              const int q = k0 / dist.k_rows;
              ma = &dist.a[q];
              ak0 = k0 - q * dist.k_rows;
            }
            if (dist.b_sharded == NX_DIST_ROWS) {
              const int q = n0 / dist.b_rows;
              mb = &dist.b[q];
              bn0 = n0 - q * dist.b_rows;
            } else if (dist.b_sharded == NX_DIST_K) {
              const int q = k0 / dist.k_rows;
              mb = &dist.b[q];
              bk0 = k0 - q * dist.k_rows;
            }
          }
          if (!A_MN) {
            tma_load_3d(sa, ma, &full_bar[stage], ak0, am0, w.batch);
          } else {
#pragma unroll
            for (int j = 0; j < kBM / 64; ++j)
              tma_load_3d(sa + j * (64 * kBK * 2), ma, &full_bar[stage], am0 + 64 * j, ak0, w.batch);
          }
          if (!B_MN) {
            tma_load_3d(sb, mb, &full_bar[stage], bk0, bn0, w.batch);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * (64 * kBK * 2), mb, &full_bar[stage], bn0 + 64 * j, bk0, w.batch);
          }
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if constexpr (PAIR) {
        // The even CTA's commits also arrive on this CTA's barriers: wait until every stage filled here has been
        // released, so that no arrival is still on its way when the CTA leaves.
        for (int s = 0; s < C::kStages && ok; ++s) {
          ok = mbar_wait_bounded(&empty_bar[stage], phase ^ 1u, abort_flag);
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    // The whole warp walks the loop so that addresses and descriptors stay in uniform registers; one elected lane
    // issues the MMAs and the commits (issuing from a lone lane of a diverged warp costs ~100 cycles per MMA in
    // register-to-uniform moves).
    if (cta_rank == 0) {
      const bool leader = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      NX_PROF(long long t_acc = 0; long long t_tma = 0; long long t_issue = 0; long long n_kb = 0; long long n_tiles = 0;
              const long long t_begin = clock64();)
      for (int u = unit_first; u < p.num_units && ok; u += unit_step) {
        Unit w = decode_unit<kTileM>(p, u);
        NX_PROF(const long long c0 = clock64();)
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(&tempty_bar[acc], acc_phase ^ 1u, abort_flag))) {
          if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
          break;
        }
        NX_PROF(t_acc += clock64() - c0; ++n_tiles;)
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = w.kb_begin; kb < w.kb_end; ++kb) {
          NX_PROF(const long long c1 = clock64();)
          if (!__all_sync(0xffffffffu, mbar_wait_bounded(&full_bar[stage], phase, abort_flag))) {
            ok = false;
            if (leader) atomicCAS(p.status, 0, kStatusTimeoutMma);
            break;
          }
          NX_PROF(const long long c2 = clock64(); t_tma += c2 - c1; ++n_kb;)
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stage_base + stage * C::kStageBytes);
          const uint32_t sb = sa + C::kABytes;
          const uint64_t da0 = make_smem_desc_sw128(sa, A_MN ? 64 * kBK * 2 : 16, 1024);
          const uint64_t db0 = make_smem_desc_sw128(sb, B_MN ? 64 * kBK * 2 : 16, 1024);
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < kBK / 16; ++ks) {
              // K-major: 16 elements = 32 bytes inside the swizzled row.  MN-major: 16 k-rows = 2 KiB.  (address field: >> 4)
              const uint64_t da = da0 + static_cast<uint64_t>(A_MN ? ks * 128 : ks * 2);
              const uint64_t db = db0 + static_cast<uint64_t>(B_MN ? ks * 128 : ks * 2);
              if constexpr (PAIR)
                umma_f16_ss_pair(tmem_d, da, db, idesc, (kb > w.kb_begin || ks > 0) ? 1u : 0u);
              else if (p.fp8)
                umma_f8_ss(tmem_d, da, db, idesc, (kb > w.kb_begin || ks > 0) ? 1u : 0u);
              else
                umma_f16_ss(tmem_d, da, db, idesc, (kb > w.kb_begin || ks > 0) ? 1u : 0u);
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if constexpr (PAIR) umma_commit_pair(&empty_bar[stage], 3);
            else umma_commit(&empty_bar[stage]);
          }
          __syncwarp();
          NX_PROF(t_issue += clock64() - c2;)
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        // accumulator complete (each CTA of a pair holds its 128 rows)
        if (leader) {
          if constexpr (PAIR) umma_commit_pair(&tfull_bar[acc], 3);
          else umma_commit(&tfull_bar[acc]);
        }
        __syncwarp();
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      NX_PROF(if (blockIdx.x < kProfRows && leader) {
        long long* o = g_mma_prof + (PAIR ? blockIdx.x >> 1 : blockIdx.x) * 8;
        o[0] = clock64() - t_begin; o[1] = t_acc; o[2] = t_tma; o[3] = t_issue; o[4] = n_kb; o[5] = n_tiles;
      })
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;         // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;     // which half of the tile's columns this warp handles
    int acc = 0;
    uint32_t acc_phase = 0;
    int ring = 0;  // next staging tile of this warp
    (void)ring;

    if constexpr (FAST) {
      uint8_t* const st_base = store_base + (warp - 2) * (C::kStoreSlots * 2048);
      const int per = p.aux_out != nullptr ? 2 : 1;
      const int group = C::kStoreSlots / per;  // chunks per proxy fence and committed store group
      const int c_begin = half * (BN / 64), c_end = (half + 1) * (BN / 64);
      int tile_parity = 0;
      for (int u = unit_first; u < p.num_units; u += unit_step, tile_parity ^= 1) {
        Unit w = decode_unit<kTileM>(p, u);
        w.m0 += m_off;
        const int n0 = w.n0 * BN;
        const int row = w.m0 + quarter * 32 + lane;
        const bool row_ok = row < p.m;
        // While the tile's MMAs still run: the first warp of each column half puts the half's 128 bias values in
        // shared memory (zeros past N); the four warps of the half meet on a named barrier.  Two strips alternate,
        // so a warp that is a tile ahead does not overwrite what a slower one still reads.
        const float* strip = bias_strip + (tile_parity * 2 + half) * 128;
        if (p.bias != nullptr) {
          if (quarter == 0) {
            const int col = n0 + half * 128 + lane * 4;
            float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (col + 3 < p.n && (p.bias_dtype == NX_F32 || (col & 3) == 0)) {
              if (p.bias_dtype == NX_F32) {
                const float* bp = reinterpret_cast<const float*>(p.bias) + col;
                b4 = make_float4(bp[0], bp[1], bp[2], bp[3]);
              } else {
                const uint2 q = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.bias) + col);
                unpack_bf16x2(q.x, b4.x, b4.y);
                unpack_bf16x2(q.y, b4.z, b4.w);
              }
            } else {
              float t[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                t[j] = 0.0f;
                if (col + j < p.n)
                  t[j] = p.bias_dtype == NX_F32 ? reinterpret_cast<const float*>(p.bias)[col + j]
                                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + j]);
              }
              b4 = make_float4(t[0], t[1], t[2], t[3]);
            }
            *reinterpret_cast<float4*>(const_cast<float*>(strip) + lane * 4) = b4;
          }
          asm volatile("bar.sync %0, 128;" ::"r"(1 + half) : "memory");
        }
        const __nv_bfloat16* aux_row = reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + static_cast<int64_t>(row) * p.ld_aux;
        const bool dgelu = p.act == NX_ACT_DGELU && p.aux_in != nullptr;
        if (dgelu && row_ok && n0 + c_begin * 32 < p.n) prefetch_l1(aux_row + n0 + c_begin * 32);
        const bool got = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag);
        if (!__all_sync(0xffffffffu, got)) {  // warp-uniform exit: the TMEM loads below need the whole warp
          if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
          break;
        }
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
        const int row0 = w.m0 + quarter * 32;
        int gpos = 0, gcol0 = 0;
        bool released = false;
        uint32_t r[32];
        if (n0 + c_begin * 32 < p.n) tmem_ld_32x32b_x32(taddr + c_begin * 32, r);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.n) break;  // warp-uniform
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          const bool last_chunk = (c + 1 == c_end) || (col0 + 32 >= p.n);
          if (!last_chunk) {
            tmem_ld_32x32b_x32(taddr + (c + 1) * 32, r);  // runs under this chunk's arithmetic
            if (dgelu && row_ok) prefetch_l1(aux_row + col0 + 32);
          } else {
            // everything this warp needs from the accumulator is in registers: the MMA warp may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
            released = true;
          }
          if (gpos == 0) {
            // the staging tiles are free once the previous group's stores have read them (long ago, as a rule)
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
            gcol0 = col0;
          }
          if (p.alpha != 1.0f) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= p.alpha;
          }
          if (p.bias != nullptr) {
            const float4* b4 = reinterpret_cast<const float4*>(strip + (c - c_begin) * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 b = b4[i];  // same address in every lane: one broadcast read
              v[4 * i + 0] += b.x;
              v[4 * i + 1] += b.y;
              v[4 * i + 2] += b.z;
              v[4 * i + 3] += b.w;
            }
          }
          uint8_t* st_out = st_base + gpos * per * 2048;
          if (dgelu && row_ok) {
            const int valid = min(32, p.n - col0);
            float a[32];
            load_row32<__nv_bfloat16>(aux_row + col0, (valid == 32) && ((p.ld_aux & 7) == 0), valid, a);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh_f(a[j]);
          }
          if (p.aux_out != nullptr) stage_row32_bf16(st_out + 2048, lane, v);
          if (p.act == NX_ACT_GELU) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = gelu_tanh_f(v[j]);
          }
          stage_row32_bf16(st_out, lane, v);
          if (++gpos == group || last_chunk) {
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
            __syncwarp();
            if (lane == 0 && row0 < p.m) {
              for (int g = 0; g < gpos; ++g) {
                const uint8_t* sg = st_base + g * per * 2048;
                // a tiled store never starts at a negative or out-of-range coordinate, and x stays 16-byte aligned
                if (!NX_INDEX_OK(gcol0 + 32 * g >= 0 && gcol0 + 32 * g < p.n && ((gcol0 + 32 * g) & 7) == 0 && row0 >= 0,
                                 p.status))
                  continue;
                if (p.aux_out != nullptr) tma_store_3d(&tmap_aux, sg + 2048, gcol0 + 32 * g, row0, w.batch);
                tma_store_3d(&tmap_out, sg, gcol0 + 32 * g, row0, w.batch);
              }
              tma_store_commit();
            }
            gpos = 0;
          }
        }
        if (!released) {  // no column of this warp's half lies inside the matrix
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
        }
        if (p.rs_ranks > 1 && lane == 0) {
          // reduce-scatter form: this warp's part of the tile is in global memory -> count it on the tile's row block
          tma_store_wait_all();
          __threadfence();
          atomicAdd(p.rs_done + (w.m0 - m_off) / (2 * kBM), 1);
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (lane == 0) tma_store_wait_all();  // the staging tiles die with the CTA
    } else {
    NX_PROF(long long e_busy = 0; long long e_ld = 0; long long e_slot = 0; long long e_tiles = 0;
            long long e_bias = 0; long long e_stage = 0; long long e_fence = 0; long long e_issue = 0;)
    for (int u = unit_first; u < p.num_units; u += unit_step) {
      Unit w = decode_unit<kTileM>(p, u);
      w.m0 += m_off;
      const int n0 = w.n0 * BN;
      const int row = w.m0 + quarter * 32 + lane;
      const bool row_ok = row < p.m;
      const int c_begin = half * (BN / 64), c_end = (half + 1) * (BN / 64);
      // While the tile's MMAs still run: pull what the epilogue will read (this warp's bias columns, the first
      // chunk of this lane's aux_in / residual row) into L1, so that the loads below do not wait on L2.
      auto prefetch_row_inputs = [&](int col) {
        if (!row_ok || col >= p.n) return;
        if (p.act == NX_ACT_DGELU && p.aux_in != nullptr)
          prefetch_l1(reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + static_cast<int64_t>(row) * p.ld_aux + col);
        if (p.residual != nullptr)
          prefetch_l1(reinterpret_cast<const uint8_t*>(p.residual) +
                      (static_cast<int64_t>(row) * p.ld_res + col) * (p.res_dtype == NX_F32 ? 4 : 2));
      };
      if (p.bias != nullptr && lane < 4) {
        const int eb = p.bias_dtype == NX_F32 ? 4 : 2;
        const int col = n0 + c_begin * 32 + lane * (128 / eb);
        if (col < p.n) prefetch_l1(reinterpret_cast<const uint8_t*>(p.bias) + static_cast<int64_t>(col) * eb);
      }
      prefetch_row_inputs(n0 + c_begin * 32);
      const bool got = mbar_wait_bounded(&tfull_bar[acc], acc_phase, abort_flag);
      if (!__all_sync(0xffffffffu, got)) {  // warp-uniform exit: the TMEM loads below need the whole warp
        if (lane == 0) atomicCAS(p.status, 0, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      NX_PROF(const long long e0 = clock64();)
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      // Tiled stores: `per` staging tiles per chunk (out, aux_out); `group` chunks share one proxy fence and one
      // committed store group; the ring holds kStoreSlots / (per * group) groups.
      const int per = p.aux_out != nullptr ? 2 : 1;
      const int group = (C::kStoreSlots / per >= 4) ? 2 : 1;
      int gpos = 0, gcol0 = 0;
      bool released = false;  // accumulator handed back to the MMA warp
      uint32_t r[32];
      if (n0 + c_begin * 32 < p.n) tmem_ld_32x32b_x32(taddr + c_begin * 32, r);
#pragma unroll 1
      for (int c = c_begin; c < c_end; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;  // warp-uniform
        NX_PROF(const long long e1 = clock64();)
        tmem_ld_wait();
        NX_PROF(e_ld += clock64() - e1;)
        float v[32];
        if (p.alpha != 1.0f) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        }
        const bool last_chunk = (c + 1 == c_end) || (col0 + 32 >= p.n);
        if (!last_chunk) {
          // the next chunk's TMEM read and row inputs run under this chunk's arithmetic and stores
          tmem_ld_32x32b_x32(taddr + (c + 1) * 32, r);
          prefetch_row_inputs(col0 + 32);
        } else {
          // everything this warp needs from the accumulator is in registers: the MMA warp may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
            else mbar_arrive(&tempty_bar[acc]);
          }
          released = true;
        }
        uint8_t* const st_base = store_base + (warp - 2) * (C::kStoreSlots * 2048);
        uint8_t* st_out = st_base;
        if (p.tma_store) {
          // A staging tile may be rewritten once the store group that last used it has read it.  Every lane stays
          // in the loop (rows past M carry garbage that the tiled store clips).
          if (gpos == 0) {
            NX_PROF(const long long e2 = clock64();)
            if (lane == 0) {
              if (C::kStoreSlots / (per * group) >= 2) tma_store_wait_read<1>();
              else tma_store_wait_read<0>();
            }
            __syncwarp();
            NX_PROF(e_slot += clock64() - e2;)
            gcol0 = col0;
          }
          st_out += (ring + gpos * per) * 2048;  // the ring runs on across tiles, in step with the committed groups
        } else if (!row_ok) {
          continue;
        }
        const int valid = min(32, p.n - col0);
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
          if (dist.out_scatter == NX_SCATTER_SLOTS_BF16) {
            // GEMM -> reduce-scatter, slot form: this rank's partial tile goes, as BF16, into slot `rank` of the
            // buffer of the rank that owns these rows; the owner sums the slots in rank order afterwards
            const int owner = row / dist.out_rows;
            __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(dist.out[owner]) +
                                (static_cast<int64_t>(dist.rank) * dist.out_rows + (row - owner * dist.out_rows)) * p.ldo + col0;
            store_row32_bf16(op, (valid == 32) && ((p.ldo & 7) == 0), valid, v);
            continue;
          }
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
        NX_PROF(const long long e3 = clock64();)
        if (p.bias != nullptr) {
          float b[32];
          const bool vec = (valid == 32) && ((col0 & 7) == 0);
          load_any32(p.bias, p.bias_dtype, col0, vec, valid, b);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += b[j];
        }
        NX_PROF(e_bias += clock64() - e3;)
        const int64_t aux_off = static_cast<int64_t>(row) * p.ld_aux + col0;
        const bool aux_vec = (valid == 32) && ((p.ld_aux & 7) == 0);
        if (p.act == NX_ACT_DGELU && p.aux_in != nullptr && row_ok) {
          float a[32];
          load_row32<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(p.aux_in) + aux_off, aux_vec, valid, a);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= dgelu_tanh_f(a[j]);
        }
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
          NX_PROF(const long long e4 = clock64();)
          stage_row32_bf16(st_out, lane, v);
          NX_PROF(const long long e5 = clock64(); e_stage += e5 - e4;)
          if (++gpos == group || last_chunk) {
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA engine
            __syncwarp();
            NX_PROF(const long long e6 = clock64(); e_fence += e6 - e5;)
            const int row0 = w.m0 + quarter * 32;
            if (lane == 0 && row0 < p.m) {
              for (int g = 0; g < gpos; ++g) {
                const uint8_t* sg = st_base + (ring + g * per) * 2048;
                if (p.aux_out != nullptr) tma_store_3d(&tmap_aux, sg + 2048, gcol0 + 32 * g, row0, w.batch);
                tma_store_3d(&tmap_out, sg, gcol0 + 32 * g, row0, w.batch);
              }
              tma_store_commit();
            }
            ring = (ring + per * group) % C::kStoreSlots;
            gpos = 0;
            NX_PROF(e_issue += clock64() - e6;)
          }
        } else if (!NX_INDEX_OK(row < p.m && col0 < p.n && valid > 0, p.status)) {
          continue;
        } else if (p.out_dtype == NX_F32) {
          store_row32_f32(reinterpret_cast<float*>(p.out) + out_off, out_vec, valid, v);
        } else {
          store_row32_bf16(reinterpret_cast<__nv_bfloat16*>(p.out) + out_off, out_vec, valid, v);
        }
      }
      NX_PROF(e_busy += clock64() - e0; ++e_tiles;)
      if (!released) {  // no column of this warp's half lies inside the matrix
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[acc]), 0));
          else mbar_arrive(&tempty_bar[acc]);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    NX_PROF(if (warp == 2 && lane == 0 && blockIdx.x < kProfRows) {
      long long* o = g_epi_prof + blockIdx.x * 8;
      o[0] = e_busy; o[1] = e_ld; o[2] = e_slot; o[3] = e_tiles;
      o[4] = e_bias; o[5] = e_stage; o[6] = e_fence; o[7] = e_issue;
    })
    if (p.tma_store && lane == 0) tma_store_wait_all();  // the staging tiles die with the CTA
    }  // generic epilogue
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
  if constexpr (PAIR) cluster_sync_all();  // neither CTA frees TMEM or leaves while the other may still use the pair
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, C::kTmemCols);
    else tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// CTA-pair variant: clusters of two CTAs, one 256 x 256 tile per cluster.  `max_ctas` caps the grid.
template <bool A_MN, bool B_MN, bool FAST>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const DevParams& p, uint32_t in_fmt, int max_ctas,
                cudaStream_t stream, const CUtensorMap* t_out, const CUtensorMap* t_aux) {
  using C = Cfg<256, true>;
  static int max_clusters = 0;  // 0: not asked yet, < 0: clusters of two cannot be placed
  auto kern = gemm_kernel<256, A_MN, B_MN, false, true, FAST>;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // prologue may overlap the previous kernel's tail
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  static const bool no_pdl = std::getenv("NX_NO_PDL") != nullptr;  // measurement switch
  cfg.numAttrs = no_pdl ? 1 : 2;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) return -2;
    cfg.gridDim = dim3(2 * 74);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) {
      (void)cudaGetLastError();
      max_clusters = -1;
    } else {
      max_clusters = n;
    }
  }
  if (max_clusters < 0) return -3;
  int clusters = std::min(p.num_units, max_clusters);
  if (max_ctas > 1) clusters = std::min(clusters, max_ctas / 2);
  if (p.ag_ranks > 1 || p.rs_ranks > 1) {
    // copier clusters share the device with the GEMM clusters: all of them must be resident at once
    const int copier_clusters = (p.ag_ranks > 1 ? p.ag_copiers : p.rs_copiers) / 2;
    if (copier_clusters < 1 || copier_clusters >= max_clusters) return -1;
    clusters = std::min(clusters, max_clusters - copier_clusters) + copier_clusters;
  }
  cfg.gridDim = dim3(2 * clusters);
  const uint32_t idesc = make_idesc(in_fmt, in_fmt, A_MN, B_MN, 2 * kBM, 256);
  DistParam<false> dist{};
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, p, idesc, dist, t_out ? *t_out : ta, t_aux ? *t_aux : ta) != cudaSuccess) {
    (void)cudaGetLastError();
    return -2;
  }
  return 0;
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

// Sums the K slices of a split GEMM (fixed order) and applies what the GEMM's own epilogue would have: bias,
// activation, and the add into the existing output.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, void* out, int out_dtype, int64_t ldo, int m,
                                     int n, int split_k, int accumulate, const void* bias, int bias_dtype, int act) {
  const int64_t total = static_cast<int64_t>(m) * n;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float s = 0.0f;
    for (int k = 0; k < split_k; ++k) s += ws[static_cast<int64_t>(k) * total + i];
    const int r = static_cast<int>(i / n), c = static_cast<int>(i % n);
    if (bias != nullptr)
      s += bias_dtype == NX_F32 ? reinterpret_cast<const float*>(bias)[c]
                                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[c]);
    if (act == NX_ACT_GELU) s = gelu_tanh_f(s);
    else if (act == NX_ACT_RELU) s = fmaxf(s, 0.0f);
    else if (act == NX_ACT_SILU) s = silu_f(s);
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
  return nx_splitk_reduce_epilogue(workspace, out, out_dtype, ldo, m, n, split_k, accumulate, nullptr, NX_F32, NX_ACT_NONE,
                                   stream);
}

extern "C" int nx_splitk_reduce_epilogue(const float* workspace, void* out, int out_dtype, int64_t ldo, int m, int n,
                                         int split_k, int accumulate, const void* bias, int bias_dtype, int act,
                                         nx_stream_t stream) {
  const int64_t total = static_cast<int64_t>(m) * n;
  if (total == 0) return 0;
  if (act != NX_ACT_NONE && act != NX_ACT_GELU && act != NX_ACT_RELU && act != NX_ACT_SILU) return -1;
  int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 148 * 8));
  splitk_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(workspace, out, out_dtype, ldo, m, n,
                                                                              split_k, accumulate, bias, bias_dtype, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

namespace {
int gemm_impl(const NxGemmArgs* a, const NxGemmAg* ag, nx_stream_t stream_, const NxGemmRs* rs = nullptr);
}
extern "C" int nx_gemm(const NxGemmArgs* a, nx_stream_t stream_) { return gemm_impl(a, nullptr, stream_); }

// GEMM fused with the reduce-scatter of its output; see nx_api_comm.h.
extern "C" int nx_gemm_rs(const NxGemmArgs* a, const NxGemmRs* rs, nx_stream_t stream_) {
  if (a == nullptr || rs == nullptr) return -1;
  const int n = rs->n_ranks;
  if (n < 2 || n > NX_MAX_PEERS || rs->rank < 0 || rs->rank >= n || rs->done == nullptr) return -1;
  if (a->in_dtype != NX_BF16 || a->out_dtype != NX_BF16 || a->batch != 1 || a->split_k > 1 || a->accumulate) return -1;
  if (a->bias != nullptr || a->residual != nullptr || a->aux_in != nullptr || a->aux_out != nullptr || a->act != NX_ACT_NONE)
    return -1;
  if (a->m % n || (a->m / n) % (2 * kBM) || a->n < 256 || (a->n & 7) || (a->ldo & 7)) return -1;
  const int c = rs->copier_ctas;
  if (c < 2 || (c & 1)) return -1;  // whole clusters of two
  for (int q = 0; q < n; ++q)
    if (rs->slots[q] == nullptr || (reinterpret_cast<uintptr_t>(rs->slots[q]) & 15)) return -1;
  return gemm_impl(a, nullptr, stream_, rs);
}

// All-gather fused into the GEMM; see nx_api_comm.h.
extern "C" int nx_gemm_ag(const NxGemmArgs* a, const NxGemmAg* ag, nx_stream_t stream_) {
  if (a == nullptr || ag == nullptr) return -1;
  const int n = ag->n_ranks;
  if (n < 2 || n > NX_MAX_PEERS || ag->rank < 0 || ag->rank >= n || ag->counter == nullptr) return -1;
  if (a->in_dtype != NX_BF16 || a->a_mn_major || a->batch != 1 || a->split_k > 1) return -1;
  if (a->m % n || (a->m / n) % (2 * kBM) || a->n < 256 || (a->k & 7)) return -1;
  if (ag->copier_ctas < 2 || (ag->copier_ctas & 1)) return -1;
  for (int q = 0; q < n; ++q)
    if (ag->gather[q] == nullptr || ag->flags[q] == nullptr || (reinterpret_cast<uintptr_t>(ag->gather[q]) & 15)) return -1;
  if (a->a != ag->gather[ag->rank]) return -1;  // A is this rank's gather buffer
  return gemm_impl(a, ag, stream_);
}

namespace {
int gemm_impl(const NxGemmArgs* a, const NxGemmAg* ag, nx_stream_t stream_, const NxGemmRs* rs) {
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

  // Two-CTA tiles (256 x 256 over a cluster of two) whenever the problem has at least one such tile of BF16/FP16.
  static const bool single_only = std::getenv("NX_GEMM_SINGLE_CTA") != nullptr;  // measurement switch
  static bool pair_ok = true;  // cleared when the device cannot place clusters of two
  const bool pair = bn == 256 && !fp8 && a->m >= 2 * kBM && pair_ok && (!single_only || ag != nullptr || rs != nullptr) &&
                    (a->max_ctas <= 0 || a->max_ctas >= 2);
  if ((ag != nullptr || rs != nullptr) && !pair) return -3;  // the fused forms run on the CTA-pair kernel only
  const int tile_m = pair ? 2 * kBM : kBM;

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
  p.tiles_m = (a->m + tile_m - 1) / tile_m;
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
  // Units that run at the same time should share the larger operand's tile: walk along N when B is the smaller
  // matrix (its whole K-panel set stays in L2 while each A tile is fetched from DRAM once), else along M.
  static const char* order_env = std::getenv("NX_GEMM_ORDER");  // measurement switch: "m" or "n"
  p.n_fastest = order_env ? (order_env[0] == 'n') : (a->n < a->m);
  if (ag != nullptr) {
    p.n_fastest = 1;  // all column tiles of a row block run together: rows are consumed in their order of arrival
    p.ag_ranks = ag->n_ranks;
    p.ag_rank = ag->rank;
    p.ag_rows = a->m / ag->n_ranks;
    p.rot_rows = ag->rank * p.ag_rows;
    p.ag_copiers = ag->copier_ctas;
    p.ag_ld_bytes = a->lda * 2;
    p.ag_row_bytes = a->k * 2;
    p.ag_counter = ag->counter;
    for (int q = 0; q < ag->n_ranks; ++q) {
      p.ag_gather[q] = ag->gather[q];
      p.ag_flags[q] = ag->flags[q];
    }
  }

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
    rc = nx::make_tensor_map_3d(&tb, dt, eb, a->b, a->k, a->n, a->batch, a->ldb, sb, bk, pair ? bn / 2 : bn);
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

  if (pair) {
    const CUtensorMap* po = p.tma_store ? &to : nullptr;
    const CUtensorMap* px = (p.tma_store && a->aux_out) ? &tx : nullptr;
    // the lean epilogue covers what the training step's BF16-output GEMMs ask for
    static const bool generic_only = std::getenv("NX_GEMM_GENERIC_EPILOGUE") != nullptr;  // measurement switch
    if (rs != nullptr) {
      if (!p.tma_store) return -1;  // the reduce-scatter form counts tiles in the lean epilogue (tiled BF16 stores)
      p.n_fastest = 1;              // row blocks finish one after the other, in ring order
      p.rs_ranks = rs->n_ranks;
      p.rs_rank = rs->rank;
      p.rs_rows = a->m / rs->n_ranks;
      p.rot_rows = ((rs->rank + 1) % rs->n_ranks) * p.rs_rows;  // the rows this rank keeps come last
      p.rs_copiers = rs->copier_ctas;
      p.rs_expected = 16 * p.tiles_n;
      p.rs_copy_own = rs->copy_own;
      p.rs_done = rs->done;
      for (int q = 0; q < rs->n_ranks; ++q) p.rs_slots[q] = rs->slots[q];
    }
    const bool fast = (rs != nullptr || !generic_only) && p.tma_store && a->residual == nullptr && a->scale_a == nullptr &&
                      a->scale_b == nullptr && a->amax_out == nullptr && (reinterpret_cast<uintptr_t>(a->bias) & 15) == 0 &&
                      (a->aux_in == nullptr || (reinterpret_cast<uintptr_t>(a->aux_in) & 15) == 0) &&
                      (a->act == NX_ACT_NONE || a->act == NX_ACT_GELU || (a->act == NX_ACT_DGELU && a->aux_in != nullptr));
#define NX_PAIR(AM_, BM_) \
  rc = fast ? launch_pair<AM_, BM_, true>(ta, tb, p, fmt, sms, stream, po, px) \
            : launch_pair<AM_, BM_, false>(ta, tb, p, fmt, sms, stream, po, px)
    if (!a->a_mn_major && !a->b_mn_major) NX_PAIR(false, false);
    else if (!a->a_mn_major && a->b_mn_major) NX_PAIR(false, true);
    else if (a->a_mn_major && !a->b_mn_major) NX_PAIR(true, false);
    else NX_PAIR(true, true);
#undef NX_PAIR
    if (rc != -3) return rc;
    // no room for clusters of two on this device: rebuild the launch for single-CTA tiles
    pair_ok = false;
    return gemm_impl(a, ag, stream_, rs);
  }

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
}  // namespace

// BF16; batch 1; no split-K.  Rows (or K rows) per rank must be multiples of the tile size.
extern "C" int nx_gemm_dist(const NxGemmArgs* a, const NxGemmDist* d, nx_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || d == nullptr || a->m <= 0 || a->n <= 0 || a->k <= 0 || a->status == nullptr) return -1;
  if (a->batch != 1 || a->in_dtype != NX_BF16) return -1;
  const int n = d->n_ranks;
  if (n < 1 || n > NX_MAX_PEERS || d->rank < 0 || d->rank >= n || (a->lda & 7) || (a->ldb & 7)) return -1;
  const bool a_mn = a->a_mn_major != 0, b_mn = a->b_mn_major != 0;
  // a row-sharded operand is K-major, a K-sharded one MN-major
  if (d->a_sharded == NX_DIST_ROWS && (a_mn || a->m % n || (a->m / n) % kBM)) return -1;
  if (d->a_sharded == NX_DIST_K && (!a_mn || a->k % n || (a->k / n) % kBK)) return -1;
  if (d->b_sharded == NX_DIST_K && (!b_mn || a->k % n || (a->k / n) % kBK)) return -1;
  if (d->a_sharded < 0 || d->a_sharded > 2 || d->b_sharded < 0 || d->b_sharded > 2 || d->out_scatter < 0 ||
      d->out_scatter > 2)
    return -1;
  int bn = (a->n >= 256) ? 256 : 128;
  if (d->b_sharded == NX_DIST_ROWS) {
    if (b_mn || a->n % n) return -1;
    const int per = a->n / n;
    if (per % 256 == 0) bn = 256;
    else if (per % 128 == 0) bn = 128;
    else return -1;
  }
  if (d->out_scatter && (a->m % n || (a->m / n) % kBM)) return -1;
  if (d->out_scatter == NX_SCATTER_ADD_F32 && a->out_dtype != NX_F32) return -1;
  if (d->out_scatter == NX_SCATTER_SLOTS_BF16 && a->out_dtype != NX_BF16) return -1;
  if (a_mn && !b_mn) return -1;  // (MN, K) is not instantiated for the distributed kernel

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
  // units that run together share the smaller operand through L2 (same rule as nx_gemm)
  p.n_fastest = a->n < a->m;

  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  DistParam<true> dist{};
  dist.a_sharded = d->a_sharded;
  dist.b_sharded = d->b_sharded;
  dist.out_scatter = d->out_scatter;
  dist.rank = d->rank;
  dist.a_rows = d->a_sharded == NX_DIST_ROWS ? a->m / n : a->m;
  dist.b_rows = d->b_sharded == NX_DIST_ROWS ? a->n / n : a->n;
  dist.out_rows = d->out_scatter ? a->m / n : a->m;
  dist.k_rows = (d->a_sharded == NX_DIST_K || d->b_sharded == NX_DIST_K) ? a->k / n : a->k;
  CUtensorMap ta, tb;
  int rc;
  // K-major operand: [rows][K] with a {64, tile rows} box; MN-major operand: [K][rows] with a {64, 64} box
  auto map_a = [&](CUtensorMap* t, const void* base, int rows, int krows) {
    return a_mn ? nx::make_tensor_map_3d(t, dt, 2, base, rows, krows, 1, a->lda, 0, 64, kBK)
                : nx::make_tensor_map_3d(t, dt, 2, base, krows, rows, 1, a->lda, 0, kBK, kBM);
  };
  auto map_b = [&](CUtensorMap* t, const void* base, int rows, int krows) {
    return b_mn ? nx::make_tensor_map_3d(t, dt, 2, base, rows, krows, 1, a->ldb, 0, 64, kBK)
                : nx::make_tensor_map_3d(t, dt, 2, base, krows, rows, 1, a->ldb, 0, kBK, bn);
  };
  const int a_map_rows = d->a_sharded == NX_DIST_ROWS ? dist.a_rows : a->m;
  const int b_map_rows = d->b_sharded == NX_DIST_ROWS ? dist.b_rows : a->n;
  const int a_map_k = d->a_sharded == NX_DIST_K ? dist.k_rows : a->k;
  const int b_map_k = d->b_sharded == NX_DIST_K ? dist.k_rows : a->k;
  for (int q = 0; q < n; ++q) {
    if (d->a_sharded) {
      if (d->a_ptrs[q] == nullptr || (reinterpret_cast<uintptr_t>(d->a_ptrs[q]) & 15)) return -1;
      if ((rc = map_a(&dist.a[q], d->a_ptrs[q], a_map_rows, a_map_k))) return rc;
    }
    if (d->b_sharded) {
      if (d->b_ptrs[q] == nullptr || (reinterpret_cast<uintptr_t>(d->b_ptrs[q]) & 15)) return -1;
      if ((rc = map_b(&dist.b[q], d->b_ptrs[q], b_map_rows, b_map_k))) return rc;
    }
    if (d->out_scatter && d->out_ptrs[q] == nullptr) return -1;
    dist.out[q] = static_cast<float*>(d->out_ptrs[q]);
  }
  const void* a0 = d->a_sharded ? d->a_ptrs[d->rank] : a->a;
  const void* b0 = d->b_sharded ? d->b_ptrs[d->rank] : a->b;
  if (a0 == nullptr || b0 == nullptr) return -1;
  if ((rc = map_a(&ta, a0, a_map_rows, a_map_k))) return rc;
  if ((rc = map_b(&tb, b0, b_map_rows, b_map_k))) return rc;
  int sms = nx_sm_count();
  if (sms <= 0) return -2;
  const int grid = p.num_units < sms ? p.num_units : sms;
#define NX_DIST_LAUNCH(BN_, AM_, BM_) launch_variant<BN_, AM_, BM_, true>(ta, tb, p, kFmtBF16, grid, stream, dist)
  if (bn == 256) {
    if (!a_mn && !b_mn) return NX_DIST_LAUNCH(256, false, false);
    if (!a_mn && b_mn) return NX_DIST_LAUNCH(256, false, true);
    return NX_DIST_LAUNCH(256, true, true);
  }
  if (!a_mn && !b_mn) return NX_DIST_LAUNCH(128, false, false);
  if (!a_mn && b_mn) return NX_DIST_LAUNCH(128, false, true);
  return NX_DIST_LAUNCH(128, true, true);
#undef NX_DIST_LAUNCH
}

#ifdef NX_PROFILE_MMA
extern "C" int nx_gemm_prof_read(long long* out) {
  return cudaMemcpyFromSymbol(out, g_mma_prof, sizeof(long long) * kProfRows * 8) == cudaSuccess ? 0 : -1;
}
extern "C" int nx_gemm_prof_read_epilogue(long long* out) {
  return cudaMemcpyFromSymbol(out, g_epi_prof, sizeof(long long) * kProfRows * 8) == cudaSuccess ? 0 : -1;
}
#endif
