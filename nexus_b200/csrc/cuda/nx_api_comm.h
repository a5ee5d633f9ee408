// C ABI of the kernels that combine computation with NVLink communication over peer-mapped memory.
// A peer table holds, for every rank of the group, the device pointer (as mapped in THIS process) of
// that rank's copy of a symmetric buffer.  All waits inside these kernels are bounded (2 s); a wait
// that runs out writes nx::kStatusTimeoutPeer into the status word.
#pragma once
#include "nx_api_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define NX_MAX_PEERS 8

typedef struct NxPeerTable {
  void* ptr[NX_MAX_PEERS];
} NxPeerTable;

// flags: per rank an int[n] array (zero-initialised).  `counter`: this rank's barrier generation, one int in
// device memory, zero-initialised; every barrier-bearing call (this one, nx_comm_norm_exchange,
// nx_vocab_ce_exchange) waits for generation *counter + 1 and then stores it, so all ranks must issue the same
// sequence of such calls.  Because the generation is read on the device, these kernels stay correct when a
// captured CUDA graph replays them.
int nx_comm_barrier(const NxPeerTable* flags, int rank, int n, int* counter, int* status, nx_stream_t stream);

// out[i] = scale * sum_p grads[p][shard_off + i] (p = 0..n-1 in order), i < count; partial[] receives
// per-block FP64 square sums (nx_comm_reduce_partials(count) entries).  shard_off % 4 == 0.
int64_t nx_comm_reduce_partials(int64_t count);
int nx_comm_reduce_shard(const NxPeerTable* grads, int n, int64_t shard_off, int64_t count, float scale, float* out,
                         double* partial, nx_stream_t stream);
// slots: per rank a double[n] array.  Publishes this rank's square sum to every rank, waits for all,
// then fills grad_norm / clip_coef / found_inf / step / bias corrections of `state`.
int nx_comm_norm_exchange(const double* partial, int nparts, const NxPeerTable* slots, const NxPeerTable* flags,
                          int rank, int n, int* counter, NxOptState* state, int* status, nx_stream_t stream);
// AdamW on shard-local FP32 state; chunks carry GLOBAL offsets inside [shard_off, shard_off + shard);
// the BF16 weights are written into every rank's full shadow buffer (the all-gather).  fp32_tails
// (optional): per rank an FP32 buffer holding the parameters at global offsets >= tail_off, which
// receive the FP32 values too (norm scales and biases that the model reads in full precision).
int nx_comm_adamw_allgather(float* master, const float* grad, float* m, float* v, const NxPeerTable* shadows,
                            const NxPeerTable* fp32_tails, int64_t tail_off, int n, int64_t shard_off,
                            const NxAdamChunk* chunks, int nchunks, const NxOptState* state, nx_stream_t stream);

// All-reduce with the cast fused in.  The caller owns [shard_off, shard_off + count) (multiples of 8
// elements): it sums that range over the n_in input buffers (FP32 or BF16, rank order, FP32 math),
// scales, and stores into the first n_out output buffers (FP32 or BF16).  Bracket with nx_comm_barrier.
int nx_comm_allreduce_shard(const NxPeerTable* in, int in_dtype, int n_in, const NxPeerTable* out, int out_dtype,
                            int n_out, int64_t shard_off, int64_t count, float scale, nx_stream_t stream);

// The two communicating kernels of the sharded optimizer through NVSwitch (`*_mc`: multicast addresses of the
// symmetric gradient, BF16 shadow and FP32 tail buffers).  Same arguments and results as nx_comm_reduce_shard /
// nx_comm_adamw_allgather; the reduce reads each element once from the switch (`multimem.ld_reduce`), the update
// writes each result once for all ranks (`multimem.st`).
int nx_comm_reduce_shard_multimem(void* grads_mc, int64_t shard_off, int64_t count, float scale, float* out,
                                  double* partial, nx_stream_t stream);
// (`shadows`: the peer table of the BF16 shadow, for single values at ragged chunk ends: a multicast store is at least
// 32 bits wide.)
int nx_comm_adamw_allgather_multimem(float* master, const float* grad, float* m, float* v, void* shadow_mc, void* tail_mc,
                                     const NxPeerTable* shadows, int n, int64_t tail_off, int64_t shard_off,
                                     const NxAdamChunk* chunks, int nchunks, const NxOptState* state, nx_stream_t stream);

// All-gather by peer loads: out[q * shard_bytes + ...] = shards[q][0 .. shard_bytes) for q < n (shard_bytes a multiple of
// 16; `out` local).  Bracket with nx_comm_barrier: the shards must be written before, and stay untouched until every
// rank has read them.
int nx_comm_gather_shards(const NxPeerTable* shards, int n, int64_t shard_bytes, void* out, nx_stream_t stream);

// The same all-reduce done by NVSwitch (NVLS): `multicast_ptr` is the multicast address of a symmetric buffer (one
// address for the same offset in every rank's copy; from the symmetric-memory rendezvous, null when the fabric has no
// multicast).  The caller owns [shard_off, shard_off + count) elements (FP32: multiples of 4, BF16: of 8): the switch
// sums that range over all ranks (FP32 accumulation), the result times `scale` is stored into every rank's copy, in
// place.  Bracket with nx_comm_barrier like the peer-load form.
int nx_comm_allreduce_multimem(void* multicast_ptr, int dtype, int64_t shard_off, int64_t count, float scale,
                               nx_stream_t stream);

// Ulysses all-to-all by peer stores (BF16, D % 8 == 0, H % n == 0).  mode 0: x [B, Tl, H, D] ->
// out[q] [B, n*Tl, H/n, D] (heads scattered, sequence gathered); mode 1: the inverse.  Bracket with barriers.
int nx_comm_a2a_heads(const void* x, const NxPeerTable* out, int B, int Tl, int H, int D, int rank, int n, int mode,
                      nx_stream_t stream);

// Expert parallelism.  bufs[q]: rank q's [local_experts, capacity, d] BF16 buffer.  Row r of the
// assignment list goes to expert expert_of[r], slot slot_of[r] (negative: dropped, skipped); its source
// row is x[token_of[r]] (token_of null: x[r / rows_per_token]); row_scale (optional) multiplies the copy.
int nx_moe_dispatch(const void* x, const int32_t* token_of, const int32_t* expert_of, const int32_t* slot_of,
                    const NxPeerTable* bufs, int rows, int d, int local_experts, int capacity, int src_rank,
                    int n_ranks, const float* row_scale, int rows_per_token, nx_stream_t stream);
int nx_moe_combine(const NxPeerTable* bufs, const int32_t* expert, const int32_t* slot, const float* gate, void* y,
                   int tokens, int top_k, int d, int local_experts, int capacity, nx_stream_t stream);

// dgate[t, j] = dy[t] . expert_output[owner][local expert][slot] with the row read from its owner's buffer.
int nx_moe_gate_grad_peers(const void* dy, const NxPeerTable* bufs, const int32_t* expert, const int32_t* slot,
                           float* dgate, int tokens, int top_k, int d, int local_experts, int capacity,
                           nx_stream_t stream);

// Vocabulary-parallel CE: local_stats [rows][3]; tables[q]: float[n][rows][3]; merged [rows][3].
int nx_vocab_ce_exchange(const float* local_stats, const NxPeerTable* tables, const NxPeerTable* flags, int rank, int n,
                         int rows, int* counter, float* merged, int* status, nx_stream_t stream);

// Distributed GEMM (see nx_gemm): an operand is sharded over the ranks and its tiles are fetched by
// (non-multicast) TMA straight from the owning rank's memory, and/or the output is reduce-scattered from
// inside the epilogue.  BF16 operands; each operand K-major or MN-major as in nx_gemm (a_mn_major / b_mn_major).
//   a_sharded / b_sharded = 1 (NX_DIST_ROWS): the operand is K-major and rank q holds its rows
//       [q*M/n, (q+1)*M/n) (A) or [q*N/n, (q+1)*N/n) (B): all-gather fused into the GEMM.
//   a_sharded / b_sharded = 2 (NX_DIST_K): the operand is MN-major (stored [K][M or N]) and rank q holds the
//       K rows [q*K/n, (q+1)*K/n): the contraction runs over a dimension that is spread over the ranks
//       (weight gradients of a sequence-parallel layer).  K/n must be a multiple of 64.
//   out_scatter = 1 (NX_SCATTER_ADD_F32): rank q owns output rows [q*M/n, (q+1)*M/n); every rank adds its partial
//       tile into the owner's FP32 buffer with vector reductions (order of the additions is not fixed).
//   out_scatter = 2 (NX_SCATTER_SLOTS_BF16): the owner's buffer is BF16 [n][M/n][ldo]; rank r stores its partial
//       tile into slot r, and the owner sums the n slots in rank order afterwards (nx_comm_sum_slots): half the
//       NVLink bytes of the FP32 form and a deterministic result.
#define NX_DIST_ROWS 1
#define NX_DIST_K 2
#define NX_SCATTER_ADD_F32 1
#define NX_SCATTER_SLOTS_BF16 2
typedef struct NxGemmDist {
  const void* a_ptrs[NX_MAX_PEERS];  // per rank: its part of A (used when a_sharded)
  const void* b_ptrs[NX_MAX_PEERS];  // per rank: its part of B (used when b_sharded)
  void* out_ptrs[NX_MAX_PEERS];      // per rank: its output buffer (used when out_scatter)
  int32_t n_ranks, rank;
  int32_t a_sharded, b_sharded, out_scatter;
} NxGemmDist;
int nx_gemm_dist(const NxGemmArgs* args, const NxGemmDist* dist, nx_stream_t stream);

// All-gather fused into ONE tcgen05 GEMM kernel (the CTA-pair kernel of nx_gemm), push form.  Every rank owns a
// peer-mapped gather buffer [M][lda] (BF16) whose row block `rank` it has already filled; args->a must be
// gather[rank].  The last `copier_ctas` CTAs of the grid store this rank's rows into every peer's buffer, 128 rows
// at a time, and raise flags[peer][rank][chunk] to the call's generation (*counter + 1, release at system scope).
// The GEMM CTAs compute the local row block first and then the other ranks' blocks in ring order, each producer
// waiting (bounded: kStatusTimeoutPeer) for the flag of the rows it is about to load.  Each row crosses NVLink once
// and the transfer overlaps the tensor-core work tile by tile; afterwards every rank also holds the complete
// gathered A for later use (e.g. the weight-gradient GEMM).  The caller bumps *counter on every rank after the
// call (nx_comm_bump) and orders re-use of the gather buffers with nx_comm_barrier.
// Requirements: BF16, K-major A, M / n_ranks a multiple of 256, N >= 256, copier_ctas even and >= 2.
typedef struct NxGemmAg {
  void* gather[NX_MAX_PEERS];
  int* flags[NX_MAX_PEERS];   // per rank: int[n_ranks][M / n_ranks / 128], zero-initialised once
  const int* counter;         // this rank's generation counter of the flag array (device memory)
  int32_t n_ranks, rank, copier_ctas;
} NxGemmAg;
int nx_gemm_ag(const NxGemmArgs* args, const NxGemmAg* ag, nx_stream_t stream);
// GEMM fused with the reduce-scatter of its output in ONE kernel (the CTA-pair kernel of nx_gemm), push form.
// args->out is a LOCAL BF16 [M][ldo] buffer that receives this rank's partial sums through the kernel's normal tiled
// stores; every epilogue warp then counts its finished tile on done[row block].  The last `copier_ctas` CTAs of the
// grid wait for a 256-row block to be complete and store it into slot `rank` of the buffer slots[owner]
// (BF16 [n_ranks][M / n_ranks][ldo]) of the rank that owns those rows, over NVLink, while the tensor-core CTAs are
// already on the next blocks; work starts with the next rank's rows and ends with this rank's own.  Afterwards
// (nx_comm_barrier, then nx_comm_sum_slots) each owner adds the n slots in rank order: deterministic, BF16 on the wire.
// `done`: int[M / 256] in local device memory, zeroed by the caller before every call.
// Requirements: BF16 in and out, no epilogue extras, M / n_ranks a multiple of 256, N >= 256, copier_ctas a power
// of two in [2, 256].
// copy_own = 0: the row block this rank owns is not copied into its own slot; it stays in args->out, and the caller
// hands nx_comm_sum_slots that block as the rank's own contribution (own_rows).
typedef struct NxGemmRs {
  void* slots[NX_MAX_PEERS];
  int* done;
  int32_t n_ranks, rank, copier_ctas, copy_own;
} NxGemmRs;
int nx_gemm_rs(const NxGemmArgs* args, const NxGemmRs* rs, nx_stream_t stream);
// *counter += 1 (one thread), stream-ordered after the kernels that read it.
int nx_comm_bump(int* counter, nx_stream_t stream);

// out[r][c] = (residual ? residual[r][c] : 0) + sum_{q < n} slots[q][r][c] (q in order, FP32 accumulation):
// the owner's half of the slot form of GEMM -> reduce-scatter.  slots: BF16 [n][rows][ld_slots]; residual / out:
// FP32 or BF16 with row strides ld_res / ld_out; out_lp (optional): a BF16 copy of the result, row stride ld_lp.
// own_rows (optional): BF16 [rows][ld_slots] that stands in for slot `own_rank` (that slot is then not read).
int nx_comm_sum_slots(const void* slots, int n, int rows, int cols, int64_t ld_slots, const void* residual,
                      int res_dtype, int64_t ld_res, void* out, int out_dtype, int64_t ld_out, void* out_lp,
                      int64_t ld_lp, const void* own_rows, int own_rank, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
