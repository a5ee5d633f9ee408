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

// Vocabulary-parallel CE: local_stats [rows][3]; tables[q]: float[n][rows][3]; merged [rows][3].
int nx_vocab_ce_exchange(const float* local_stats, const NxPeerTable* tables, const NxPeerTable* flags, int rank, int n,
                         int rows, int* counter, float* merged, int* status, nx_stream_t stream);

// Distributed GEMM (see nx_gemm): operand A and/or B is row-sharded over the ranks and its tiles are
// fetched by (non-multicast) TMA straight from the owning rank's memory; the output can be
// reduce-scattered by adding each tile into the owning rank's FP32 buffer.
typedef struct NxGemmDist {
  const void* a_ptrs[NX_MAX_PEERS];  // when a_sharded: rank q holds rows [q*M/n, (q+1)*M/n) of A (K-major)
  const void* b_ptrs[NX_MAX_PEERS];  // when b_sharded: rank q holds rows [q*N/n, (q+1)*N/n) of B (K-major)
  void* out_ptrs[NX_MAX_PEERS];      // when out_scatter: rank q owns output rows [q*M/n, (q+1)*M/n), FP32
  int32_t n_ranks, rank;
  int32_t a_sharded, b_sharded, out_scatter;
} NxGemmDist;
int nx_gemm_dist(const NxGemmArgs* args, const NxGemmDist* dist, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
