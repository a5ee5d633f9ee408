// Kernels of the tensor-parallel (vocabulary-parallel + sequence-parallel) language-model path.
// Parity (behaviour): VocabParallelEmbedding and the vocabulary-parallel loss of the reference's ParallelLm
// (src/dist/parallel_lm.cpp:560-665), which run on CPU ranks with all-reduces there.
#pragma once
#include "nx_api_comm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Embedding lookup when the table is split by vocabulary rows over the ranks: every rank holds rows
// [q*v_per, (q+1)*v_per) of the BF16 table in a peer-mapped buffer.  out[i] = table_of_owner(tokens[i])[tokens[i] - owner*v_per]
// for this rank's `rows` tokens, read straight from the owner's memory (plain peer loads).  out: FP32 [rows][d].
int nx_tp_embed_gather(const int32_t* tokens, const NxPeerTable* tables, int n_ranks, int v_per, int d, float* out,
                       int rows, nx_stream_t stream);
// Gradient of that lookup for this rank's vocabulary rows: for every token i of the WHOLE batch (`total` tokens; row i
// of the activation gradient lives on rank i / rows_per_rank in a peer-mapped BF16 buffer [rows_per_rank][d]) whose id
// falls into [v0, v0 + v_per): dtable[id - v0] += dh[i].  FP32 atomics into the local gradient.
int nx_tp_embed_bwd(const int32_t* tokens_all, int total, const NxPeerTable* dh, int rows_per_rank, int v0, int v_per,
                    int d, float* dtable, nx_stream_t stream);

// Vocabulary-parallel cross-entropy, local part 1: per row (max, sum exp(l - max), logit of the target or 0) over
// this rank's `cols` logits columns [v0, v0 + cols).  targets: global ids, < 0 = ignored row.  stats: [rows][3].
int nx_tp_ce_stats(const void* logits, int64_t ld, int rows, int cols, const int32_t* targets, int v0, float* stats,
                   nx_stream_t stream);
// Local part 2, in place: logits <- (exp(l - lse) - [col == target]) * scale for valid rows, 0 for ignored ones,
// with lse = merged[row][0] + log(merged[row][1]) from nx_vocab_ce_exchange.  `scale` is read from device memory
// (1 / valid rows times the micro-step weight), so a captured step can change it.
int nx_tp_ce_grad(void* logits, int64_t ld, int rows, int cols, const int32_t* targets, int v0, const float* merged,
                  const float* scale, nx_stream_t stream);
// loss_out (+)= weight * sum over valid rows of (lse - target logit) * inv_valid.
int nx_tp_ce_loss(const float* merged, const int32_t* targets, int rows, float inv_valid, float weight, int accumulate,
                  float* loss_out, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
