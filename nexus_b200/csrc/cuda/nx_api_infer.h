// C ABI of the inference kernels: paged KV cache, decode attention, skinny GEMM, sampling, RoPE,
// gated activations and weight-only quantisation.  All tensors are BF16 unless stated otherwise.
#pragma once
#include "nx_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// KV cache layout: [num_blocks, block_size, kv_heads, head_dim]; slot = block * block_size + offset.
// kv_kind: 0 BF16, 1 INT8, 2 FP8-E4M3; the 8-bit kinds keep one FP32 scale per (slot, kv head).
// A negative slot skips the token (padding rows of a captured batch).
int nx_kv_append(const void* k, const void* v, int64_t k_row_stride, int64_t v_row_stride, const int32_t* slots,
                 void* k_cache, void* v_cache, float* k_scale, float* v_scale, int tokens, int kv_heads,
                 int head_dim, int kv_kind, nx_stream_t stream);

typedef struct NxPagedArgs {
  const void* q;            // [rows, heads, head_dim]
  int64_t q_row_stride;     // elements
  const void* k_cache;
  const void* v_cache;
  const float* k_scale;     // 8-bit kinds only
  const float* v_scale;
  const int32_t* block_table;  // [num_seqs, max_blocks]
  const int32_t* row_seq;      // [rows] sequence (block-table row) of each query row
  const int32_t* ctx_len;      // [rows] number of cached tokens visible to the row
  void* out;                // [rows, heads, head_dim]
  int64_t o_row_stride;
  float* part_o;            // splits > 1: [rows, heads, splits, head_dim]
  float* part_ml;           // splits > 1: [rows, heads, splits, 2]
  float scale;
  int rows, heads, kv_heads, head_dim, block_size, max_blocks, splits, kv_kind;
  int num_blocks;           // blocks in the pool (0: unknown).  With a BF16 cache, 16-token pages and a status word the
                            // pages are fetched by TMA into a shared-memory ring; otherwise by plain loads
  int* status;              // device status word for the bounded waits of the TMA form (may be null: plain loads)
} NxPagedArgs;

// One query row per (sequence, position): decode steps and speculative verification rows alike.
int nx_paged_attention_decode(const NxPagedArgs* args, nx_stream_t stream);

// y[m][n] = act(x[m][:] . w[n][:] + bias[n]) + residual[m][n], 1 <= m <= nx_skinny_max_rows().
// The reduction order of a row is fixed, so a row's result does not depend on the batch it is in.
int nx_skinny_max_rows(void);
// y and residual share out_dtype (BF16 or FP32); y may alias residual.
int nx_skinny_gemm(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* bias, const void* residual,
                   int64_t ldr, void* y, int64_t ldy, int out_dtype, int m, int n, int k, int act,
                   nx_stream_t stream);

int nx_gather_rows(const void* x, const int32_t* rows, void* out, int n, int cols, nx_stream_t stream);
// counts[row_of[i]][tokens[i]] += 1
int nx_count_tokens(const int32_t* tokens, const int32_t* row_of, int32_t* counts, int n, int vocab,
                    nx_stream_t stream);
// out[r] = logsumexp(logits[r]) - logits[r][targets[r]]   (FP32 logits)
int nx_nll(const float* logits, int64_t ld, const int32_t* targets, float* out, int rows, int vocab,
           nx_stream_t stream);

typedef struct NxSampleParams {
  float temperature;         // <= 0: greedy (ties -> lowest id)
  float top_p;               // (0, 1): nucleus;  otherwise off
  float min_p;               // > 0: drop tokens below min_p * p_max
  float repetition_penalty;  // 1: off
  float frequency_penalty;
  float presence_penalty;
  int top_k;                 // <= 0: off
  int pad;
  uint64_t seed;             // Philox key; the draw of a row uses counter offsets[row]
} NxSampleParams;

// logits: FP32 [rows, ld].  work: FP32 [rows, vocab] scratch.  counts_all / counts_out (optional): INT32
// [*, vocab] occurrences of each token in prompt + output (repetition penalty) and in the output only
// (frequency / presence penalties); row r uses table row count_row[r] (or r when count_row is null).
int nx_sample(const float* logits, int64_t ld, int vocab, const NxSampleParams* params, const int32_t* counts_all,
              const int32_t* counts_out, const int32_t* count_row, const uint64_t* offsets, float* work, int32_t* out,
              int rows, nx_stream_t stream);

// In-place rotary embedding on [rows, heads, head_dim]; cos/sin: FP32 [max_pos, rot_dim / 2].
int nx_rope(void* x, int64_t row_stride, const int32_t* positions, const float* cos_t, const float* sin_t, int rows,
            int heads, int head_dim, int rot_dim, int inverse, int interleaved, nx_stream_t stream);

// h: [n, 2F] = [gate | up];  y = act(gate) * up;  act 0 = SiLU (SwiGLU), 1 = GELU-tanh (GeGLU)
int nx_gated_fwd(const void* h, void* y, int64_t n, int F, int act, nx_stream_t stream);
int nx_gated_bwd(const void* h, const void* dy, void* dh, int64_t n, int F, int act, nx_stream_t stream);

// Weight-only quantisation.  bits 8: INT8 [n, k] with one scale per output row.  bits 4: two nibbles
// per byte [n, k/2], value = (nibble - 8) * scale[row][col / group].
int nx_wq_gemv(const void* x, int64_t ldx, const void* wq, const float* scales, int bits, int group, const void* bias,
               void* y, int64_t ldy, int m, int n, int k, nx_stream_t stream);
int nx_wq_dequant(const void* wq, const float* scales, int bits, int group, void* w, int n, int k,
                  nx_stream_t stream);
// Per-row symmetric INT8 quantisation of activations; inv_smooth (optional): per-column multipliers.
// Any of q (INT8 codes), fake_quant (BF16 code * scale) and row_scale may be null.
int nx_quant_rows(const void* x, const float* inv_smooth, void* q, void* fake_quant, float* row_scale, int rows,
                  int cols, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
