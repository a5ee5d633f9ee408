// C ABI of the attention kernels.  A view addresses element (b, t, h, d) at
// ptr[b*batch_stride + t*row_stride + h*head_stride + d]; strides are in elements and multiples of 8,
// which covers packed QKV ([B,T,3,H,D]) as well as separate [B,T,H,D] tensors.  BF16 only.
#pragma once
#include "nx_api.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct NxAttnView {
  void* ptr;
  int64_t row_stride, head_stride, batch_stride;
} NxAttnView;

typedef struct NxAttnArgs {
  NxAttnView q, k, v, o;        // o: forward output (read by backward)
  NxAttnView d_o, dq, dk, dv;   // backward only
  float* lse;                   // [B, H, Tq] natural-log log-sum-exp
  float* dsum;                  // [B, H, Tq] scratch for backward (rowsum(dO * O))
  int* status;                  // device int, non-zero when a bounded wait ran out
  int32_t batch, heads, kv_heads, tq, tk, head_dim;
  int32_t causal;               // bottom-right aligned when tq != tk
  int32_t window;               // <= 0: unlimited; else each query sees the last `window` keys
  float scale;                  // softmax scale (1/sqrt(head_dim) by convention)
  // Forward only, optional: running FP32 output [B, Tq, H, D] and log-sum-exp [B, H, Tq] of earlier
  // key/value chunks (start: zeros / -inf).  The kernel merges this chunk into them (softmax over the
  // union of the key sets) and writes the merged result to `o` and `lse` as well: one launch per ring step.
  float* merge_o;
  float* merge_lse;
  float softcap;                // > 0: scores become softcap * tanh(scale * s / softcap) (forward and backward)
  const float* alibi_slopes;    // [heads] or null: slope_h * (key position - query position), positions aligned
                                // bottom-right like the causal mask, is added to the scaled score
  // Attention dropout, 0 <= dropout_p < 1: P[b, h, q, k] is dropped (and the rest scaled by 1 / (1 - p)) when
  // element ((b * heads + h) * tq + q) * tk + k of the Philox stream (seed, offset) is below p; the mask is
  // regenerated in the backward kernels.  Out-of-range values are rejected.
  float dropout_p;
  uint64_t dropout_seed, dropout_offset;
} NxAttnArgs;

int nx_attention_fwd(const NxAttnArgs* args, nx_stream_t stream);
int nx_attention_bwd(const NxAttnArgs* args, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
