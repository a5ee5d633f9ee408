// C ABI of the MoE routing kernels.
#pragma once
#include "nx_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// logits: FP32 [tokens, experts].  expert / gate: [tokens, k]; gate = softmax over the k selected logits;
// ties go to the lower expert id.
int nx_moe_topk(const float* logits, int tokens, int experts, int k, int32_t* expert, float* gate, nx_stream_t stream);
// slot[t, j] = position of the assignment inside its expert's buffer in priority order (j, then t), or -1
// beyond `capacity`; counts[e] = rows kept by expert e; *dropped += assignments dropped (may be null).
int nx_moe_assign(const int32_t* expert, int tokens, int k, int experts, int capacity, int32_t* slot, int32_t* counts,
                  int32_t* dropped, nx_stream_t stream);
// Capacity per group of tokens (`tokens / groups` consecutive tokens each) and the Reroute overflow policy.  The
// assignments of a group are visited in priority order (j, then t).  `order` null: an assignment past its expert's
// capacity is dropped (slot -1).  `order` [tokens, experts] (each token's experts by descending score): such an
// assignment moves to the token's best expert that has room and is none of its own choices (`expert` is updated in
// place, *rerouted counts them) and is dropped only when there is none.  slot = group * capacity + position, i.e.
// the expert buffers are [experts, groups * capacity, d]; counts[g * experts + e] = rows of group g kept by expert e.
int nx_moe_assign_groups(int32_t* expert, const int32_t* order, int tokens, int k, int experts, int groups,
                         int capacity, int32_t* slot, int32_t* counts, int32_t* dropped, int32_t* rerouted,
                         nx_stream_t stream);
// dgate[t, j] = dy[t] . expert_out[expert[t,j]][slot[t,j]]  (BF16 rows of d elements)
int nx_moe_gate_grad(const void* dy, const void* expert_out, const int32_t* expert, const int32_t* slot, float* dgate,
                     int tokens, int k, int d, int capacity, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
