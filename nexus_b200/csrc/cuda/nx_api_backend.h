// C ABI of the FP32 driver kernels used by the backend abstraction and of the tensor-dispatcher helpers.
#pragma once
#include "nx_api.h"

#ifdef __cplusplus
extern "C" {
#endif

enum NxEwOp {
  NX_EW_ADD = 0, NX_EW_SUB = 1, NX_EW_MUL = 2, NX_EW_DIV = 3, NX_EW_NEG = 4, NX_EW_EXP = 5, NX_EW_LOG = 6,
  NX_EW_SQRT = 7, NX_EW_RSQRT = 8, NX_EW_TANH = 9, NX_EW_SIGMOID = 10, NX_EW_SILU = 11, NX_EW_RELU = 12,
  NX_EW_SCALE = 13,  // x * scalar
  NX_EW_AXPY = 14    // x * scalar + b
};
enum NxRowOp { NX_ROW_SOFTMAX = 0, NX_ROW_RMSNORM = 1, NX_ROW_LAYERNORM = 2 };

int nx_bk_elementwise(const float* a, const float* b, float* out, int64_t n, float scalar, int op,
                      nx_stream_t stream);
// Deterministic sum: partial must hold nx_bk_reduce_partials(n) doubles.
int64_t nx_bk_reduce_partials(int64_t n);
int nx_bk_reduce_sum(const float* x, int64_t n, double* partial, float* out, nx_stream_t stream);
// C = alpha * op(A) * op(B) + beta * C (row-major; trans_a: A stored [k][lda]; trans_b: B stored [n][ldb])
int nx_bk_matmul_f32(const float* a, const float* b, float* c, int m, int n, int k, int lda, int ldb, int ldc,
                     int trans_a, int trans_b, float alpha, float beta, nx_stream_t stream);
// q, k, v, o: [bh, T, D] FP32, D <= 128
int nx_bk_attention_f32(const float* q, const float* k, const float* v, float* o, int bh, int T, int D, float scale,
                        int causal, nx_stream_t stream);
int nx_bk_norm_softmax(const float* x, const float* gamma, const float* beta, float* y, int rows, int cols, int op,
                       float eps, nx_stream_t stream);
// x, y: [bh, T, 2 * half]; pair j of position t (+ pos_offset) rotates by t / theta^(j / half)
int nx_bk_rope_pairs(const float* x, float* y, int bh, int T, int half, int pos_offset, float theta,
                     nx_stream_t stream);
// x: [rows, 2 * hidden] = [gate | up]
int nx_bk_swiglu_f32(const float* x, float* y, int rows, int hidden, nx_stream_t stream);
// p -= lr * (m_hat / (sqrt(v_hat) + eps) + weight_decay * p), bc = 1 - beta^t
int nx_bk_adamw_step(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1, float beta2,
                     float eps, float weight_decay, float bc1, float bc2, nx_stream_t stream);
// a: FP32 [m, k]; wq: [n, k] packed INT8 (bits 8) or nibble-8 (bits 4); scales: [n, k / group]
int nx_bk_quant_matmul(const float* a, const void* wq, const float* scales, float* c, int m, int n, int k, int group,
                       int bits, nx_stream_t stream);

int nx_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, nx_stream_t stream);
int nx_fill(void* dst, int dtype, int64_t n, float value, nx_stream_t stream);
// dy == null: out = gelu_tanh(x); else out = dy * gelu_tanh'(x)
int nx_gelu(const void* x, const void* dy, void* out, int dtype, int64_t n, nx_stream_t stream);
// scores [rows, T] with row r at position r % T; dy == null: out = softmax(scale * x) under the causal
// mask; else x holds the probabilities and out = d(scores)
int nx_causal_softmax(const float* x, const float* dy, float* out, int64_t rows, int T, float scale,
                      nx_stream_t stream);
// merge == 0: packed [B, T, 3, H, D] -> q, k, v [B, H, T, D]; merge == 1: the inverse (BF16)
int nx_split_heads(void* qkv, void* q, void* k, void* v, int B, int T, int H, int D, int merge, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
