// C ABI of the low-precision kernels: FP8 quantisation and the 8-bit blockwise AdamW.
#pragma once
#include "nx_api_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

// dst = fp8(src * *scale) (scale null: 1); *amax = max(*amax, max |src|) (amax null: skipped).  fmt: NX_E4M3 / NX_E5M2.
int nx_fp8_quantize(const void* src, int src_dtype, void* dst, int fmt, int64_t n, const float* scale, float* amax,
                    nx_stream_t stream);
// Per-row dynamic scaling: dst[r] = fp8(src[r] * fmax / amax_r); scale_inv[r] = amax_r / fmax (the GEMM's row scale).
int nx_fp8_quantize_rows(const void* src, int src_dtype, void* dst, int fmt, int rows, int cols, float* scale_inv,
                         nx_stream_t stream);
int nx_fp8_dequantize(const void* src, int fmt, void* dst, int dst_dtype, int64_t n, const float* scale_inv,
                      nx_stream_t stream);

// ---- block-scaled FP8 (MX): one power-of-two scale (E8M0 byte, value 2^(byte-127)) per 32 elements along K ----
// Scale storage ("atoms"): for a matrix of R rows and K columns the scales of row block rb = r / 128 and column block
// kb = k / 128 form one 512-byte atom at byte offset (rb * ceil(K/128) + kb) * 512; inside the atom the scale of row r
// and 32-element block j = (k / 32) % 4 sits at byte (r % 32) * 16 + ((r % 128) / 32) * 4 + j.  This is the order the
// tensor core reads scale factors from tensor memory, so the GEMM moves an atom with one bulk copy and no shuffle.
size_t nx_mx_scale_bytes(int rows, int cols);
// Quantise src [rows][ld] (BF16 / F32 / F16) to FP8 codes with E8M0 block scales chosen so that no value saturates.
// transpose == 0: codes [rows][cols], blocks run along the columns (the matrix is a K-major GEMM operand as stored).
// transpose == 1: codes [cols][rows] (the transposed matrix), blocks run along the source's rows - the operand form
//                 the backward GEMMs need.  `scales` has nx_mx_scale_bytes(rows of the codes, columns of the codes).
int nx_mx_quantize(const void* src, int src_dtype, int64_t ld, int rows, int cols, void* codes, void* scales, int fmt,
                   int transpose, nx_stream_t stream);
// dst [rows][cols] = codes * scale (the inverse of nx_mx_quantize with transpose == 0); for tests and fallbacks.
int nx_mx_dequantize(const void* codes, const void* scales, int fmt, int rows, int cols, void* dst, int dst_dtype,
                     nx_stream_t stream);
// out[m][n] = act(alpha * sum_k (A[m][k] sfa[m][k/32]) * (B[n][k] sfb[n][k/32]) + bias[n]) on the block-scaled tensor
// core path (tcgen05 kind::mxf8f6f4, scales in tensor memory).  A is [M][lda], B is [N][ldb], both K contiguous,
// pitches multiples of 16.  out_dtype NX_BF16 / NX_F32 writes the values; NX_E4M3 / NX_E5M2 writes block-scaled codes
// [M][ldo] plus `out_scales` (atoms of an M x N matrix: the K-major operand of the next GEMM), N a multiple of 32.
typedef struct NxMxGemmArgs {
  const void* a;
  const void* b;
  const void* sfa;   // scale atoms of A
  const void* sfb;   // scale atoms of B
  void* out;
  void* out_scales;  // only for 8-bit out_dtype
  const void* bias;  // [N], may be null
  float* amax_out;   // receives max |value| (zeroed by the caller), may be null
  int* status;       // device int, receives a non-zero status when a wait timed out
  int64_t lda, ldb, ldo;
  int32_t m, n, k;
  int32_t a_dtype, b_dtype;  // NX_E4M3 / NX_E5M2
  int32_t out_dtype, bias_dtype, act;
  float alpha;
  int32_t max_ctas;  // 0 = one per SM
} NxMxGemmArgs;
int nx_gemm_mxf8(const NxMxGemmArgs* args, nx_stream_t stream);

// 8-bit AdamW.  Moments are one byte per element plus one FP32 absmax per block of nx_adamw8_block()
// elements (all zero at the start).  master (FP32) and shadow (BF16) may each be null, not both.
// clip: device pointer to the clip factor to use (null: state->clip_coef) - lets a per-layer update run
// inside the backward pass with the factor derived from the previous step's norm.
int nx_adamw8_block(void);
int nx_adamw8(float* master, void* shadow, float* grad, void* qm, void* qv, float* absmax_m, float* absmax_v, int64_t n,
              const NxOptState* state, float wd_scale, float lr_scale, const float* clip, int zero_grad,
              nx_stream_t stream);
// *accum += sum(grad^2)
int nx_grad_sq_accumulate(const float* grad, int64_t n, double* accum, nx_stream_t stream);
// *clip = min(1, max_norm / (sqrt(*accum) + 1e-6)); *norm_out = sqrt(*accum); *accum = 0
int nx_delayed_clip_finish(float* clip, float* norm_out, double* accum, double max_norm, nx_stream_t stream);

#ifdef __cplusplus
}
#endif
