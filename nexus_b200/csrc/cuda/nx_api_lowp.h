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
