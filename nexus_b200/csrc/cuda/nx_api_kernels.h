// C ABI of the memory-bound kernels (norms, embedding, cross-entropy, dropout, optimizer,
// elementwise, LM helpers, FP8, inference).  Conventions as in nx_api.h.
#pragma once
#include "nx_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Device-resident optimizer state: the host writes lr / hyper-parameters before a step (or a CUDA
// graph replay), kernels read them from here, so a captured step never bakes a learning rate in.
typedef struct NxOptState {
  double local_sq;      // out: local sum of squared gradients (before any cross-rank reduce)
  float lr;             // in
  float weight_decay;   // in
  float beta1, beta2;   // in
  float eps;            // in
  float max_grad_norm;  // in, <= 0 disables clipping
  float loss_scale;     // in/out, 0 or 1 = none
  float grad_norm;      // out
  float clip_coef;      // out: min(1, max/(norm+1e-6)) / loss_scale
  float inv_bias1;      // out: 1 / (1 - beta1^step)
  float inv_bias2;      // out
  int32_t step;         // in/out: accepted optimizer steps
  int32_t found_inf;    // out
  int32_t skipped;      // out: steps skipped because of non-finite gradients
  int32_t good_steps;   // loss-scale growth counter
  int32_t reserved;
} NxOptState;

typedef struct NxAdamChunk {
  int64_t offset;  // element offset into the flat buffers
  int64_t count;
  float wd_scale;  // multiplies weight_decay (0 for biases / norms)
  float lr_scale;  // multiplies lr
} NxAdamChunk;

// ---- norms -------------------------------------------------------------------------------------
int nx_norm_fwd(int rms, const void* x, int x_dtype, const void* residual, void* sum_out, const void* gamma,
                const void* beta, int param_dtype, void* y, int y_dtype, float* mean, float* rstd, int rows, int cols,
                float eps, nx_stream_t stream);
size_t nx_norm_bwd_scratch_bytes(int rows, int cols);
int nx_norm_bwd(int rms, const void* dy, int dy_dtype, const void* x, int x_dtype, const void* gamma,
                int param_dtype, const float* mean, const float* rstd, const void* add, void* dx, int dx_dtype,
                void* dx_lp /* optional BF16 copy of dx */, float* dgamma, float* dbeta, int accumulate_params,
                float* scratch, int rows, int cols, nx_stream_t stream);
// The same, plus `dx_colsum` ([cols], optional): column sums of `dx_lp` (the bias gradient of the linear layer whose
// output gradient `dx_lp` is), accumulated like dgamma / dbeta.  -4: no single-pass instance for this shape / types.
int nx_norm_bwd_colsum(int rms, const void* dy, int dy_dtype, const void* x, int x_dtype, const void* gamma,
                       int param_dtype, const float* mean, const float* rstd, const void* add, void* dx, int dx_dtype,
                       void* dx_lp, float* dgamma, float* dbeta, float* dx_colsum, int accumulate_params, float* scratch,
                       int rows, int cols, nx_stream_t stream);

// ---- embedding ---------------------------------------------------------------------------------
int nx_embedding_pos_fwd(const int32_t* tokens, const int32_t* positions, const void* wte, const void* wpe,
                         int w_dtype, void* out, int out_dtype, int64_t rows, int seq_len, int cols,
                         nx_stream_t stream);
// dwte/dwpe are FP32 and accumulated into.  With `sorted_tokens` + `order` (rows sorted by token)
// the token-embedding gradient is summed in a fixed order; without them it uses atomics.
int nx_embedding_bwd(const int32_t* tokens, const int32_t* sorted_tokens, const int64_t* order, const void* dx,
                     int dx_dtype, float* dwte, float* dwpe, int batch, int seq_len, int cols, nx_stream_t stream);

// ---- cross-entropy -----------------------------------------------------------------------------
size_t nx_ce_state_bytes(void);
// targets == null: shifted targets tokens[b, t+1], last position of every sequence ignored.
// Logits [rows, ld] are overwritten with d(loss * grad_scale)/dlogits when write_grad != 0.
int nx_cross_entropy_shifted(void* logits, int logits_dtype, const int32_t* tokens, const int32_t* targets,
                             float* row_loss, void* ce_state, float* loss_out, float loss_weight,
                             int accumulate_loss, int64_t rows, int seq_len, int vocab, int64_t ld, int ignore_index,
                             float smoothing, float z_loss, float grad_scale, int write_grad, nx_stream_t stream);
// The same with a second, device-resident gradient multiplier (`grad_scale_dev`, may be null): the dynamic loss scale
// of the optimizer state, read on the device so that a captured step follows its changes.
int nx_cross_entropy_shifted_scaled(void* logits, int logits_dtype, const int32_t* tokens, const int32_t* targets,
                                    float* row_loss, void* ce_state, float* loss_out, float loss_weight,
                                    int accumulate_loss, int64_t rows, int seq_len, int vocab, int64_t ld,
                                    int ignore_index, float smoothing, float z_loss, float grad_scale,
                                    const float* grad_scale_dev, int write_grad, nx_stream_t stream);

// ---- dropout / rng -----------------------------------------------------------------------------
int nx_dropout(const void* in, void* out, int dtype, int64_t n, float p, uint64_t seed, uint64_t offset,
               int backward, nx_stream_t stream);
int nx_philox_uniform(float* out, int64_t n, uint64_t seed, uint64_t offset, nx_stream_t stream);

// ---- optimizer ---------------------------------------------------------------------------------
int64_t nx_grad_norm_partials(int64_t n);
// local_only: publish state->local_sq and stop (caller reduces across ranks, then calls again with
// extra_sq pointing at the global square sum).  extra_sq != null: skip the local pass.
int nx_grad_norm(const void* grad, int grad_dtype, int64_t n, double* partial, NxOptState* state,
                 const double* extra_sq, int local_only, nx_stream_t stream);
int nx_adamw(float* master, const void* grad, int grad_dtype, float* m, float* v, void* shadow, int shadow_dtype,
             const NxAdamChunk* chunks, int nchunks, const NxOptState* state, int zero_grad, uint64_t sr_seed,
             nx_stream_t stream);
int nx_loss_scale_update(NxOptState* state, float growth, float backoff, int growth_interval, float min_scale,
                         float max_scale, nx_stream_t stream);
int nx_count_nonfinite(const void* x, int dtype, int64_t n, int* count, nx_stream_t stream);
size_t nx_colsum_scratch_bytes(int rows, int cols);
int nx_colsum(const void* dy, int dtype, float* out, float* scratch, int rows, int cols, int64_t ld, int accumulate,
              nx_stream_t stream);

// ---- column sums for callers that cannot allocate -----------------------------------------------
// (This entry point has no counterpart in the reference; it exists for embedders of this library.)
//
// Same result as nx_colsum, but the partial-sum scratch is a fixed 2 MiB array inside the library
// image instead of a caller buffer, and the call performs no device allocation of any kind.  It is
// meant for hosts that must not call cudaMalloc while running: a server that handed all free HBM
// to its own arena (a KV cache, say) at start-up and has nothing left for the driver to give, or a
// latency-critical loop that cannot afford the device-wide synchronisation an allocation implies.
//
//   * cols <= nx_colsum_static_max_cols() (8192); larger inputs return -5 with a message on stderr.
//   * The first call on each device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and caches it; make that first call during set-up, before any stream
//     capture begins.  Every GPU that loads the library keeps the 2 MiB until the process exits.
//   * The device that holds the data must be the current device, and `stream` must be one of its streams: the
//     array that is used is the current device's copy.  Data on another device returns -6.
//   * All calls on a device share the one array and it keeps the previous call's partials.  Each
//     call overwrites every entry it later reads, so nothing needs clearing, but two calls that
//     overlap on the GPU (different streams) race on it: keep them on one stream or order them.
int nx_colsum_static_max_cols(void);
int nx_colsum_static(const void* dy, int dtype, float* out, int rows, int cols, int64_t ld, int accumulate,
                     nx_stream_t stream);

#ifdef __cplusplus
}
#endif
