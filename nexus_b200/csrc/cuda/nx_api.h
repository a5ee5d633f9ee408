// C ABI of the sm_100a kernel library (libnexus_b200_cuda.so).
// Every entry point takes raw device pointers plus the CUDA stream to launch on and returns 0 on
// success or a negative error code (-1 bad argument, -2 CUDA launch error, -3 driver entry missing).
// Nothing here allocates device memory: scratch buffers are supplied by the caller.
// Parity: the reference exposes its kernels the same way, as free functions over device pointers
// and a cudaStream_t (include/nexus/cuda/kernels.hpp:32-271, include/nexus/cuda/gemm.hpp:50-80).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* nx_stream_t;

enum NxDType { NX_BF16 = 0, NX_F32 = 1, NX_F16 = 2, NX_E4M3 = 3, NX_E5M2 = 4 };
enum NxAct { NX_ACT_NONE = 0, NX_ACT_GELU = 1, NX_ACT_RELU = 2, NX_ACT_DGELU = 3, NX_ACT_SILU = 4 };

// out[b][m][n] = epilogue( alpha * sum_k A[b][m][k] * B[b][n][k] )
// Operand memory: a_mn_major == 0 -> A is [M][lda] (K contiguous); 1 -> A is [K][lda] (M contiguous).
//                 b_mn_major == 0 -> B is [N][ldb] (K contiguous); 1 -> B is [K][ldb] (N contiguous).
// Epilogue order: v = alpha*acc; v += bias[n]; (DGELU: v *= gelu'(aux_in[m][n])); aux_out[m][n] = v;
//                 v = act(v); v += residual[m][n]; (accumulate: v += out[m][n]); out[m][n] = v.
typedef struct NxGemmArgs {
  const void* a;
  const void* b;
  void* out;
  const void* bias;      // [N], dtype bias_dtype, may be null
  const void* aux_in;    // bf16 [M][ld_aux], pre-activation for DGELU, may be null
  void* aux_out;         // bf16 [M][ld_aux], receives the pre-activation, may be null
  const void* residual;  // [M][ld_res], dtype res_dtype, may be null
  float* workspace;      // split-K partials: split_k * M * N floats (batch must be 1)
  int* status;           // device int, receives a non-zero nx::StatusCode when a wait timed out
  int64_t lda, ldb, ldo, ld_aux, ld_res;
  int64_t stride_a, stride_b, stride_o;  // batch strides in elements
  int32_t m, n, k, batch;
  int32_t a_mn_major, b_mn_major;
  int32_t in_dtype;   // NX_BF16, NX_F16, or NX_E4M3 / NX_E5M2 (8-bit: K-major operands, pitches % 16 == 0)
  int32_t out_dtype;  // NX_BF16 or NX_F32
  int32_t bias_dtype, res_dtype;
  int32_t act;
  int32_t accumulate;  // 0 overwrite, 1 out += v, 2 (split_k > 1, FP32 out) slices add with vector reductions
  int32_t split_k;  // 1 = none
  int32_t block_n;  // 0 = choose; else 128 or 256
  float alpha;
  int32_t max_ctas;  // 0 = one per SM
  int32_t b_dtype_plus1;  // 8-bit inputs: dtype of B plus one (0: same as A), e.g. E5M2 grads x E4M3 weights
  const float* scale_a;   // [M] per-row dequantisation scale of A, may be null
  const float* scale_b;   // [N] per-row dequantisation scale of B, may be null
  float* amax_out;        // receives max |out| (must be zeroed by the caller), may be null
} NxGemmArgs;

int nx_gemm(const NxGemmArgs* args, nx_stream_t stream);
// Sum split-K partials in slice order and apply "out (+)= v" with the dtype of `out`.
int nx_splitk_reduce(const float* workspace, void* out, int out_dtype, int64_t ldo, int m, int n, int split_k,
                     int accumulate, nx_stream_t stream);
// The same, with the epilogue the split GEMM could not apply itself: out = act(sum of slices + bias) (+ out when
// `accumulate`).  act: NX_ACT_NONE / GELU / RELU / SILU.
int nx_splitk_reduce_epilogue(const float* workspace, void* out, int out_dtype, int64_t ldo, int m, int n, int split_k,
                              int accumulate, const void* bias, int bias_dtype, int act, nx_stream_t stream);
int nx_sm_count(void);
size_t nx_gemm_workspace_bytes(int m, int n, int split_k);

#ifdef __cplusplus
}
#endif
