// FP32 driver kernels behind the backend abstraction (elementwise set, deterministic sum, tiled FP32
// matmul with transpose flags and alpha/beta, causal online-softmax attention, row softmax / RMSNorm /
// LayerNorm, interleaved-pair RoPE, SwiGLU, AdamW in decay-in-lr form, group-quantised Q8 / Q4 matmul)
// plus the tensor-dispatcher helpers (cast, fill, GELU fwd/bwd, causal softmax fwd/bwd, split / merge of
// packed QKV heads).  The same math exists in the reference as Vulkan compute shaders
// (shaders/vulkan/{elementwise,reduce_sum,matmul,attention,norm_softmax,special_ops,quant_matmul}.comp)
// and as CUDA helpers (src/cuda/kernels_elementwise.cu, src/cuda/tensor_kernels.cu); here they are CUDA
// kernels written for 32-wide warps, 16-byte accesses and shuffle reductions.
#include "common.cuh"
#include "nx_api_backend.h"
#include "sm100_ptx.cuh"

namespace {
using namespace nx;

// ------------------------------------------------------------------------------------------------
// elementwise (15 ops), float4 main loop + scalar tail
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float ew_apply(int op, float x, float y, float s) {
  switch (op) {
    case NX_EW_ADD: return x + y;
    case NX_EW_SUB: return x - y;
    case NX_EW_MUL: return x * y;
    case NX_EW_DIV: return x / y;
    case NX_EW_NEG: return -x;
    case NX_EW_EXP: return expf(x);
    case NX_EW_LOG: return logf(x);
    case NX_EW_SQRT: return sqrtf(x);
    case NX_EW_RSQRT: return rsqrtf(x);
    case NX_EW_TANH: return tanhf(x);
    case NX_EW_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case NX_EW_SILU: return x / (1.0f + expf(-x));
    case NX_EW_RELU: return fmaxf(x, 0.0f);
    case NX_EW_SCALE: return x * s;
    case NX_EW_AXPY: return x * s + y;
    default: return x;
  }
}

__global__ void elementwise_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                                   int64_t n, float scalar, int op, int vec_ok) {
  const bool binary = op <= NX_EW_DIV || op == NX_EW_AXPY;
  const int64_t n4 = vec_ok ? n >> 2 : 0;
  NX_GRID_STRIDE(i, n4) {
    const float4 x = reinterpret_cast<const float4*>(a)[i];
    const float4 y = binary ? reinterpret_cast<const float4*>(b)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 r;
    r.x = ew_apply(op, x.x, y.x, scalar);
    r.y = ew_apply(op, x.y, y.y, scalar);
    r.z = ew_apply(op, x.z, y.z, scalar);
    r.w = ew_apply(op, x.w, y.w, scalar);
    reinterpret_cast<float4*>(o)[i] = r;
  }
  NX_GRID_STRIDE(j, n - 4 * n4) {
    const int64_t i = 4 * n4 + j;
    o[i] = ew_apply(op, a[i], binary ? b[i] : 0.0f, scalar);
  }
}

// deterministic sum: fixed chunk per block (FP32 inside the block in a fixed tree, FP64 across blocks)
constexpr int kSumChunk = 8192;
__global__ void reduce_partial_kernel(const float* __restrict__ x, int64_t n, double* __restrict__ partial) {
  __shared__ float s_scratch[32];
  const int64_t begin = static_cast<int64_t>(blockIdx.x) * kSumChunk;
  const int64_t end = min(n, begin + kSumChunk);
  float acc = 0.0f;
  for (int64_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc += x[i];
  acc = block_sum<float>(acc, s_scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = static_cast<double>(acc);
}
__global__ void reduce_final_kernel(const double* __restrict__ partial, int n, float* __restrict__ out) {
  __shared__ double s_scratch[32];
  double acc = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partial[i];
  acc = block_sum<double>(acc, s_scratch);
  if (threadIdx.x == 0) *out = static_cast<float>(acc);
}

// ------------------------------------------------------------------------------------------------
// FP32 matmul: C = alpha * op(A) op(B) + beta * C, 64x64 tile, 16-deep k slab, 4x4 per thread
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
matmul_f32_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c, int m, int n, int k,
                  int lda, int ldb, int ldc, int trans_a, int trans_b, float alpha, float beta) {
  __shared__ float sa[16][65];
  __shared__ float sb[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      const int kk = e & 15, r = e >> 4;
      const int gr = row0 + r, gk = k0 + kk;
      sa[kk][r] = (gr < m && gk < k) ? (trans_a ? a[static_cast<int64_t>(gk) * lda + gr] : a[static_cast<int64_t>(gr) * lda + gk]) : 0.0f;
      const int gc = col0 + r;
      sb[kk][r] = (gc < n && gk < k) ? (trans_b ? b[static_cast<int64_t>(gc) * ldb + gk] : b[static_cast<int64_t>(gk) * ldb + gc]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = sa[kk][ty * 4 + i];
        bv[i] = sb[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + ty * 4 + i, cc = col0 + tx * 4 + j;
      if (r < m && cc < n) {
        float* p = c + static_cast<int64_t>(r) * ldc + cc;
        *p = beta == 0.0f ? alpha * acc[i][j] : alpha * acc[i][j] + beta * *p;
      }
    }
}

// ------------------------------------------------------------------------------------------------
// FP32 causal attention, one warp per query row, lanes own head_dim/32 (<= 4) channels
// ------------------------------------------------------------------------------------------------
__global__ void attention_f32_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                     const float* __restrict__ v, float* __restrict__ o, int bh, int T, int D,
                                     float scale, int causal) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= bh * T) return;
  const int t = warp % T;
  const int64_t base = static_cast<int64_t>(warp / T) * T * D;
  float qv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 4; ++j) qv[j] = (lane + 32 * j < D) ? q[base + static_cast<int64_t>(t) * D + lane + 32 * j] * scale : 0.0f;
  float mx = -INFINITY, l = 0.0f;
  const int last = causal ? t : T - 1;
  for (int s = 0; s <= last; ++s) {
    float dot = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (lane + 32 * j < D) dot += qv[j] * k[base + static_cast<int64_t>(s) * D + lane + 32 * j];
    dot = warp_sum(dot);
    const float mn = fmaxf(mx, dot);
    const float alpha = __expf(mx - mn), p = __expf(dot - mn);
    l = l * alpha + p;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (lane + 32 * j < D) acc[j] = acc[j] * alpha + p * v[base + static_cast<int64_t>(s) * D + lane + 32 * j];
    mx = mn;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (lane + 32 * j < D) o[base + static_cast<int64_t>(t) * D + lane + 32 * j] = acc[j] / l;
}

// ------------------------------------------------------------------------------------------------
// row softmax / RMSNorm / LayerNorm (FP32), block per row
// ------------------------------------------------------------------------------------------------
__global__ void norm_softmax_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                    const float* __restrict__ beta, float* __restrict__ y, int cols, int op,
                                    float eps) {
  __shared__ float s_scratch[32];
  const float* xr = x + static_cast<int64_t>(blockIdx.x) * cols;
  float* yr = y + static_cast<int64_t>(blockIdx.x) * cols;
  if (op == NX_ROW_SOFTMAX) {
    float mx = -INFINITY;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) mx = fmaxf(mx, xr[c]);
    mx = block_max(mx, s_scratch);
    float se = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) se += expf(xr[c] - mx);
    se = block_sum<float>(se, s_scratch);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = expf(xr[c] - mx) / se;
  } else if (op == NX_ROW_RMSNORM) {
    float ss = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += xr[c] * xr[c];
    ss = block_sum<float>(ss, s_scratch);
    const float r = rsqrtf(ss / cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) yr[c] = xr[c] * r * (gamma ? gamma[c] : 1.0f);
  } else {
    float s1 = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s1 += xr[c];
    const float mu = block_sum<float>(s1, s_scratch) / cols;
    float s2 = 0.0f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s2 += (xr[c] - mu) * (xr[c] - mu);
    const float r = rsqrtf(block_sum<float>(s2, s_scratch) / cols + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
      yr[c] = (xr[c] - mu) * r * (gamma ? gamma[c] : 1.0f) + (beta ? beta[c] : 0.0f);
  }
}

// interleaved-pair RoPE with on-the-fly angles: pair j of position t rotates by t / theta^(2j / (2*half))
__global__ void rope_pairs_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t pairs, int T, int half,
                                  int pos_offset, float theta) {
  NX_GRID_STRIDE(i, pairs) {
    const int j = static_cast<int>(i % half);
    const int64_t row = i / half;
    const int t = static_cast<int>(row % T) + pos_offset;
    const float ang = static_cast<float>(t) / powf(theta, static_cast<float>(2 * j) / static_cast<float>(2 * half));
    float s, c;
    sincosf(ang, &s, &c);
    const float x0 = x[row * 2 * half + 2 * j], x1 = x[row * 2 * half + 2 * j + 1];
    y[row * 2 * half + 2 * j] = x0 * c - x1 * s;
    y[row * 2 * half + 2 * j + 1] = x0 * s + x1 * c;
  }
}

__global__ void swiglu_f32_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n, int hidden) {
  NX_GRID_STRIDE(i, n) {
    const int64_t row = i / hidden;
    const int col = static_cast<int>(i % hidden);
    const float g = x[row * 2 * hidden + col], u = x[row * 2 * hidden + hidden + col];
    y[i] = g / (1.0f + expf(-g)) * u;
  }
}

// AdamW, decay inside the learning-rate term: p -= lr * (m_hat / (sqrt(v_hat) + eps) + wd * p)
__global__ void adamw_decay_in_lr_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                         float* __restrict__ v, int64_t n, float lr, float b1, float b2, float eps,
                                         float wd, float bc1, float bc2) {
  NX_GRID_STRIDE(i, n) {
    const float gi = g[i];
    const float mi = b1 * m[i] + (1.0f - b1) * gi;
    const float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float pi = p[i];
    p[i] = pi - lr * ((mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi);
  }
}

// group-quantised matmul, FP32 activations: c[r][col] = sum_g scale[col][g] * sum_{j in g} a[r][j] * q[col][j]
// One warp per output column; rows in register chunks of 8.  bits 8: int8; bits 4: nibble - 8.
template <int BITS>
__global__ void __launch_bounds__(256)
quant_matmul_kernel(const float* __restrict__ a, const uint32_t* __restrict__ wq, const float* __restrict__ ws,
                    float* __restrict__ c, int m, int n, int k, int group) {
  const int col = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (col >= n) return;
  constexpr int PER = BITS == 8 ? 4 : 8;  // weights per 32-bit word
  const int words = k / PER;
  const uint32_t* wrow = wq + static_cast<int64_t>(col) * words;
  const float* srow = ws + static_cast<int64_t>(col) * (k / group);
  for (int r0 = 0; r0 < m; r0 += 8) {
    float acc[8] = {};
    for (int w = lane; w < words; w += 32) {
      const uint32_t word = wrow[w];
      const float sc = srow[(w * PER) / group];
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const float qv = BITS == 8 ? static_cast<float>(static_cast<int8_t>((word >> (8 * j)) & 0xFF))
                                   : static_cast<float>(static_cast<int>((word >> (4 * j)) & 0xF) - 8);
        const float wv = qv * sc;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (r0 + i < m) acc[i] += a[static_cast<int64_t>(r0 + i) * k + w * PER + j] * wv;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = warp_sum(acc[i]);
      if (lane == 0 && r0 + i < m) c[static_cast<int64_t>(r0 + i) * n + col] = s;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// tensor-dispatcher helpers
// ------------------------------------------------------------------------------------------------
__global__ void cast_kernel(const void* __restrict__ src, int src_dtype, void* __restrict__ dst, int dst_dtype,
                            int64_t n) {
  NX_GRID_STRIDE(i, n) store_from_float(dst, dst_dtype, i, load_as_float(src, src_dtype, i));
}
__global__ void fill_kernel(void* __restrict__ dst, int dtype, int64_t n, float value) {
  NX_GRID_STRIDE(i, n) store_from_float(dst, dtype, i, value);
}
__global__ void gelu_kernel(const void* __restrict__ x, const void* __restrict__ dy, void* __restrict__ out, int dtype,
                            int64_t n) {
  NX_GRID_STRIDE(i, n) {
    const float v = load_as_float(x, dtype, i);
    store_from_float(out, dtype, i, dy ? load_as_float(dy, dtype, i) * dgelu_tanh_f(v) : gelu_tanh_f(v));
  }
}
// causal softmax over [rows = B*H*T, T] scores (row t sees columns <= t); dy == null: forward
__global__ void causal_softmax_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ out,
                                      int T, float scale) {
  __shared__ float s_scratch[32];
  const int64_t row = blockIdx.x;
  const int t = static_cast<int>(row % T);
  const float* xr = x + row * T;
  float* orow = out + row * T;
  if (dy == nullptr) {
    float mx = -INFINITY;
    for (int c = threadIdx.x; c <= t; c += blockDim.x) mx = fmaxf(mx, xr[c] * scale);
    mx = block_max(mx, s_scratch);
    float se = 0.0f;
    for (int c = threadIdx.x; c <= t; c += blockDim.x) se += expf(xr[c] * scale - mx);
    se = block_sum<float>(se, s_scratch);
    for (int c = threadIdx.x; c < T; c += blockDim.x) orow[c] = c <= t ? expf(xr[c] * scale - mx) / se : 0.0f;
  } else {  // x holds the probabilities y: dx = scale * y * (dy - sum(y * dy))
    const float* gr = dy + row * T;
    float dot = 0.0f;
    for (int c = threadIdx.x; c <= t; c += blockDim.x) dot += xr[c] * gr[c];
    dot = block_sum<float>(dot, s_scratch);
    for (int c = threadIdx.x; c < T; c += blockDim.x) orow[c] = c <= t ? scale * xr[c] * (gr[c] - dot) : 0.0f;
  }
}
// packed [B, T, 3, H, D] <-> three [B, H, T, D] tensors
__global__ void split_heads_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q,
                                   __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v, int B, int T, int H,
                                   int D, int merge) {
  const int64_t n = static_cast<int64_t>(B) * T * H * D;
  NX_GRID_STRIDE(i, n) {
    const int d = static_cast<int>(i % D);
    const int h = static_cast<int>((i / D) % H);
    const int t = static_cast<int>((i / (static_cast<int64_t>(D) * H)) % T);
    const int b = static_cast<int>(i / (static_cast<int64_t>(D) * H * T));
    const int64_t src = ((static_cast<int64_t>(b) * T + t) * 3 * H + h) * D + d;
    const int64_t dst = ((static_cast<int64_t>(b) * H + h) * T + t) * D + d;
    const int64_t hd = static_cast<int64_t>(H) * D;
    if (merge) {
      const_cast<__nv_bfloat16*>(qkv)[src] = q[dst];
      const_cast<__nv_bfloat16*>(qkv)[src + hd] = k[dst];
      const_cast<__nv_bfloat16*>(qkv)[src + 2 * hd] = v[dst];
    } else {
      q[dst] = qkv[src];
      k[dst] = qkv[src + hd];
      v[dst] = qkv[src + 2 * hd];
    }
  }
}

inline cudaStream_t S(nx_stream_t s) { return static_cast<cudaStream_t>(s); }
}  // namespace

extern "C" int nx_bk_elementwise(const float* a, const float* b, float* out, int64_t n, float scalar, int op,
                                 nx_stream_t stream) {
  if (n <= 0) return 0;
  if (op < 0 || op > NX_EW_AXPY) return -1;
  const bool binary = op <= NX_EW_DIV || op == NX_EW_AXPY;
  if (binary && b == nullptr) return -1;
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out) | (binary ? reinterpret_cast<uintptr_t>(b) : 0);
  elementwise_kernel<<<blocks_for((n + 3) / 4, 256), 256, 0, S(stream)>>>(a, b, out, n, scalar, op, (bits & 15) == 0);
  return launch_status();
}

extern "C" int64_t nx_bk_reduce_partials(int64_t n) { return (n + kSumChunk - 1) / kSumChunk; }

extern "C" int nx_bk_reduce_sum(const float* x, int64_t n, double* partial, float* out, nx_stream_t stream) {
  if (n <= 0 || partial == nullptr) return -1;
  const int blocks = static_cast<int>(nx_bk_reduce_partials(n));
  reduce_partial_kernel<<<blocks, 256, 0, S(stream)>>>(x, n, partial);
  reduce_final_kernel<<<1, 1024, 0, S(stream)>>>(partial, blocks, out);
  return launch_status();
}

extern "C" int nx_bk_matmul_f32(const float* a, const float* b, float* c, int m, int n, int k, int lda, int ldb,
                                int ldc, int trans_a, int trans_b, float alpha, float beta, nx_stream_t stream) {
  if (m <= 0 || n <= 0 || k < 0) return -1;
  dim3 grid((n + 63) / 64, (m + 63) / 64);
  matmul_f32_kernel<<<grid, 256, 0, S(stream)>>>(a, b, c, m, n, k, lda, ldb, ldc, trans_a, trans_b, alpha, beta);
  return launch_status();
}

extern "C" int nx_bk_attention_f32(const float* q, const float* k, const float* v, float* o, int bh, int T, int D,
                                   float scale, int causal, nx_stream_t stream) {
  if (bh <= 0 || T <= 0 || D <= 0 || D > 128) return -1;
  const int64_t warps = static_cast<int64_t>(bh) * T;
  attention_f32_kernel<<<static_cast<int>((warps + 7) / 8), 256, 0, S(stream)>>>(q, k, v, o, bh, T, D, scale, causal);
  return launch_status();
}

extern "C" int nx_bk_norm_softmax(const float* x, const float* gamma, const float* beta, float* y, int rows, int cols,
                                  int op, float eps, nx_stream_t stream) {
  if (rows <= 0 || cols <= 0 || op < 0 || op > NX_ROW_LAYERNORM) return -1;
  norm_softmax_kernel<<<rows, cols >= 1024 ? 512 : 128, 0, S(stream)>>>(x, gamma, beta, y, cols, op, eps);
  return launch_status();
}

extern "C" int nx_bk_rope_pairs(const float* x, float* y, int bh, int T, int half, int pos_offset, float theta,
                                nx_stream_t stream) {
  const int64_t pairs = static_cast<int64_t>(bh) * T * half;
  if (pairs <= 0) return 0;
  rope_pairs_kernel<<<blocks_for(pairs, 256), 256, 0, S(stream)>>>(x, y, pairs, T, half, pos_offset, theta);
  return launch_status();
}

extern "C" int nx_bk_swiglu_f32(const float* x, float* y, int rows, int hidden, nx_stream_t stream) {
  const int64_t n = static_cast<int64_t>(rows) * hidden;
  if (n <= 0) return 0;
  swiglu_f32_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(x, y, n, hidden);
  return launch_status();
}

extern "C" int nx_bk_adamw_step(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1,
                                float beta2, float eps, float weight_decay, float bc1, float bc2, nx_stream_t stream) {
  if (n <= 0) return 0;
  adamw_decay_in_lr_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(p, g, m, v, n, lr, beta1, beta2, eps,
                                                                      weight_decay, bc1, bc2);
  return launch_status();
}

extern "C" int nx_bk_quant_matmul(const float* a, const void* wq, const float* scales, float* c, int m, int n, int k,
                                  int group, int bits, nx_stream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || group <= 0 || k % group || (bits != 8 && bits != 4)) return -1;
  if (group % (bits == 8 ? 4 : 8)) return -1;
  const int blocks = (n + 7) / 8;
  if (bits == 8)
    quant_matmul_kernel<8><<<blocks, 256, 0, S(stream)>>>(a, static_cast<const uint32_t*>(wq), scales, c, m, n, k, group);
  else
    quant_matmul_kernel<4><<<blocks, 256, 0, S(stream)>>>(a, static_cast<const uint32_t*>(wq), scales, c, m, n, k, group);
  return launch_status();
}

extern "C" int nx_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t n, nx_stream_t stream) {
  if (n <= 0) return 0;
  if (src_dtype < 0 || src_dtype > NX_F16 || dst_dtype < 0 || dst_dtype > NX_F16) return -1;
  cast_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(src, src_dtype, dst, dst_dtype, n);
  return launch_status();
}

extern "C" int nx_fill(void* dst, int dtype, int64_t n, float value, nx_stream_t stream) {
  if (n <= 0) return 0;
  if (dtype < 0 || dtype > NX_F16) return -1;
  fill_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(dst, dtype, n, value);
  return launch_status();
}

extern "C" int nx_gelu(const void* x, const void* dy, void* out, int dtype, int64_t n, nx_stream_t stream) {
  if (n <= 0) return 0;
  if (dtype < 0 || dtype > NX_F16) return -1;
  gelu_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(x, dy, out, dtype, n);
  return launch_status();
}

extern "C" int nx_causal_softmax(const float* x, const float* dy, float* out, int64_t rows, int T, float scale,
                                 nx_stream_t stream) {
  if (rows <= 0 || T <= 0) return 0;
  causal_softmax_kernel<<<static_cast<unsigned>(rows), T >= 512 ? 256 : 64, 0, S(stream)>>>(x, dy, out, T, scale);
  return launch_status();
}

extern "C" int nx_split_heads(void* qkv, void* q, void* k, void* v, int B, int T, int H, int D, int merge,
                              nx_stream_t stream) {
  const int64_t n = static_cast<int64_t>(B) * T * H * D;
  if (n <= 0) return 0;
  split_heads_kernel<<<blocks_for(n, 256), 256, 0, S(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k),
      static_cast<__nv_bfloat16*>(v), B, T, H, D, merge);
  return launch_status();
}
