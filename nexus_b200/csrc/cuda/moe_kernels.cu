// Mixture-of-experts routing on the GPU: top-k selection with the gate softmax over the selected
// experts (FP32 router logits in), capacity assignment in priority order (choice j first, then token
// index: a per-expert counting sort, deterministic), and the gate gradient of the combine step.
// Tokens are then gathered into per-expert [capacity, d] buffers and combined by the dispatch / combine
// kernels (which also serve expert parallelism over peer memory); the expert FFN itself is a strided
// batched tcgen05 GEMM over the padded buffers.
// Parity: src/moe/moe.cpp (router, capacity, permutation) of the reference, which runs on the CPU.
#include "common.cuh"
#include "nx_api_moe.h"

namespace {
using namespace nx;

// warp per token; E <= 1024; k <= 8
__global__ void moe_topk_kernel(const float* __restrict__ logits, int tokens, int E, int k,
                                int32_t* __restrict__ expert, float* __restrict__ gate) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const float* row = logits + static_cast<int64_t>(t) * E;
  float sel_v[8];
  int sel_i[8];
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      bool taken = false;
      for (int q = 0; q < j; ++q) taken |= sel_i[q] == e;
      const float v = row[e];
      if (!taken && (v > best || (v == best && e < bi))) {
        best = v;
        bi = e;
      }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    sel_v[j] = best;
    sel_i[j] = bi;
  }
  if (lane == 0) {
    float mx = sel_v[0], se = 0.0f;
    for (int j = 0; j < k; ++j) se += expf(sel_v[j] - mx);
    for (int j = 0; j < k; ++j) {
      expert[t * k + j] = sel_i[j];
      gate[t * k + j] = expf(sel_v[j] - mx) / se;
    }
  }
}

// One block per expert.  Entries are visited in priority order p = j * tokens + t; entry (t, j) of this
// expert gets slot = number of earlier entries of the same expert, or -1 beyond the capacity.
__global__ void __launch_bounds__(1024)
moe_assign_kernel(const int32_t* __restrict__ expert, int tokens, int k, int capacity, int32_t* __restrict__ slot,
                  int32_t* __restrict__ counts, int32_t* __restrict__ dropped) {
  __shared__ int s_warp[32];
  __shared__ int s_run;
  const int e = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_run = 0;
  __syncthreads();
  const int total = tokens * k;
  int ndrop = 0;
  for (int base = 0; base < total; base += blockDim.x) {
    const int p = base + threadIdx.x;
    int t = 0, j = 0;
    bool mine = false;
    if (p < total) {
      j = p / tokens;
      t = p % tokens;
      mine = expert[t * k + j] == e;
    }
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    const int within = __popc(ballot & ((1u << lane) - 1));
    if (lane == 0) s_warp[warp] = __popc(ballot);
    __syncthreads();
    int before = s_run;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    if (mine) {
      const int s = before + within;
      const bool ok = s < capacity;
      slot[t * k + j] = ok ? s : -1;
      ndrop += ok ? 0 : 1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int sum = 0;
      for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) sum += s_warp[w];
      s_run += sum;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = min(s_run, capacity);
  if (dropped != nullptr && ndrop > 0) atomicAdd(dropped, ndrop);
}

// Capacity per GROUP of tokens and the Reroute overflow policy.  One warp per group walks the group's assignments in
// priority order (choice j, then token t) with the per-expert fill counters in shared memory: an assignment whose
// expert is full is dropped (slot -1) or, with `order` given ([tokens, E]: every token's experts by descending
// score), moved to the token's best expert that still has room and is not one of the token's own choices; the lanes
// test 32 candidates per trip.  slot = group * capacity + position inside the group's share of the expert's buffer,
// so the buffers are [E, groups * capacity, d].  counts[g * E + e] = rows of group g accepted by expert e.
__global__ void __launch_bounds__(32)
moe_assign_groups_kernel(int32_t* __restrict__ expert, const int32_t* __restrict__ order, int tokens, int k, int E,
                         int groups, int capacity, int32_t* __restrict__ slot, int32_t* __restrict__ counts,
                         int32_t* __restrict__ dropped, int32_t* __restrict__ rerouted) {
  extern __shared__ int s_fill[];  // [E]
  const int g = blockIdx.x, lane = threadIdx.x;
  const int ng = tokens / groups, t0 = g * ng;
  for (int e = lane; e < E; e += 32) s_fill[e] = 0;
  __syncwarp();
  int ndrop = 0, nmove = 0;
  for (int j = 0; j < k; ++j) {
    for (int t = t0; t < t0 + ng; ++t) {
      int e = expert[t * k + j];
      bool full = s_fill[e] >= capacity;
      if (full && order != nullptr) {
        int alt = -1;
        for (int c0 = 0; c0 < E && alt < 0; c0 += 32) {
          const int c = c0 + lane;
          bool ok = false;
          int cand = -1;
          if (c < E) {
            cand = order[static_cast<int64_t>(t) * E + c];
            ok = s_fill[cand] < capacity;
            for (int q = 0; q < k; ++q) ok = ok && expert[t * k + q] != cand;
          }
          const unsigned b = __ballot_sync(0xffffffffu, ok);
          if (b != 0u) alt = __shfl_sync(0xffffffffu, cand, __ffs(b) - 1);
        }
        if (alt >= 0) {
          e = alt;
          full = false;
          ++nmove;
          if (lane == 0) expert[t * k + j] = e;
        }
      }
      if (lane == 0) {
        slot[t * k + j] = full ? -1 : g * capacity + s_fill[e];
        if (!full) s_fill[e] += 1;
      }
      ndrop += full ? 1 : 0;
      __syncwarp();
    }
  }
  for (int e = lane; e < E; e += 32) counts[g * E + e] = s_fill[e];
  if (lane == 0) {
    if (dropped != nullptr && ndrop > 0) atomicAdd(dropped, ndrop);
    if (rerouted != nullptr && nmove > 0) atomicAdd(rerouted, nmove);
  }
}

// dgate[t, j] = dy[t] . expert_out[e_tj][slot_tj]   (0 for dropped assignments); warp per (t, j)
__global__ void moe_gate_grad_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ buf,
                                     const int32_t* __restrict__ expert, const int32_t* __restrict__ slot,
                                     float* __restrict__ dgate, int entries, int k, int d, int capacity) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (i >= entries) return;
  const int s = slot[i];
  float acc = 0.0f;
  if (s >= 0) {
    const __nv_bfloat16* a = dy + static_cast<int64_t>(i / k) * d;
    const __nv_bfloat16* b = buf + (static_cast<int64_t>(expert[i]) * capacity + s) * d;
    for (int c = lane * 2; c < d; c += 64) {
      const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(a + c);
      const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(b + c);
      acc += __low2float(x) * __low2float(y) + __high2float(x) * __high2float(y);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dgate[i] = acc;
}
}  // namespace

extern "C" int nx_moe_topk(const float* logits, int tokens, int experts, int k, int32_t* expert, float* gate,
                           nx_stream_t stream) {
  if (tokens <= 0) return 0;
  if (k < 1 || k > 8 || k > experts || experts > 1024) return -1;
  moe_topk_kernel<<<(tokens + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(logits, tokens, experts, k, expert, gate);
  return launch_status();
}

extern "C" int nx_moe_assign(const int32_t* expert, int tokens, int k, int experts, int capacity, int32_t* slot,
                             int32_t* counts, int32_t* dropped, nx_stream_t stream) {
  if (tokens <= 0 || experts <= 0) return 0;
  if (capacity < 0) return -1;
  moe_assign_kernel<<<experts, 1024, 0, static_cast<cudaStream_t>(stream)>>>(expert, tokens, k, capacity, slot, counts, dropped);
  return launch_status();
}

extern "C" int nx_moe_assign_groups(int32_t* expert, const int32_t* order, int tokens, int k, int experts, int groups,
                                    int capacity, int32_t* slot, int32_t* counts, int32_t* dropped, int32_t* rerouted,
                                    nx_stream_t stream) {
  if (tokens <= 0 || experts <= 0) return 0;
  if (groups < 1 || tokens % groups || capacity < 0 || k < 1 || k > 8 || experts > 8192) return -1;
  moe_assign_groups_kernel<<<groups, 32, experts * sizeof(int), static_cast<cudaStream_t>(stream)>>>(
      expert, order, tokens, k, experts, groups, capacity, slot, counts, dropped, rerouted);
  return launch_status();
}

extern "C" int nx_moe_gate_grad(const void* dy, const void* expert_out, const int32_t* expert, const int32_t* slot,
                                float* dgate, int tokens, int k, int d, int capacity, nx_stream_t stream) {
  const int entries = tokens * k;
  if (entries <= 0) return 0;
  if (d & 1) return -1;
  moe_gate_grad_kernel<<<(entries + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(expert_out), expert, slot, dgate, entries,
      k, d, capacity);
  return launch_status();
}
