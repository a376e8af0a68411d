// The step right before routing, as one kernel each way: softmax over the gate logits, top-k expert ids written in
// the route-major int32 layout the routing kernel reads, and the GShard auxiliary loss
//     l = (1/T) sum_e mass_e * ce_e,   mass_e = sum_t softmax(logits)[t,e],   ce_e = (E/T) #{t : top-1(t) = e}
// (reference hexa_moe/impls/cascaded_moe.py:568-598, impls/layers.py:480-489, impls/losses.py:12-19), plus the
// gradient of l with respect to the logits.  The [T,E] score matrix is never written: the backward kernel
// recomputes the softmax from the logits it has to read anyway.
//
// One warp per token, lane l holding columns l, l+32, ...; column sums stay in registers across the tokens of a
// warp, meet in shared memory once per block (one row per warp, added in warp order) and leave the block as one
// partial row in the workspace; the block that finishes last adds the partial rows in block order.  Every float
// sum therefore has a fixed order: mass and loss are bit-identical from run to run.  The only atomics are the
// integer top-1 histogram and the completion ticket.
// Ties: the lowest expert id wins, and the k ids of a token come out in descending score order.  The selection is
// total: a score that is NaN ranks below every number, so a row of NaN / inf logits (an overflowed fp16 step) still
// yields k distinct ids in [0, E) - the lowest free columns - and only the loss carries the NaN, as it does through
// F.softmax -> torch.topk in the reference.
#include <float.h>

#include "hexa_common.cuh"

namespace hexa {
namespace {

constexpr int kGateThreads = 256;
constexpr int kGateWarps = kGateThreads / 32;
constexpr int kGateMaxExperts = 512;
constexpr int kGateMaxBlocks = 1024;   // partial-mass rows the workspace holds
constexpr size_t kGateTicketBytes = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// softmax of one token's logits, spread over the warp; columns >= E come out as 0
template <int VPT>
__device__ __forceinline__ void warp_softmax(const float* __restrict__ row, int E, int lane, float (&s)[VPT]) {
  float m = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    s[i] = c < E ? __ldg(row + c) : -FLT_MAX;
    m = fmaxf(m, s[i]);
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    s[i] = (lane + 32 * i) < E ? expf(s[i] - m) : 0.f;
    sum += s[i];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int i = 0; i < VPT; ++i) s[i] = s[i] / sum;
}

template <int VPT>
__global__ void __launch_bounds__(kGateThreads)
gate_topk_kernel(const float* __restrict__ logits, int64_t ld, int64_t T, int E, int k, int32_t* __restrict__ ids,
                 float* __restrict__ mass, int32_t* __restrict__ first_count, float* __restrict__ loss,
                 unsigned int* __restrict__ ticket, float* __restrict__ partial) {
  __shared__ float mass_w[kGateWarps][32 * VPT];
  __shared__ int cnt_s[32 * VPT];
  __shared__ float red_s[kGateWarps];
  __shared__ bool last_s;
  for (int e = threadIdx.x; e < 32 * VPT; e += blockDim.x) cnt_s[e] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * kGateWarps + warp;
  const int64_t nwarps = (int64_t)gridDim.x * kGateWarps;
  float acc[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) acc[i] = 0.f;
  for (int64_t t = warp0; t < T; t += nwarps) {
    float s[VPT];
    warp_softmax<VPT>(logits + t * ld, E, lane, s);
#pragma unroll
    for (int i = 0; i < VPT; ++i) acc[i] += s[i];
    unsigned int taken = 0;
    for (int j = 0; j < k; ++j) {
      // candidates: this lane's free columns; NaN counts as -inf, and the first free column is taken even at -inf,
      // so some lane always has a candidate while fewer than E columns are taken (k <= E is checked by the host)
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = lane + 32 * i;
        if (c < E && !((taken >> i) & 1u)) {
          const float v = s[i] == s[i] ? s[i] : -INFINITY;
          if (bi == 0x7fffffff || v > best) { best = v; bi = c; }   // ascending c: the first maximum stays
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      const bool valid = (unsigned)bi < (unsigned)E;     // always true; kept so that no index derived from data is trusted
      if (valid && (bi & 31) == lane) taken |= 1u << (bi >> 5);
      if (lane == 0) {
        ids[(int64_t)j * T + t] = valid ? bi : -1;         // -1 is a row the routing kernel skips
        if (j == 0 && valid) atomicAdd(&cnt_s[bi], 1);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) mass_w[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float m = 0.f;
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) m += mass_w[w][e];
    partial[(int64_t)blockIdx.x * E + e] = m;
    if (cnt_s[e]) atomicAdd(&first_count[e], cnt_s[e]);
  }
  // the block that finishes last adds the partial rows (in block order) and folds the two [E] vectors into the loss
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  float part = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float m = 0.f;
    for (unsigned b = 0; b < gridDim.x; ++b) m += __ldcg(partial + (int64_t)b * E + e);
    mass[e] = m;
    part += m * (float)__ldcg(first_count + e);
  }
  // fixed-order block reduction: lanes by xor tree, warps in index order
  part = warp_sum(part);
  if (lane == 0) red_s[warp] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < kGateWarps; ++w) tot += red_s[w];
    loss[0] = tot * ((float)E / (float)T) / (float)T;
  }
}

// dlogits[t,e] = s[t,e] * (g_e - sum_e' s[t,e'] g_e') with g_e = dloss * ce_e / T: the chain rule through
// mass = column sums of the softmax (ce counts top-1 choices and carries no gradient)
template <int VPT>
__global__ void __launch_bounds__(kGateThreads)
gate_loss_grad_kernel(const float* __restrict__ logits, int64_t ld, int64_t T, int E, const int32_t* __restrict__ first_count,
                      const float* __restrict__ dloss, float* __restrict__ dlogits, int64_t ldd) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * (kGateThreads / 32) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (kGateThreads / 32);
  const float scale = __ldg(dloss) * ((float)E / (float)T) / (float)T;
  float g[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    g[i] = c < E ? scale * (float)__ldg(first_count + c) : 0.f;
  }
  for (int64_t t = warp0; t < T; t += nwarps) {
    float s[VPT];
    warp_softmax<VPT>(logits + t * ld, E, lane, s);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) dot += s[i] * g[i];
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < E) dlogits[t * ldd + c] = s[i] * (g[i] - dot);
    }
  }
}

int gate_grid(int64_t T) {
  const int64_t want = ceil_div(T, kGateThreads / 32);
  int64_t cap = (int64_t)sm_count() * 4;
  if (cap > kGateMaxBlocks) cap = kGateMaxBlocks;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace
}  // namespace hexa

using namespace hexa;

extern "C" int hexa_gate_max_experts(void) { return kGateMaxExperts; }

extern "C" size_t hexa_gate_workspace_bytes(void) {
  return kGateTicketBytes + (size_t)kGateMaxBlocks * kGateMaxExperts * sizeof(float);   // ticket + partial-mass rows (2 MiB)
}

extern "C" int hexa_gate_topk(const float* logits, int64_t ld, int64_t num_tokens, int num_experts, int top_k, int32_t* ids,
                              float* mass, int32_t* first_count, float* loss, void* workspace, size_t workspace_bytes,
                              void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HEXA_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= kGateMaxExperts, "hexa_gate_topk: needs 1 <= experts <= %d (got %d)",
               kGateMaxExperts, num_experts);
  HEXA_REQUIRE(top_k >= 1 && top_k <= num_experts, "hexa_gate_topk: top_k %d out of range for %d experts", top_k, num_experts);
  HEXA_REQUIRE(mass && first_count && loss && workspace && workspace_bytes >= hexa_gate_workspace_bytes(),
               "hexa_gate_topk: null output or workspace smaller than hexa_gate_workspace_bytes()");
  HEXA_REQUIRE(num_tokens == 0 || (logits && ids && ld >= num_experts), "hexa_gate_topk: null logits/ids or ld < experts");
  HEXA_REQUIRE(aligned16(workspace), "hexa_gate_topk: workspace must be 16-byte aligned");
  HEXA_CUDA(cudaMemsetAsync(mass, 0, sizeof(float) * num_experts, stream));
  HEXA_CUDA(cudaMemsetAsync(first_count, 0, sizeof(int32_t) * num_experts, stream));
  HEXA_CUDA(cudaMemsetAsync(loss, 0, sizeof(float), stream));
  HEXA_CUDA(cudaMemsetAsync(workspace, 0, 16, stream));
  if (num_tokens == 0) return HEXA_OK;
  unsigned int* ticket = static_cast<unsigned int*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kGateTicketBytes);
  const int grid = gate_grid(num_tokens);
#define HEXA_GATE_FWD(V) \
  gate_topk_kernel<V><<<grid, kGateThreads, 0, stream>>>(logits, ld, num_tokens, num_experts, top_k, ids, mass, first_count, loss, ticket, partial)
  const int vpt = (num_experts + 31) / 32;
  if (vpt <= 1) HEXA_GATE_FWD(1);
  else if (vpt <= 2) HEXA_GATE_FWD(2);
  else if (vpt <= 4) HEXA_GATE_FWD(4);
  else if (vpt <= 8) HEXA_GATE_FWD(8);
  else HEXA_GATE_FWD(16);
#undef HEXA_GATE_FWD
  HEXA_LAUNCH_CHECK("gate_topk_kernel");
  return HEXA_OK;
}

extern "C" int hexa_gate_loss_grad(const float* logits, int64_t ld, int64_t num_tokens, int num_experts,
                                   const int32_t* first_count, const float* dloss, float* dlogits, int64_t ldd, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HEXA_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= kGateMaxExperts, "hexa_gate_loss_grad: needs 1 <= experts <= %d (got %d)",
               kGateMaxExperts, num_experts);
  if (num_tokens == 0) return HEXA_OK;
  HEXA_REQUIRE(logits && first_count && dloss && dlogits && ld >= num_experts && ldd >= num_experts,
               "hexa_gate_loss_grad: null pointer or leading dimension < experts");
  const int grid = gate_grid(num_tokens);
#define HEXA_GATE_BWD(V) \
  gate_loss_grad_kernel<V><<<grid, kGateThreads, 0, stream>>>(logits, ld, num_tokens, num_experts, first_count, dloss, dlogits, ldd)
  const int vpt = (num_experts + 31) / 32;
  if (vpt <= 1) HEXA_GATE_BWD(1);
  else if (vpt <= 2) HEXA_GATE_BWD(2);
  else if (vpt <= 4) HEXA_GATE_BWD(4);
  else if (vpt <= 8) HEXA_GATE_BWD(8);
  else HEXA_GATE_BWD(16);
#undef HEXA_GATE_BWD
  HEXA_LAUNCH_CHECK("gate_loss_grad_kernel");
  return HEXA_OK;
}
