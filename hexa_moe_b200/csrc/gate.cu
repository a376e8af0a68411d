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


// ---- the load-importance loss (reference impls/losses.py:21-43) -------------------------------------------------------
//   importance_e = sum_t softmax(logits)[t,e]                          (clean logits)
//   load_e       = sum_t Phi((softmax(logits)[t,e] - thr_t) / sigma)   thr_t = the k-th largest NOISY logit of token t,
//                                                                      sigma = gate_noise / E  (the reference compares a
//                                                                      score with a logit: kept as it is)
//   loss         = (cv2(importance) + cv2(load)) / 2,   cv2(v) = var(v) / (mean(v)^2 + 1e-10), var unbiased
// The top-k ids are those of the noisy logits (softmax is monotonic, so they equal torch.topk of softmax(noisy)).
__device__ __forceinline__ float normal_cdf(float z) { return 0.5f * (1.f + erff(z * 0.70710678118654752f)); }

// k-th pick of one token's noisy logits held as v[VPT] per lane; writes the ids, returns the last picked value.
template <int VPT>
__device__ __forceinline__ float warp_topk(const float (&v)[VPT], int E, int k, int lane, int32_t* __restrict__ ids, int64_t T,
                                           int64_t t, int* last_id) {
  unsigned int taken = 0;
  float thr = 0.f;
  int bi_last = 0;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < E && !((taken >> i) & 1u)) {
        const float x = v[i] == v[i] ? v[i] : -INFINITY;
        if (bi == 0x7fffffff || x > best) { best = x; bi = c; }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const bool valid = (unsigned)bi < (unsigned)E;
    if (valid && (bi & 31) == lane) taken |= 1u << (bi >> 5);
    if (lane == 0 && ids) ids[(int64_t)j * T + t] = valid ? bi : -1;
    thr = best;
    bi_last = valid ? bi : -1;
  }
  *last_id = bi_last;
  return thr;
}

// cv2 of an [E] vector and its gradient factors, computed by one warp (every warp that needs them recomputes them:
// E <= 512 values).  Returns mean and var through references.
__device__ __forceinline__ void warp_mean_var(const float* __restrict__ v, int E, int lane, float& mean, float& var) {
  float s = 0.f;
  for (int e = lane; e < E; e += 32) s += __ldcg(v + e);
  mean = warp_sum(s) / (float)E;
  float q = 0.f;
  for (int e = lane; e < E; e += 32) { const float d = __ldcg(v + e) - mean; q += d * d; }
  var = warp_sum(q) / (float)(E - 1);
}

template <int VPT>
__global__ void __launch_bounds__(kGateThreads)
gate_topk_li_kernel(const float* __restrict__ logits, const float* __restrict__ noisy, int64_t ld, int64_t T, int E, int k,
                    float inv_sigma, int32_t* __restrict__ ids, float* __restrict__ importance, float* __restrict__ load,
                    float* __restrict__ loss, unsigned int* __restrict__ ticket, float* __restrict__ partial) {
  __shared__ float sum_w[kGateWarps][2 * 32 * VPT];
  __shared__ bool last_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t warp0 = (int64_t)blockIdx.x * kGateWarps + warp;
  const int64_t nwarps = (int64_t)gridDim.x * kGateWarps;
  float imp[VPT], ld_acc[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) { imp[i] = 0.f; ld_acc[i] = 0.f; }
  for (int64_t t = warp0; t < T; t += nwarps) {
    float s[VPT], v[VPT];
    warp_softmax<VPT>(logits + t * ld, E, lane, s);
#pragma unroll
    for (int i = 0; i < VPT; ++i) { const int c = lane + 32 * i; v[i] = c < E ? __ldg(noisy + t * ld + c) : -INFINITY; }
    int last_id;
    const float thr = warp_topk<VPT>(v, E, k, lane, ids, T, t, &last_id);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (lane + 32 * i < E) { imp[i] += s[i]; ld_acc[i] += normal_cdf((s[i] - thr) * inv_sigma); }
    }
  }
#pragma unroll
  for (int i = 0; i < VPT; ++i) { sum_w[warp][lane + 32 * i] = imp[i]; sum_w[warp][32 * VPT + lane + 32 * i] = ld_acc[i]; }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {       // per-block partial rows, warps added in index order
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int w = 0; w < kGateWarps; ++w) { a += sum_w[w][e]; b += sum_w[w][32 * VPT + e]; }
    partial[(int64_t)blockIdx.x * 2 * E + e] = a;
    partial[(int64_t)blockIdx.x * 2 * E + E + e] = b;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = atomicAdd(ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {       // blocks added in index order
    float a = 0.f, b = 0.f;
    for (unsigned blk = 0; blk < gridDim.x; ++blk) {
      a += __ldcg(partial + (int64_t)blk * 2 * E + e);
      b += __ldcg(partial + (int64_t)blk * 2 * E + E + e);
    }
    importance[e] = a;
    load[e] = b;
  }
  __threadfence();
  __syncthreads();
  if (warp == 0) {
    float mi, vi, ml, vl;
    warp_mean_var(importance, E, lane, mi, vi);
    warp_mean_var(load, E, lane, ml, vl);
    if (lane == 0) loss[0] = 0.5f * (vi / (mi * mi + 1e-10f) + vl / (ml * ml + 1e-10f));
  }
}

// d loss / d logits for gate_topk_li_kernel's loss, times dloss[0].  With g_i = d loss / d importance and g_l = d loss /
// d load (from the forward's totals), pdf_e = phi(z_e) / sigma:
//   d s_e = g_i[e] + g_l[e] pdf_e ;  d thr = - sum_e g_l[e] pdf_e  (reaches the clean logit of the k-th choice: the noise is a constant)
//   d logits_e = s_e (d s_e - sum_e' s_e' d s_e') + [e = k-th choice] d thr
template <int VPT>
__global__ void __launch_bounds__(kGateThreads)
gate_li_grad_kernel(const float* __restrict__ logits, const float* __restrict__ noisy, int64_t ld, int64_t T, int E, int k,
                    float inv_sigma, const float* __restrict__ importance, const float* __restrict__ load,
                    const float* __restrict__ dloss, float* __restrict__ dlogits, int64_t ldd) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kGateWarps + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * kGateWarps;
  float mi, vi, ml, vl;
  warp_mean_var(importance, E, lane, mi, vi);
  warp_mean_var(load, E, lane, ml, vl);
  const float up = 0.5f * __ldg(dloss);
  const float di = mi * mi + 1e-10f, dl = ml * ml + 1e-10f;
  float gi[VPT], gl[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + 32 * i;
    // d cv2 / d v_e = 2 (v_e - mean) / ((E-1) den) - var * 2 mean / (E den^2)
    gi[i] = c < E ? up * (2.f * (__ldg(importance + c) - mi) / ((float)(E - 1) * di) - vi * 2.f * mi / ((float)E * di * di)) : 0.f;
    gl[i] = c < E ? up * (2.f * (__ldg(load + c) - ml) / ((float)(E - 1) * dl) - vl * 2.f * ml / ((float)E * dl * dl)) : 0.f;
  }
  for (int64_t t = warp0; t < T; t += nwarps) {
    float s[VPT], v[VPT];
    warp_softmax<VPT>(logits + t * ld, E, lane, s);
#pragma unroll
    for (int i = 0; i < VPT; ++i) { const int c = lane + 32 * i; v[i] = c < E ? __ldg(noisy + t * ld + c) : -INFINITY; }
    int last_id;
    const float thr = warp_topk<VPT>(v, E, k, lane, nullptr, T, t, &last_id);
    float ds[VPT];
    float dthr = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const float z = (s[i] - thr) * inv_sigma;
      const float pdf = (lane + 32 * i) < E ? 0.3989422804014327f * expf(-0.5f * z * z) * inv_sigma : 0.f;
      ds[i] = gi[i] + gl[i] * pdf;
      dthr -= gl[i] * pdf;
      dot += s[i] * ds[i];
    }
    dthr = warp_sum(dthr);
    dot = warp_sum(dot);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + 32 * i;
      if (c < E) dlogits[t * ldd + c] = s[i] * (ds[i] - dot) + (c == last_id ? dthr : 0.f);
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

extern "C" int hexa_gate_topk_load_importance(const float* logits, const float* logits_w_noise, int64_t ld, int64_t num_tokens,
                                              int num_experts, int top_k, float sigma, int32_t* ids, float* importance,
                                              float* load, float* loss, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HEXA_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= kGateMaxExperts,
               "hexa_gate_topk_load_importance: needs 1 <= experts <= %d (got %d)", kGateMaxExperts, num_experts);
  HEXA_REQUIRE(top_k >= 1 && top_k <= num_experts, "hexa_gate_topk_load_importance: top_k %d out of range for %d experts", top_k, num_experts);
  HEXA_REQUIRE(sigma > 0.f, "hexa_gate_topk_load_importance: sigma (gate_noise / experts) must be > 0");
  HEXA_REQUIRE(importance && load && loss && workspace && workspace_bytes >= hexa_gate_workspace_bytes() && aligned16(workspace),
               "hexa_gate_topk_load_importance: null output, or workspace smaller than hexa_gate_workspace_bytes() or not 16-byte aligned");
  HEXA_REQUIRE(num_tokens == 0 || (logits && logits_w_noise && ids && ld >= num_experts),
               "hexa_gate_topk_load_importance: null logits/ids or ld < experts");
  HEXA_CUDA(cudaMemsetAsync(importance, 0, sizeof(float) * num_experts, stream));
  HEXA_CUDA(cudaMemsetAsync(load, 0, sizeof(float) * num_experts, stream));
  HEXA_CUDA(cudaMemsetAsync(loss, 0, sizeof(float), stream));
  HEXA_CUDA(cudaMemsetAsync(workspace, 0, 16, stream));
  if (num_tokens == 0) return HEXA_OK;
  unsigned int* ticket = static_cast<unsigned int*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kGateTicketBytes);
  int grid = gate_grid(num_tokens);
  if (grid > kGateMaxBlocks / 2) grid = kGateMaxBlocks / 2;      // two partial rows per block
  const float inv_sigma = 1.f / sigma;
#define HEXA_GATE_LI(V)                                                                                                     \
  gate_topk_li_kernel<V><<<grid, kGateThreads, 0, stream>>>(logits, logits_w_noise, ld, num_tokens, num_experts, top_k, inv_sigma, \
                                                            ids, importance, load, loss, ticket, partial)
  const int vpt = (num_experts + 31) / 32;
  if (vpt <= 1) HEXA_GATE_LI(1);
  else if (vpt <= 2) HEXA_GATE_LI(2);
  else if (vpt <= 4) HEXA_GATE_LI(4);
  else if (vpt <= 8) HEXA_GATE_LI(8);
  else HEXA_GATE_LI(16);
#undef HEXA_GATE_LI
  HEXA_LAUNCH_CHECK("gate_topk_li_kernel");
  return HEXA_OK;
}

extern "C" int hexa_gate_load_importance_grad(const float* logits, const float* logits_w_noise, int64_t ld, int64_t num_tokens,
                                              int num_experts, int top_k, float sigma, const float* importance, const float* load,
                                              const float* dloss, float* dlogits, int64_t ldd, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HEXA_REQUIRE(num_tokens >= 0 && num_experts >= 1 && num_experts <= kGateMaxExperts,
               "hexa_gate_load_importance_grad: needs 1 <= experts <= %d (got %d)", kGateMaxExperts, num_experts);
  HEXA_REQUIRE(top_k >= 1 && top_k <= num_experts && sigma > 0.f, "hexa_gate_load_importance_grad: bad top_k or sigma");
  if (num_tokens == 0) return HEXA_OK;
  HEXA_REQUIRE(logits && logits_w_noise && importance && load && dloss && dlogits && ld >= num_experts && ldd >= num_experts,
               "hexa_gate_load_importance_grad: null pointer or leading dimension < experts");
  const int grid = gate_grid(num_tokens);
  const float inv_sigma = 1.f / sigma;
#define HEXA_GATE_LIG(V)                                                                                                     \
  gate_li_grad_kernel<V><<<grid, kGateThreads, 0, stream>>>(logits, logits_w_noise, ld, num_tokens, num_experts, top_k, inv_sigma, \
                                                            importance, load, dloss, dlogits, ldd)
  const int vpt = (num_experts + 31) / 32;
  if (vpt <= 1) HEXA_GATE_LIG(1);
  else if (vpt <= 2) HEXA_GATE_LIG(2);
  else if (vpt <= 4) HEXA_GATE_LIG(4);
  else if (vpt <= 8) HEXA_GATE_LIG(8);
  else HEXA_GATE_LIG(16);
#undef HEXA_GATE_LIG
  HEXA_LAUNCH_CHECK("gate_li_grad_kernel");
  return HEXA_OK;
}
