// Shared host/device helpers for the hexa_moe_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hexa_moe_b200.h"

namespace hexa {

// ---- host-side error plumbing -----------------------------------------------------------------
void set_error(const char* fmt, ...);
int32_t* status_word();   // status word of the current device (may be null), see hexa_set_status_word
int status_pending();     // code an earlier kernel left in the current device's status word, when the host can read it (else 0)
uint64_t wait_limit_ns(); // limit of the bounded waits inside kernels, see hexa_set_wait_limit_ns
int tc_debug_flags();     // HEXA_TC_DEBUG / hexa_set_tc_debug

// Entry points that launch kernels with bounded waits refuse to run once such a wait has been given up on this
// device: what those kernels wrote is incomplete, and so is everything computed from it.
#define HEXA_CHECK_DEVICE_STATUS(name)                                                                     \
  do {                                                                                                     \
    const int code_ = ::hexa::status_pending();                                                            \
    if (code_ != 0) {                                                                                      \
      ::hexa::set_error("%s: an earlier kernel on this device gave up a bounded wait (status code %d); "   \
                        "its outputs are incomplete.  Clear the status word to continue", name, code_);    \
      return HEXA_ERR_DEVICE;                                                                              \
    }                                                                                                      \
  } while (0)

#define HEXA_REQUIRE(cond, ...)          \
  do {                                   \
    if (!(cond)) {                       \
      ::hexa::set_error(__VA_ARGS__);    \
      return HEXA_ERR_INVALID;           \
    }                                    \
  } while (0)

#define HEXA_CUDA(call)                                                              \
  do {                                                                               \
    cudaError_t e_ = (call);                                                         \
    if (e_ != cudaSuccess) {                                                         \
      ::hexa::set_error("%s failed: %s", #call, cudaGetErrorString(e_));             \
      return HEXA_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)

#define HEXA_LAUNCH_CHECK(name)                                                      \
  do {                                                                               \
    cudaError_t e_ = cudaGetLastError();                                             \
    if (e_ != cudaSuccess) {                                                         \
      ::hexa::set_error("launch of %s failed: %s", name, cudaGetErrorString(e_));    \
      return HEXA_ERR_CUDA;                                                          \
    }                                                                                \
  } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t dtype_size(int dt) { return dt == HEXA_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int sm_count();  // SMs of the current device (cached per device)
int sm_limit();  // upper bound on the SMs persistent kernels may occupy (0 = all), see hexa_set_sm_limit

constexpr int kRowTile = 128;  // rows per GEMM tile == required segment alignment of the GEMM operators

// ---- device-side scalar conversion ------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- activations (value and derivative), shared by every epilogue ------------------------------
__device__ __forceinline__ float act_apply(int act, float x) {
  switch (act) {
    case HEXA_ACT_RELU: return x > 0.f ? x : 0.f;
    case HEXA_ACT_GELU: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case HEXA_ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case HEXA_ACT_SILU: return x / (1.f + expf(-x));
    default: return x;
  }
}

__device__ __forceinline__ float act_grad(int act, float x) {
  switch (act) {
    case HEXA_ACT_RELU: return x > 0.f ? 1.f : 0.f;
    case HEXA_ACT_GELU: {
      float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
      float pdf = 0.3989422804014327f * expf(-0.5f * x * x);
      return cdf + x * pdf;
    }
    case HEXA_ACT_GELU_TANH: {
      float x2 = x * x;
      float u = 0.7978845608028654f * (x + 0.044715f * x * x2);
      float t = tanhf(u);
      float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
    }
    case HEXA_ACT_SILU: {
      float s = 1.f / (1.f + expf(-x));
      return s * (1.f + x * (1.f - s));
    }
    default: return 1.f;
  }
}

// ---- fast variants for 16-bit epilogues -----------------------------------------------------------
// Accurate to ~2e-7 absolute, far below bf16/fp16 resolution, at roughly a third of the instructions
// of erff/expf: erf by Abramowitz-Stegun 7.1.26 (one reciprocal, one exp2, a degree-5 Horner), with
// exp(-x^2/2) shared between the Gaussian CDF and PDF.  ACT is a compile-time HEXA_ACT_* id.
__device__ __forceinline__ float rcp_fast(float x) {   // one MUFU.RCP, ~1 ulp; __frcp_rn would add a Newton step
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float ex2_fast(float x) {   // one MUFU.EX2
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// u = (1 - erf(|x| / sqrt2)) / 2 = the Gaussian tail mass beyond |x|, e = exp(-x^2 / 2).  The 1/sqrt2 of the erf
// argument and the final 1/2 are folded into the constants.
__device__ __forceinline__ void gelu_parts(float x, float& u, float& e) {
  e = ex2_fast(x * x * -0.72134752044448170f);            // exp(-x^2/2) = 2^(-x^2 / (2 ln 2))
  const float t = rcp_fast(fmaf(0.3275911f * 0.70710678118654752f, fabsf(x), 1.0f));
  float q = fmaf(0.5f * 1.061405429f, t, 0.5f * -1.453152027f);
  q = fmaf(q, t, 0.5f * 1.421413741f);
  q = fmaf(q, t, 0.5f * -0.284496736f);
  q = fmaf(q, t, 0.5f * 0.254829592f);
  u = q * t * e;
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int ACT> __device__ __forceinline__ float act_fast(float x) {
  if (ACT == HEXA_ACT_RELU) return fmaxf(x, 0.f);
  if (ACT == HEXA_ACT_GELU) {
    // x Phi(x) with Phi = 1 - u for x >= 0 and u for x < 0: both cases are max(x, 0) - |x u|, no compare or select
    float u, e;
    gelu_parts(x, u, e);
    return fmaxf(x, 0.f) - fabsf(x * u);
  }
  if (ACT == HEXA_ACT_GELU_TANH) return 0.5f * x * (1.f + tanh_fast(0.7978845608028654f * fmaf(0.044715f * x * x, x, x)));
  if (ACT == HEXA_ACT_SILU) return x * rcp_fast(1.f + __expf(-x));
  return x;
}
template <int ACT> __device__ __forceinline__ float act_grad_fast(float x) {
  if (ACT == HEXA_ACT_RELU) return x > 0.f ? 1.f : 0.f;
  if (ACT == HEXA_ACT_GELU) {   // Phi(x) + x phi(x)
    float u, e;
    gelu_parts(x, u, e);
    return fmaf(x * e, 0.3989422804014327f, x >= 0.f ? 1.0f - u : u);
  }
  if (ACT == HEXA_ACT_GELU_TANH) {
    const float x2 = x * x;
    const float t = tanh_fast(0.7978845608028654f * fmaf(0.044715f * x2, x, x));
    const float du = 0.7978845608028654f * fmaf(3.f * 0.044715f, x2, 1.f);
    return fmaf(0.5f * x * (1.f - t * t), du, 0.5f * (1.f + t));
  }
  if (ACT == HEXA_ACT_SILU) { const float sg = rcp_fast(1.f + __expf(-x)); return sg * fmaf(x, 1.f - sg, 1.f); }
  return 1.f;
}

}  // namespace hexa
