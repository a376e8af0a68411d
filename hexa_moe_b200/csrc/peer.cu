// Building blocks for collectives that run on copy engines and stream memory operations instead of SMs:
//   hexa_stream_wait_value   the stream waits until a 32-bit word in device memory is >= a value (written by a peer's
//                            copy over NVLink); with one word per peer this is an SM-free barrier between ranks
//   hexa_mean_slices         out = (local + sum of n received slices) / world, fp32 accumulation: the reduction
//                            step of a reduce-scatter whose transfers were plain peer copies
#include <cuda.h>
#include <cudaTypedefs.h>

#include "hexa_common.cuh"

namespace hexa {
namespace {

template <typename T>
__global__ void mean_slices_kernel(const T* __restrict__ local, const T* __restrict__ recv, int n_recv, int64_t elems,
                                   float scale, T* __restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  const int64_t nvec = elems / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[V];
    {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(local) + i);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = to_f32<T>(v[j]);
    }
    for (int s = 0; s < n_recv; ++s) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(recv + (int64_t)s * elems) + i);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_f32<T>(v[j]);
    }
    uint4 o;
    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < V; ++j) ov[j] = from_f32<T>(acc[j] * scale);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

PFN_cuStreamWaitValue32_v11070 wait_value_fn() {
  static PFN_cuStreamWaitValue32_v11070 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuStreamWaitValue32", &ptr, 11070, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuStreamWaitValue32_v11070>(ptr);
  }
  return fn;
}

}  // namespace
}  // namespace hexa

using namespace hexa;

extern "C" int hexa_stream_wait_value(const int32_t* addr, int32_t value, void* stream_) {
  HEXA_REQUIRE(addr, "hexa_stream_wait_value: null address");
  auto fn = wait_value_fn();
  if (!fn) { set_error("cuStreamWaitValue32 is not available from the driver"); return HEXA_ERR_CUDA; }
  CUresult r = fn((CUstream)stream_, (CUdeviceptr)(uintptr_t)addr, (cuuint32_t)value, CU_STREAM_WAIT_VALUE_GEQ);
  if (r != CUDA_SUCCESS) { set_error("cuStreamWaitValue32 failed with CUresult %d", (int)r); return HEXA_ERR_CUDA; }
  return HEXA_OK;
}

extern "C" int hexa_mean_slices(const void* local, const void* recv, int n_recv, int64_t elems, int world, void* out,
                                int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(local && out && (recv || n_recv == 0), "hexa_mean_slices: null pointer");
  HEXA_REQUIRE(n_recv >= 0 && elems >= 0 && world > 0, "hexa_mean_slices: bad sizes");
  HEXA_REQUIRE(aligned16(local) && aligned16(out) && (n_recv == 0 || aligned16(recv)), "hexa_mean_slices: pointers must be 16-byte aligned");
  const int V = 16 / (int)dtype_size(dtype);
  HEXA_REQUIRE(elems % V == 0, "hexa_mean_slices: element count must be a multiple of %d", V);
  if (elems == 0) return HEXA_OK;
  const float scale = 1.0f / (float)world;
  int64_t blocks = ceil_div(elems / V, 256);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  switch (dtype) {
    case HEXA_F32: mean_slices_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((const float*)local, (const float*)recv, n_recv, elems, scale, (float*)out); break;
    case HEXA_F16: mean_slices_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>((const __half*)local, (const __half*)recv, n_recv, elems, scale, (__half*)out); break;
    case HEXA_BF16: mean_slices_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)local, (const __nv_bfloat16*)recv, n_recv, elems, scale, (__nv_bfloat16*)out); break;
    default: HEXA_REQUIRE(false, "hexa_mean_slices: bad dtype %d", dtype);
  }
  HEXA_LAUNCH_CHECK("mean_slices");
  return HEXA_OK;
}
