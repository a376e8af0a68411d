// Building blocks for collectives that run on copy engines and stream memory operations instead of SMs:
//   hexa_stream_wait_value   the stream waits until a 32-bit word in device memory is >= a value (written by a peer's
//                            copy over NVLink); with one word per peer this is an SM-free barrier between ranks
//   hexa_mean_slices         out = (local + sum of n received slices) / world, fp32 accumulation: the reduction
//                            step of a reduce-scatter whose transfers were plain peer copies
#include <cuda.h>
#include <stdlib.h>
#include <cudaTypedefs.h>

#include "hexa_common.cuh"

namespace hexa {
namespace {

// The kernel runs on a side stream beside the persistent GEMM kernels, and what it may use is what such a kernel's CTA
// leaves of an SM.  The register file is split over the four sub-partitions (16K registers each); the GEMM CTA puts
// five warps of 96 registers on two of them (its TMA-producer and MMA-issuer warps share sub-partitions 0 and 1 with
// epilogue warps), which leaves exactly 1024 registers there: one warp of 32 registers per thread.  A block of this
// kernel is therefore four warps (one per sub-partition) compiled to at most 32 registers; with more, its blocks are
// not scheduled until a GEMM kernel has drained (measured: a launch then takes as long as a GEMM, 5-8 ms instead of
// under 1 ms).  Within 32 registers a thread keeps four independent 16-byte loads in flight: the same vector of four
// slices (or of two slices at two positions) before anything is added.  S = n_recv + 1 when that is 2, 4 or 8; other
// slice counts take the generic loop.
template <typename T, int S, int U>
__global__ void __launch_bounds__(128, 16)
mean_slices_kernel(const T* __restrict__ local, const T* __restrict__ recv, int n_recv, int64_t elems, float scale,
                   T* __restrict__ out) {
  constexpr int V = 16 / sizeof(T);
  constexpr int B = S > 4 ? 4 : (S > 0 ? S : 1);      // slices loaded together
  const int64_t nvec = elems / V;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const uint4* loc4 = reinterpret_cast<const uint4*>(local);
  const uint4* rcv4 = reinterpret_cast<const uint4*>(recv);
  uint4* out4 = reinterpret_cast<uint4*>(out);
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (S > 0) {
    for (; i + (U - 1) * stride < nvec; i += U * stride) {
#pragma unroll
      for (int u0 = 0; u0 < U; u0 += (B == 2 ? 2 : 1)) {
        constexpr int UB = B == 2 ? 2 : 1;             // positions handled together (two when only two slices exist)
        float acc[UB][V];
#pragma unroll
        for (int s0 = 0; s0 < S; s0 += B) {
          uint4 raw[UB][B];
#pragma unroll
          for (int u = 0; u < UB; ++u)
#pragma unroll
            for (int s = 0; s < B; ++s) {
              const int64_t pos = i + (u0 + u) * stride;
              raw[u][s] = (s0 + s == 0) ? __ldg(loc4 + pos) : __ldg(rcv4 + (int64_t)(s0 + s - 1) * nvec + pos);
            }
#pragma unroll
          for (int u = 0; u < UB; ++u)
#pragma unroll
            for (int s = 0; s < B; ++s) {              // fixed order: local, then the received slices by index
              const T* v = reinterpret_cast<const T*>(&raw[u][s]);
#pragma unroll
              for (int j = 0; j < V; ++j) acc[u][j] = (s0 + s == 0) ? to_f32<T>(v[j]) : acc[u][j] + to_f32<T>(v[j]);
            }
        }
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          uint4 o;
          T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
          for (int j = 0; j < V; ++j) ov[j] = from_f32<T>(acc[u][j] * scale);
          out4[i + (u0 + u) * stride] = o;
        }
      }
    }
  }
  for (; i < nvec; i += stride) {      // generic slice count, and the tail of the unrolled loop
    float acc[V];
    {
      const uint4 raw = __ldg(loc4 + i);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = to_f32<T>(v[j]);
    }
    for (int s = 0; s < n_recv; ++s) {
      const uint4 raw = __ldg(rcv4 + (int64_t)s * nvec + i);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_f32<T>(v[j]);
    }
    uint4 o;
    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < V; ++j) ov[j] = from_f32<T>(acc[j] * scale);
    out4[i] = o;
  }
}

// Grid size in multiples of the SM count (A/B switch HEXA_MEAN_BLOCKS_PER_SM, read at every call; default 4).
int mean_env(const char* name, int dflt) {
  const char* v = getenv(name);
  return v ? atoi(v) : dflt;
}
constexpr int kMeanThreads = 128;

// Blocks of two kernels share an SM only if both run with the same split of the SM's L1 / shared-memory array.  The
// GEMM kernels this one is meant to run beside take the largest shared-memory carve-out, so the same preference is set
// here (the kernel itself uses no shared memory); without it the blocks wait for a GEMM kernel to drain.
template <typename K>
void prefer_max_shared_carveout(K kernel) {
  static bool done[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return;
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
      (void)cudaGetLastError();
    done[dev] = true;
  }
}

template <typename T, int S, int U>
void mean_slices_launch_su(const T* l, const T* r, int n_recv, int64_t elems, float scale, T* o, unsigned blocks, cudaStream_t stream) {
  prefer_max_shared_carveout(mean_slices_kernel<T, S, U>);
  mean_slices_kernel<T, S, U><<<blocks, kMeanThreads, 0, stream>>>(l, r, n_recv, elems, scale, o);
}

template <typename T>
void mean_slices_launch(const void* local, const void* recv, int n_recv, int64_t elems, float scale, void* out, unsigned blocks,
                        cudaStream_t stream) {
  const T* l = static_cast<const T*>(local);
  const T* r = static_cast<const T*>(recv);
  T* o = static_cast<T*>(out);
  switch (n_recv + 1) {
    case 2: mean_slices_launch_su<T, 2, 2>(l, r, n_recv, elems, scale, o, blocks, stream); break;
    case 4: mean_slices_launch_su<T, 4, 1>(l, r, n_recv, elems, scale, o, blocks, stream); break;
    case 8: mean_slices_launch_su<T, 8, 1>(l, r, n_recv, elems, scale, o, blocks, stream); break;
    default: mean_slices_launch_su<T, 0, 1>(l, r, n_recv, elems, scale, o, blocks, stream); break;
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
  int64_t blocks = ceil_div(elems / V, kMeanThreads * 4);
  int per_sm = mean_env("HEXA_MEAN_BLOCKS_PER_SM", 4);
  if (per_sm < 1) per_sm = 1;
  const int64_t cap = (int64_t)sm_count() * per_sm;   // a few waves of one-block-per-SM residency beside a GEMM kernel
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  switch (dtype) {
    case HEXA_F32: mean_slices_launch<float>(local, recv, n_recv, elems, scale, out, (unsigned)blocks, stream); break;
    case HEXA_F16: mean_slices_launch<__half>(local, recv, n_recv, elems, scale, out, (unsigned)blocks, stream); break;
    case HEXA_BF16: mean_slices_launch<__nv_bfloat16>(local, recv, n_recv, elems, scale, out, (unsigned)blocks, stream); break;
    default: HEXA_REQUIRE(false, "hexa_mean_slices: bad dtype %d", dtype);
  }
  HEXA_LAUNCH_CHECK("mean_slices");
  return HEXA_OK;
}
