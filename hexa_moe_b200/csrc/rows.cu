// HBM-bound row kernels on the sorted-row layout: gather, combine, pad-row masking and ESS.
//
// Bytes per unit (what the roofline of these kernels is computed from):
//   gather   reads cols*size per real row, writes cols*size per padded row, 4 B of row_token per row
//   combine  reads top_k*cols*size and writes cols*size per token, 4*top_k B of token_row
//   ESS      reads cols*size per padded row once; partials add 4*cols B per 128 rows (write + read)
#include "hexa_common.cuh"

namespace hexa {
namespace {

// ---- gather: warp per sorted row, 16-byte vectors ---------------------------------------------
template <int VEC_BYTES>
__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, int64_t src_ld_bytes,
                                   const int32_t* __restrict__ row_token, const int32_t* __restrict__ pad_offsets,
                                   int E, int64_t row_bytes, uint8_t* __restrict__ dst, int64_t dst_ld_bytes) {
  const int64_t n_pad = pad_offsets[E];
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_pad) return;
  const int32_t tok = row_token[row];
  uint8_t* d = dst + row * dst_ld_bytes;
  if (VEC_BYTES == 16) {
    const int64_t n = row_bytes >> 4;
    if (tok >= 0) {
      const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)tok * src_ld_bytes);
      for (int64_t i = lane; i < n; i += 32) reinterpret_cast<uint4*>(d)[i] = __ldg(s + i);
    } else {
      for (int64_t i = lane; i < n; i += 32) reinterpret_cast<uint4*>(d)[i] = make_uint4(0, 0, 0, 0);
    }
  } else {  // 2-byte granularity
    const int64_t n = row_bytes >> 1;
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src + (int64_t)(tok >= 0 ? tok : 0) * src_ld_bytes);
    for (int64_t i = lane; i < n; i += 32) reinterpret_cast<uint16_t*>(d)[i] = tok >= 0 ? s[i] : (uint16_t)0;
  }
}

// ---- combine: warp per token, fp32 accumulation over the k routes in fixed order --------------
// K > 0: top_k known at compile time - the token's K row indices are read once, and the K row loads of a column
// chunk are issued together before anything is added (the adds keep the order j = 0..K-1, so the result does not
// depend on K being a template parameter).  K = 0: any top_k.
template <typename T, int K>
__global__ void combine_rows_kernel(const T* __restrict__ src, int64_t src_ld, const int32_t* __restrict__ token_row,
                                    int64_t num_tokens, int top_k, int64_t cols, T* __restrict__ dst, int64_t dst_ld) {
  constexpr int V = 16 / sizeof(T);
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= num_tokens) return;
  const bool vec_ok = (cols % V == 0) && (src_ld % V == 0) && (dst_ld % V == 0);
  if (K > 0 && vec_ok) {
    const T* rows[K > 0 ? K : 1];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int32_t r = __ldg(token_row + t * K + j);
      rows[j] = r >= 0 ? src + (int64_t)r * src_ld : nullptr;
    }
#pragma unroll 2
    for (int64_t c = (int64_t)lane * V; c < cols; c += 32 * V) {
      uint4 raw[K > 0 ? K : 1];
#pragma unroll
      for (int j = 0; j < K; ++j)
        raw[j] = rows[j] ? __ldg(reinterpret_cast<const uint4*>(rows[j] + c)) : make_uint4(0, 0, 0, 0);
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (rows[j]) {      // an unrouted choice adds nothing (not even -0 + 0)
          const T* v = reinterpret_cast<const T*>(&raw[j]);
#pragma unroll
          for (int i = 0; i < V; ++i) acc[i] += to_f32<T>(v[i]);
        }
      }
      uint4 outv;
      T* o = reinterpret_cast<T*>(&outv);
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = from_f32<T>(acc[i]);
      *reinterpret_cast<uint4*>(dst + t * dst_ld + c) = outv;
    }
  } else if (vec_ok) {
    for (int64_t c = (int64_t)lane * V; c < cols; c += 32 * V) {
      float acc[V];
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const int32_t r = token_row[t * top_k + j];
        if (r < 0) continue;
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)r * src_ld + c));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += to_f32<T>(v[i]);
      }
      uint4 outv;
      T* o = reinterpret_cast<T*>(&outv);
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = from_f32<T>(acc[i]);
      *reinterpret_cast<uint4*>(dst + t * dst_ld + c) = outv;
    }
  } else {
    for (int64_t c = lane; c < cols; c += 32) {
      float acc = 0.f;
      for (int j = 0; j < top_k; ++j) {
        const int32_t r = token_row[t * top_k + j];
        if (r >= 0) acc += to_f32<T>(src[(int64_t)r * src_ld + c]);
      }
      dst[t * dst_ld + c] = from_f32<T>(acc);
    }
  }
}

template <typename T>
void combine_launch(const void* src, int64_t src_ld, const int32_t* token_row, int64_t T_, int top_k, int64_t cols, void* dst,
                    int64_t dst_ld, cudaStream_t stream) {
  const int warps = 8;
  const unsigned grid = (unsigned)ceil_div(T_, warps);
#define HEXA_COMBINE(K_)                                                                                              \
  combine_rows_kernel<T, K_><<<grid, warps * 32, 0, stream>>>((const T*)src, src_ld, token_row, T_, top_k, cols, (T*)dst, dst_ld)
  switch (top_k) {
    case 1: HEXA_COMBINE(1); break;
    case 2: HEXA_COMBINE(2); break;
    case 4: HEXA_COMBINE(4); break;
    default: HEXA_COMBINE(0); break;
  }
#undef HEXA_COMBINE
}

// ---- mask: zero the pad rows of a sorted buffer -------------------------------------------------
__global__ void mask_pad_rows_kernel(uint8_t* __restrict__ buf, int64_t ld_bytes, const int32_t* __restrict__ row_token,
                                     const int32_t* __restrict__ pad_offsets, int E, int64_t row_bytes) {
  const int64_t n_pad = pad_offsets[E];
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_pad || row_token[row] >= 0) return;
  uint16_t* d = reinterpret_cast<uint16_t*>(buf + row * ld_bytes);
  for (int64_t i = lane; i < (row_bytes >> 1); i += 32) d[i] = 0;
}

// ---- ESS pass 1: column sums of one 128-row tile (one expert) ------------------------------------
// block = 64 column groups x 4 row groups; a thread sums 32 rows of V adjacent columns.
template <typename T>
__global__ void __launch_bounds__(256)
ess_partial_kernel(const T* __restrict__ src, int64_t src_ld, const int32_t* __restrict__ pad_offsets, int E,
                   int64_t cols, float* __restrict__ partial) {
  constexpr int V = 16 / sizeof(T);
  __shared__ float red[4][64 * V];
  const int64_t n_pad = pad_offsets[E];
  const int64_t row0 = (int64_t)blockIdx.y * kRowTile;
  if (row0 >= n_pad) return;
  const int cx = threadIdx.x & 63, ry = threadIdx.x >> 6;
  const int64_t col = ((int64_t)blockIdx.x * 64 + cx) * V;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (col < cols) {
    const bool vec_ok = (col + V <= cols) && (src_ld % V == 0);
    for (int r = ry; r < kRowTile; r += 4) {
      const T* p = src + (row0 + r) * src_ld + col;
      if (vec_ok) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
        const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += to_f32<T>(v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i)
          if (col + i < cols) acc[i] += to_f32<T>(p[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[ry][cx * V + i] = acc[i];
  __syncthreads();
  if (ry == 0 && col < cols) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      if (col + i < cols) {
        float s = red[0][cx * V + i] + red[1][cx * V + i] + red[2][cx * V + i] + red[3][cx * V + i];
        partial[(int64_t)blockIdx.y * cols + col + i] = s;
      }
    }
  }
}

// ---- ESS pass 2: per expert, add its tiles' partial rows in ascending order ---------------------
__global__ void ess_final_kernel(const float* __restrict__ partial, const int32_t* __restrict__ pad_offsets,
                                 int64_t cols, float* __restrict__ out, int64_t ldo) {
  const int e = blockIdx.y;
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t t0 = pad_offsets[e] / kRowTile, t1 = pad_offsets[e + 1] / kRowTile;
  float s = 0.f;
  for (int64_t t = t0; t < t1; ++t) s += partial[t * cols + c];
  out[(int64_t)e * ldo + c] = s;
}

}  // namespace
}  // namespace hexa

using namespace hexa;

extern "C" int hexa_gather_rows(const void* src, int64_t src_ld, const int32_t* row_token, const int32_t* pad_offsets,
                                int E, int64_t row_cap, int64_t cols, void* dst, int64_t dst_ld, int dtype,
                                void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(row_token && pad_offsets && dst, "hexa_gather_rows: null pointer");   // src may be null when there are no tokens
  HEXA_REQUIRE(E > 0 && row_cap >= 0 && cols > 0 && src_ld >= cols && dst_ld >= cols, "hexa_gather_rows: bad sizes");
  HEXA_REQUIRE(dtype == HEXA_F32 || dtype == HEXA_F16 || dtype == HEXA_BF16, "hexa_gather_rows: bad dtype %d", dtype);
  if (row_cap == 0) return HEXA_OK;
  const int64_t es = (int64_t)dtype_size(dtype);
  const int64_t row_bytes = cols * es, sld = src_ld * es, dld = dst_ld * es;
  const bool v16 = (row_bytes % 16 == 0) && (sld % 16 == 0) && (dld % 16 == 0) && aligned16(src) && aligned16(dst);
  const int warps = 8;
  const unsigned grid = (unsigned)ceil_div(row_cap, warps);
  if (v16)
    gather_rows_kernel<16><<<grid, warps * 32, 0, stream>>>((const uint8_t*)src, sld, row_token, pad_offsets, E, row_bytes,
                                                            (uint8_t*)dst, dld);
  else
    gather_rows_kernel<2><<<grid, warps * 32, 0, stream>>>((const uint8_t*)src, sld, row_token, pad_offsets, E, row_bytes,
                                                           (uint8_t*)dst, dld);
  HEXA_LAUNCH_CHECK("gather_rows");
  return HEXA_OK;
}

extern "C" int hexa_combine_rows(const void* src, int64_t src_ld, const int32_t* token_row, int64_t T, int top_k,
                                 int64_t cols, void* dst, int64_t dst_ld, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(T >= 0 && top_k > 0 && cols > 0 && src_ld >= cols && dst_ld >= cols, "hexa_combine_rows: bad sizes");
  if (T == 0) return HEXA_OK;
  HEXA_REQUIRE(src && token_row && dst, "hexa_combine_rows: null pointer");
  HEXA_REQUIRE(aligned16(src) && aligned16(dst), "hexa_combine_rows: pointers must be 16-byte aligned");
  if (T == 0) return HEXA_OK;
  switch (dtype) {
    case HEXA_F32: combine_launch<float>(src, src_ld, token_row, T, top_k, cols, dst, dst_ld, stream); break;
    case HEXA_F16: combine_launch<__half>(src, src_ld, token_row, T, top_k, cols, dst, dst_ld, stream); break;
    case HEXA_BF16: combine_launch<__nv_bfloat16>(src, src_ld, token_row, T, top_k, cols, dst, dst_ld, stream); break;
    default: HEXA_REQUIRE(false, "hexa_combine_rows: bad dtype %d", dtype);
  }
  HEXA_LAUNCH_CHECK("combine_rows");
  return HEXA_OK;
}

extern "C" int hexa_mask_pad_rows(void* buf, int64_t ld, const int32_t* row_token, const int32_t* pad_offsets, int E,
                                  int64_t row_cap, int64_t cols, int dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(buf && row_token && pad_offsets, "hexa_mask_pad_rows: null pointer");
  HEXA_REQUIRE(E > 0 && row_cap >= 0 && cols > 0 && ld >= cols, "hexa_mask_pad_rows: bad sizes");
  HEXA_REQUIRE(dtype == HEXA_F32 || dtype == HEXA_F16 || dtype == HEXA_BF16, "hexa_mask_pad_rows: bad dtype %d", dtype);
  if (row_cap == 0) return HEXA_OK;
  const int64_t es = (int64_t)dtype_size(dtype);
  const int warps = 8;
  mask_pad_rows_kernel<<<(unsigned)ceil_div(row_cap, warps), warps * 32, 0, stream>>>((uint8_t*)buf, ld * es, row_token,
                                                                                     pad_offsets, E, cols * es);
  HEXA_LAUNCH_CHECK("mask_pad_rows");
  return HEXA_OK;
}

extern "C" size_t hexa_ess_workspace_bytes(int64_t row_cap, int64_t cols) {
  if (row_cap < 0 || cols <= 0) return 0;
  return (size_t)ceil_div(row_cap, kRowTile) * (size_t)cols * sizeof(float);
}

namespace hexa {
int ess_finish(const float* partial, const int32_t* pad_offsets, int E, int64_t cols, float* out, int64_t ldo, cudaStream_t stream);
// Shared by hexa_ess and the entry points built on it: both passes on caller-provided scratch.
int ess_launch(const void* src, int64_t src_ld, const int32_t* pad_offsets, int E, int64_t row_cap, int64_t cols,
               float* out, int64_t ldo, int dtype, float* partial, cudaStream_t stream) {
  const int64_t tiles = ceil_div(row_cap, kRowTile);
  if (tiles > 0) {
    const int V = 16 / (int)dtype_size(dtype);
    dim3 grid((unsigned)ceil_div(cols, 64 * V), (unsigned)tiles);
    HEXA_REQUIRE(tiles <= 65535, "hexa_ess: more than 65535 row tiles (row_capacity %lld)", (long long)row_cap);
    switch (dtype) {
      case HEXA_F32: ess_partial_kernel<float><<<grid, 256, 0, stream>>>((const float*)src, src_ld, pad_offsets, E, cols, partial); break;
      case HEXA_F16: ess_partial_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)src, src_ld, pad_offsets, E, cols, partial); break;
      case HEXA_BF16: ess_partial_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)src, src_ld, pad_offsets, E, cols, partial); break;
      default: HEXA_REQUIRE(false, "hexa_ess: bad dtype %d", dtype);
    }
    HEXA_LAUNCH_CHECK("ess_partial");
  }
  return ess_finish(partial, pad_offsets, E, cols, out, ldo, stream);
}

int ess_finish(const float* partial, const int32_t* pad_offsets, int E, int64_t cols, float* out, int64_t ldo, cudaStream_t stream) {
  dim3 grid2((unsigned)ceil_div(cols, 256), (unsigned)E);
  ess_final_kernel<<<grid2, 256, 0, stream>>>(partial, pad_offsets, cols, out, ldo);
  HEXA_LAUNCH_CHECK("ess_final");
  return HEXA_OK;
}
}  // namespace hexa

extern "C" int hexa_ess(const void* src, int64_t src_ld, const int32_t* pad_offsets, int E, int64_t row_cap,
                        int64_t cols, float* out, int64_t ldo, int dtype, void* workspace, size_t workspace_bytes,
                        void* stream_) {
  HEXA_REQUIRE(src && pad_offsets && out && workspace, "hexa_ess: null pointer");
  HEXA_REQUIRE(E > 0 && E <= 65535 && row_cap >= 0 && cols > 0 && src_ld >= cols && ldo >= cols, "hexa_ess: bad sizes");
  HEXA_REQUIRE(aligned16(src), "hexa_ess: src must be 16-byte aligned");
  const size_t need = hexa_ess_workspace_bytes(row_cap, cols);
  if (workspace_bytes < need) {
    set_error("hexa_ess: workspace %zu bytes < required %zu", workspace_bytes, need);
    return HEXA_ERR_WORKSPACE;
  }
  return ess_launch(src, src_ld, pad_offsets, E, row_cap, cols, out, ldo, dtype, (float*)workspace, (cudaStream_t)stream_);
}

// ---- ESS on library-owned scratch -------------------------------------------------------------------
// Pass 1 of ESS needs one fp32 partial row per 128 sorted rows.  hexa_ess takes that scratch from the
// caller; this variant keeps it in a fixed array inside the library instead, for callers that have no
// way to obtain device memory at the point of the call.
namespace hexa {
constexpr size_t kEssStaticFloats = (size_t)8 << 20;   // 8 Mi floats = 32 MiB, resident on every device that loads the library
static __device__ __align__(256) float g_ess_static_scratch[kEssStaticFloats];
}  // namespace hexa

extern "C" size_t hexa_ess_static_capacity_bytes(void) { return hexa::kEssStaticFloats * sizeof(float); }

extern "C" int hexa_ess_static(const void* src, int64_t src_ld, const int32_t* pad_offsets, int E, int64_t row_cap,
                               int64_t cols, float* out, int64_t ldo, int dtype, void* stream_) {
  HEXA_REQUIRE(src && pad_offsets && out, "hexa_ess_static: null pointer");
  HEXA_REQUIRE(E > 0 && E <= 65535 && row_cap >= 0 && cols > 0 && src_ld >= cols && ldo >= cols, "hexa_ess_static: bad sizes");
  HEXA_REQUIRE(aligned16(src), "hexa_ess_static: src must be 16-byte aligned");
  const size_t need = hexa_ess_workspace_bytes(row_cap, cols);
  if (need > kEssStaticFloats * sizeof(float)) {
    set_error("hexa_ess_static: needs %zu bytes of scratch (row_capacity/128 * cols floats) but the built-in buffer holds %zu; "
              "use hexa_ess with caller-provided workspace for this size",
              need, kEssStaticFloats * sizeof(float));
    return HEXA_ERR_WORKSPACE;
  }
  // The array's name is only a host-side handle; the kernels need its address on the current device.
  // Looked up once per device, with that device current (first call on a device: do it before any stream capture).
  static float* dev_addr[64] = {nullptr};
  int dev = 0;
  HEXA_CUDA(cudaGetDevice(&dev));
  HEXA_REQUIRE(dev >= 0 && dev < 64, "hexa_ess_static: device ordinal %d out of range", dev);
  float* scratch = __atomic_load_n(&dev_addr[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    HEXA_CUDA(cudaGetSymbolAddress((void**)&scratch, g_ess_static_scratch));
    __atomic_store_n(&dev_addr[dev], scratch, __ATOMIC_RELEASE);
  }
  // Nothing in the scratch has to start at zero: pass 1 overwrites every partial row that pass 2 reads.
  return ess_launch(src, src_ld, pad_offsets, E, row_cap, cols, out, ldo, dtype, scratch, (cudaStream_t)stream_);
}
