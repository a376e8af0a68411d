// CUDA-core (FFMA) ESMM and ESTMM on the sorted-row layout, fp32 accumulation.
// These are the kernels for fp32 data (where a 16-bit tensor-core pass cannot meet a 1e-5
// tolerance) and for shapes the tcgen05 kernels do not take (leading dimensions that are not
// multiples of 16 bytes).  64x64 output tile, 16-deep k step, 256 threads with a 4x4 micro-tile.
#include "gemm_launch.h"
#include "hexa_common.cuh"

namespace hexa {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
esmm_simt_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int b_layout, int64_t ldb,
                 int64_t b_estride, const float* __restrict__ bias, int64_t ldbias, T* __restrict__ aux, int64_t ldaux,
                 T* __restrict__ c, int64_t ldc, const int32_t* __restrict__ tile_expert,
                 const int32_t* __restrict__ pad_offsets, const int32_t* __restrict__ row_token, int E, int64_t n_out,
                 int64_t k, int epilogue, int act, int e_begin, int e_end) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int64_t row0 = (int64_t)blockIdx.y * BM;
  if (row0 >= pad_offsets[E]) return;
  const int e = tile_expert[row0 / kRowTile];
  if (e < e_begin || e >= e_end) return;      // also the -1 of tiles beyond the last segment
  const int64_t n0 = (int64_t)blockIdx.x * BN;
  const T* be = b + (int64_t)e * b_estride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int idx = threadIdx.x + 256 * q;
      {  // A: 64 rows x 16 k, k fastest
        const int r = idx >> 4, kk = idx & 15;
        float v = 0.f;
        if (k0 + kk < k) v = to_f32<T>(a[(row0 + r) * lda + k0 + kk]);
        As[kk][r] = v;
      }
      if (b_layout == HEXA_B_NK) {  // b[e][n][k], k fastest
        const int n = idx >> 4, kk = idx & 15;
        float v = 0.f;
        if (k0 + kk < k && n0 + n < n_out) v = to_f32<T>(be[(n0 + n) * ldb + k0 + kk]);
        Bs[kk][n] = v;
      } else {  // b[e][k][n], n fastest
        const int kk = idx >> 6, n = idx & 63;
        float v = 0.f;
        if (k0 + kk < k && n0 + n < n_out) v = to_f32<T>(be[(k0 + kk) * ldb + n0 + n]);
        Bs[kk][n] = v;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row0 + ty * 4 + i;
    const bool live = row_token == nullptr || row_token[r] >= 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= n_out) continue;
      float v = acc[i][j];
      if (bias) v += bias[(int64_t)e * ldbias + n];
      float o;
      if (epilogue == HEXA_EPI_ACT) {
        if (aux) aux[r * ldaux + n] = from_f32<T>(live ? v : 0.f);
        o = act_apply(act, v);
      } else if (epilogue == HEXA_EPI_DACT) {
        o = v * act_grad(act, to_f32<T>(aux[r * ldaux + n]));
      } else {
        o = v;
      }
      c[r * ldc + n] = from_f32<T>(live ? o : 0.f);
    }
  }
}

template <typename T, typename TO>
__global__ void __launch_bounds__(256)
estmm_simt_kernel(const T* __restrict__ p, int64_t ldp, const T* __restrict__ q, int64_t ldq,
                  const int32_t* __restrict__ pad_offsets, int64_t m, int64_t n, TO* __restrict__ out, int64_t ldo,
                  int64_t o_estride, int64_t m_split, int64_t split_stride, int beta) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int e = blockIdx.z;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int64_t r_begin = pad_offsets[e], r_end = pad_offsets[e + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int64_t r0 = r_begin; r0 < r_end; r0 += BK) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const int idx = threadIdx.x + 256 * s;
      const int kk = idx >> 6, x = idx & 63;
      float va = 0.f, vb = 0.f;
      if (r0 + kk < r_end) {
        if (m0 + x < m) va = to_f32<T>(p[(r0 + kk) * ldp + m0 + x]);
        if (n0 + x < n) vb = to_f32<T>(q[(r0 + kk) * ldq + n0 + x]);
      }
      As[kk][x] = va;
      Bs[kk][x] = vb;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  TO* oe = out + (int64_t)e * o_estride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t mm = m0 + ty * 4 + i;
    if (mm >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t nn = n0 + tx * 4 + j;
      if (nn >= n) continue;
      float v = acc[i][j];
      TO* dst = oe + (mm / m_split) * split_stride + (mm % m_split) * ldo + nn;
      if (beta) v += to_f32<TO>(*dst);
      *dst = from_f32<TO>(v);
    }
  }
}

}  // namespace

int esmm_simt_launch(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                     const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                     const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token, int E,
                     int64_t row_cap, int64_t n_out, int64_t k, int dtype, int epilogue, int act, cudaStream_t stream,
                     int e_begin, int e_end) {
  if (row_cap == 0 || e_begin >= e_end) return HEXA_OK;
  if (e_begin < 0) e_begin = 0;
  dim3 grid((unsigned)ceil_div(n_out, BN), (unsigned)(row_cap / BM));
  HEXA_REQUIRE(grid.y <= 65535, "hexa_esmm (simt): row_capacity %lld too large", (long long)row_cap);
#define HEXA_ESMM_SIMT(T)                                                                                             \
  esmm_simt_kernel<T><<<grid, 256, 0, stream>>>((const T*)a, lda, (const T*)b, b_layout, ldb, b_estride, bias, ldbias, \
                                                (T*)aux, ldaux, (T*)c, ldc, tile_expert, pad_offsets, row_token, E,   \
                                                n_out, k, epilogue, act, e_begin, e_end)
  switch (dtype) {
    case HEXA_F32: HEXA_ESMM_SIMT(float); break;
    case HEXA_F16: HEXA_ESMM_SIMT(__half); break;
    case HEXA_BF16: HEXA_ESMM_SIMT(__nv_bfloat16); break;
    default: HEXA_REQUIRE(false, "hexa_esmm: bad dtype %d", dtype);
  }
#undef HEXA_ESMM_SIMT
  HEXA_LAUNCH_CHECK("esmm_simt");
  return HEXA_OK;
}

int estmm_simt_launch(const void* p, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets, int E,
                      int64_t m, int64_t n, void* out, int64_t ldo, int64_t o_estride, int64_t m_split, int64_t split_stride,
                      int dtype, int out_dtype, int beta, cudaStream_t stream) {
  dim3 grid((unsigned)ceil_div(n, BN), (unsigned)ceil_div(m, BM), (unsigned)E);
  HEXA_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "hexa_estmm (simt): grid too large");
#define HEXA_ESTMM_SIMT(T, TO)                                                                                       \
  estmm_simt_kernel<T, TO><<<grid, 256, 0, stream>>>((const T*)p, ldp, (const T*)q, ldq, pad_offsets, m, n, (TO*)out, \
                                                     ldo, o_estride, m_split, split_stride, beta)
  if (dtype == HEXA_F32 && out_dtype == HEXA_F32) HEXA_ESTMM_SIMT(float, float);
  else if (dtype == HEXA_F16 && out_dtype == HEXA_F32) HEXA_ESTMM_SIMT(__half, float);
  else if (dtype == HEXA_F16 && out_dtype == HEXA_F16) HEXA_ESTMM_SIMT(__half, __half);
  else if (dtype == HEXA_BF16 && out_dtype == HEXA_F32) HEXA_ESTMM_SIMT(__nv_bfloat16, float);
  else if (dtype == HEXA_BF16 && out_dtype == HEXA_BF16) HEXA_ESTMM_SIMT(__nv_bfloat16, __nv_bfloat16);
  else HEXA_REQUIRE(false, "hexa_estmm: unsupported dtype pair %d -> %d", dtype, out_dtype);
#undef HEXA_ESTMM_SIMT
  HEXA_LAUNCH_CHECK("estmm_simt");
  return HEXA_OK;
}

}  // namespace hexa
