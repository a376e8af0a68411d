// C-ABI entry points of the GEMM-shaped operators: argument checks and engine selection.
#include "hexa_common.cuh"

#include "gemm_launch.h"

using namespace hexa;

namespace {
// Destinations of hexa_estmm_scatter must live in the calling device's own memory.  Stores from the GEMM kernel into
// another GPU's memory (IPC-mapped buffers of a peer process) ended in an illegal-address fault in every run that
// tried them on two B200s - with peer access enabled only towards the calling device, and again with
// cudaDeviceEnablePeerAccess issued from the storing device - while the same kernel with local destinations is
// bit-identical to the packed layout.  The cause is not known, so the entry point refuses such pointers.
int require_local_destination(const void* ptr, int dev, const char* who) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
    (void)cudaGetLastError();
    set_error("%s: cannot classify destination pointer %p", who, ptr);
    return HEXA_ERR_INVALID;
  }
  if (at.type != cudaMemoryTypeDevice) {
    set_error("%s: destination %p is not device memory", who, ptr);
    return HEXA_ERR_INVALID;
  }
  if (at.device != dev) {
    set_error("%s: destination %p lives on device %d, the call runs on device %d: destinations in another GPU's memory "
              "are not supported (move the slice with a peer copy instead)", who, ptr, at.device, dev);
    return HEXA_ERR_UNSUPPORTED;
  }
  return HEXA_OK;
}
}  // namespace

extern "C" int hexa_esmm_experts(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                                 const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                                 const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                                 const int32_t* pair_block, int E, int64_t row_cap, int64_t n_out, int64_t k, int dtype,
                                 int epilogue, int act, int engine, int expert_begin, int expert_end, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(a && b && c && tile_expert && pad_offsets, "hexa_esmm: null pointer");
  HEXA_REQUIRE(expert_begin >= 0 && expert_begin <= expert_end && expert_end <= E,
               "hexa_esmm: expert range [%d, %d) is not inside [0, %d)", expert_begin, expert_end, E);
  HEXA_REQUIRE(E > 0 && row_cap >= 0 && row_cap % kRowTile == 0 && n_out > 0 && k > 0,
               "hexa_esmm: bad sizes (row_capacity must be a multiple of %d)", kRowTile);
  HEXA_REQUIRE(lda >= k && ldc >= n_out && (!aux || ldaux >= n_out) && (!bias || ldbias >= n_out), "hexa_esmm: leading dimension too small");
  HEXA_REQUIRE(b_layout == HEXA_B_NK || b_layout == HEXA_B_KN, "hexa_esmm: bad b_layout %d", b_layout);
  HEXA_REQUIRE(ldb >= (b_layout == HEXA_B_NK ? k : n_out), "hexa_esmm: ldb too small");
  HEXA_REQUIRE(dtype == HEXA_F32 || dtype == HEXA_F16 || dtype == HEXA_BF16, "hexa_esmm: bad dtype %d", dtype);
  HEXA_REQUIRE(epilogue >= HEXA_EPI_LINEAR && epilogue <= HEXA_EPI_DACT, "hexa_esmm: bad epilogue %d", epilogue);
  HEXA_REQUIRE(act >= HEXA_ACT_NONE && act <= HEXA_ACT_SILU, "hexa_esmm: bad activation %d", act);
  HEXA_REQUIRE(epilogue != HEXA_EPI_DACT || aux, "hexa_esmm: HEXA_EPI_DACT needs the saved pre-activation in aux");
  HEXA_REQUIRE(engine >= HEXA_ENGINE_AUTO && engine <= HEXA_ENGINE_SIMT, "hexa_esmm: bad engine %d", engine);
  HEXA_CHECK_DEVICE_STATUS("hexa_esmm");
  const bool tc_ok = esmm_tc_supported(a, lda, b, ldb, b_estride, aux, ldaux, c, ldc, bias, ldbias, n_out, dtype);
  if (engine == HEXA_ENGINE_TCGEN05 && !tc_ok) {
    set_error("hexa_esmm: tcgen05 engine needs 16-bit data, 16-byte aligned pointers and leading dimensions / n_out that are multiples of 8");
    return HEXA_ERR_UNSUPPORTED;
  }
  if (engine != HEXA_ENGINE_SIMT && tc_ok)
    return esmm_tc_launch(a, lda, b, b_layout, ldb, b_estride, bias, ldbias, aux, ldaux, c, ldc, tile_expert, pad_offsets,
                          row_token, pair_block, E, row_cap, n_out, k, dtype, epilogue, act, stream, expert_begin, expert_end);
  return esmm_simt_launch(a, lda, b, b_layout, ldb, b_estride, bias, ldbias, aux, ldaux, c, ldc, tile_expert, pad_offsets,
                          row_token, E, row_cap, n_out, k, dtype, epilogue, act, stream, expert_begin, expert_end);
}

extern "C" int hexa_esmm(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                         const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                         const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                         const int32_t* pair_block, int E, int64_t row_cap, int64_t n_out, int64_t k, int dtype, int epilogue,
                         int act, int engine, void* stream_) {
  return hexa_esmm_experts(a, lda, b, b_layout, ldb, b_estride, bias, ldbias, aux, ldaux, c, ldc, tile_expert, pad_offsets,
                           row_token, pair_block, E, row_cap, n_out, k, dtype, epilogue, act, engine, 0, E, stream_);
}

extern "C" int hexa_esmm_ess(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                             const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                             const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                             const int32_t* pair_block, int E, int64_t row_cap, int64_t n_out, int64_t k, int dtype, int epilogue,
                             int act, int engine, float* sums, int64_t ld_sums, void* workspace, size_t workspace_bytes,
                             void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(sums && workspace && ld_sums >= n_out, "hexa_esmm_ess: sums / workspace missing or ld_sums too small");
  HEXA_REQUIRE(E > 0 && E <= 65535 && row_cap >= 0 && n_out > 0, "hexa_esmm_ess: bad sizes");
  const size_t need = hexa_ess_workspace_bytes(row_cap, n_out);
  if (workspace_bytes < need) {
    set_error("hexa_esmm_ess: workspace %zu bytes < required %zu", workspace_bytes, need);
    return HEXA_ERR_WORKSPACE;
  }
  const bool fused = a && b && c && engine != HEXA_ENGINE_SIMT &&
                     esmm_tc_supported(a, lda, b, ldb, b_estride, aux, ldaux, c, ldc, bias, ldbias, n_out, dtype);
  if (!fused) {   // same result in two passes: the GEMM, then ESS over its output
    int rc = hexa_esmm_experts(a, lda, b, b_layout, ldb, b_estride, bias, ldbias, aux, ldaux, c, ldc, tile_expert, pad_offsets,
                               row_token, pair_block, E, row_cap, n_out, k, dtype, epilogue, act, engine, 0, E, stream_);
    if (rc != HEXA_OK) return rc;
    return ess_launch(c, ldc, pad_offsets, E, row_cap, n_out, sums, ld_sums, dtype, (float*)workspace, stream);
  }
  // the checks of hexa_esmm_experts, then the tcgen05 launch with the block sums switched on
  HEXA_REQUIRE(tile_expert && pad_offsets, "hexa_esmm_ess: null pointer");
  HEXA_REQUIRE(row_cap % kRowTile == 0 && k > 0, "hexa_esmm_ess: bad sizes (row_capacity must be a multiple of %d)", kRowTile);
  HEXA_REQUIRE(lda >= k && ldc >= n_out && (!aux || ldaux >= n_out) && (!bias || ldbias >= n_out), "hexa_esmm_ess: leading dimension too small");
  HEXA_REQUIRE(b_layout == HEXA_B_NK || b_layout == HEXA_B_KN, "hexa_esmm_ess: bad b_layout %d", b_layout);
  HEXA_REQUIRE(ldb >= (b_layout == HEXA_B_NK ? k : n_out), "hexa_esmm_ess: ldb too small");
  HEXA_REQUIRE(epilogue >= HEXA_EPI_LINEAR && epilogue <= HEXA_EPI_DACT, "hexa_esmm_ess: bad epilogue %d", epilogue);
  HEXA_REQUIRE(act >= HEXA_ACT_NONE && act <= HEXA_ACT_SILU, "hexa_esmm_ess: bad activation %d", act);
  HEXA_REQUIRE(epilogue != HEXA_EPI_DACT || aux, "hexa_esmm_ess: HEXA_EPI_DACT needs the saved pre-activation in aux");
  HEXA_CHECK_DEVICE_STATUS("hexa_esmm_ess");
  int rc = esmm_tc_launch(a, lda, b, b_layout, ldb, b_estride, bias, ldbias, aux, ldaux, c, ldc, tile_expert, pad_offsets,
                          row_token, pair_block, E, row_cap, n_out, k, dtype, epilogue, act, stream, 0, E, (float*)workspace);
  if (rc != HEXA_OK) return rc;
  return ess_finish((const float*)workspace, pad_offsets, E, n_out, sums, ld_sums, stream);
}

extern "C" size_t hexa_estmm_workspace_bytes(int E, int64_t row_cap, int64_t m, int64_t n, int dtype) {
  if (E <= 0 || row_cap <= 0 || m <= 0 || n <= 0 || (dtype != HEXA_F16 && dtype != HEXA_BF16)) return 0;
  return estmm_tc_workspace_bytes(E, row_cap, m, n);
}

extern "C" int hexa_estmm(const void* p, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets, int E,
                          int64_t row_cap, int64_t m, int64_t n, void* out, int64_t ldo, int64_t o_estride, int64_t m_split,
                          int64_t split_stride, int dtype, int out_dtype, int beta, int engine, void* workspace,
                          size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(p && q && out && pad_offsets, "hexa_estmm: null pointer");
  HEXA_REQUIRE(E > 0 && row_cap >= 0 && row_cap % kRowTile == 0 && m > 0 && n > 0,
               "hexa_estmm: bad sizes (row_capacity must be a multiple of %d)", kRowTile);
  if (m_split <= 0 || m_split >= m) { m_split = m; split_stride = 0; }   // plain [E, m, n] output
  HEXA_REQUIRE(ldp >= m && ldq >= n && ldo >= n && o_estride >= (m_split - 1) * ldo + n, "hexa_estmm: leading dimension too small");
  HEXA_REQUIRE(split_stride >= 0, "hexa_estmm: negative split_stride");
  HEXA_REQUIRE(dtype == HEXA_F32 || dtype == HEXA_F16 || dtype == HEXA_BF16, "hexa_estmm: bad dtype %d", dtype);
  HEXA_REQUIRE(out_dtype == HEXA_F32 || out_dtype == dtype, "hexa_estmm: out_dtype must be fp32 or the input dtype");
  HEXA_REQUIRE(beta == 0 || beta == 1, "hexa_estmm: beta must be 0 or 1");
  HEXA_REQUIRE(engine >= HEXA_ENGINE_AUTO && engine <= HEXA_ENGINE_SIMT, "hexa_estmm: bad engine %d", engine);
  HEXA_CHECK_DEVICE_STATUS("hexa_estmm");
  const bool tc_ok = estmm_tc_supported(p, ldp, q, ldq, out, ldo, o_estride, split_stride, n, dtype, out_dtype);
  if (engine == HEXA_ENGINE_TCGEN05 && !tc_ok) {
    set_error("hexa_estmm: tcgen05 engine needs 16-bit inputs, 16-byte aligned pointers and leading dimensions / n that are multiples of 8");
    return HEXA_ERR_UNSUPPORTED;
  }
  if (engine != HEXA_ENGINE_SIMT && tc_ok)
    return estmm_tc_launch(p, ldp, q, ldq, pad_offsets, E, row_cap, m, n, out, ldo, o_estride, m_split, split_stride, dtype, out_dtype,
                           beta, stream, nullptr, 0, workspace, workspace_bytes);
  return estmm_simt_launch(p, ldp, q, ldq, pad_offsets, E, m, n, out, ldo, o_estride, m_split, split_stride, dtype, out_dtype, beta,
                           stream);
}

extern "C" int hexa_estmm_scatter(const void* p, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets, int E,
                                  int64_t row_cap, int64_t m, int64_t n, void* const* split_out, int n_split, int64_t ldo,
                                  int64_t o_estride, int64_t m_split, int dtype, int out_dtype, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(p && q && split_out && pad_offsets, "hexa_estmm_scatter: null pointer");
  HEXA_REQUIRE(E > 0 && row_cap >= 0 && row_cap % kRowTile == 0 && m > 0 && n > 0,
               "hexa_estmm_scatter: bad sizes (row_capacity must be a multiple of %d)", kRowTile);
  HEXA_REQUIRE(m_split > 0 && n_split >= 1 && n_split <= 16 && (int64_t)n_split * m_split >= m && (int64_t)(n_split - 1) * m_split < m,
               "hexa_estmm_scatter: needs 1 <= n_split <= 16 slices of m_split rows covering m");
  HEXA_REQUIRE(ldp >= m && ldq >= n && ldo >= n && o_estride >= (m_split - 1) * ldo + n, "hexa_estmm_scatter: leading dimension too small");
  HEXA_REQUIRE(dtype == HEXA_F16 || dtype == HEXA_BF16, "hexa_estmm_scatter: 16-bit inputs only");
  HEXA_REQUIRE(out_dtype == HEXA_F32 || out_dtype == dtype, "hexa_estmm_scatter: out_dtype must be fp32 or the input dtype");
  HEXA_CHECK_DEVICE_STATUS("hexa_estmm_scatter");
  int dev = 0;
  HEXA_CUDA(cudaGetDevice(&dev));
  HEXA_REQUIRE(dev >= 0 && dev < 64, "hexa_estmm_scatter: device ordinal %d out of range", dev);
  for (int i = 0; i < n_split; ++i) {
    HEXA_REQUIRE(split_out[i], "hexa_estmm_scatter: split_out[%d] is null", i);
    const int rc = require_local_destination(split_out[i], dev, "hexa_estmm_scatter");
    if (rc != HEXA_OK) return rc;
    if (!estmm_tc_supported(p, ldp, q, ldq, split_out[i], ldo, o_estride, 0, n, dtype, out_dtype)) {
      set_error("hexa_estmm_scatter: needs 16-byte aligned pointers and leading dimensions / n that are multiples of 8");
      return HEXA_ERR_UNSUPPORTED;
    }
  }
  return estmm_tc_launch(p, ldp, q, ldq, pad_offsets, E, row_cap, m, n, split_out[0], ldo, o_estride, m_split, 0, dtype, out_dtype, 0,
                         stream, split_out, n_split);
}

extern "C" int hexa_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes, int64_t width_bytes,
                            int64_t height, void* stream_) {
  HEXA_REQUIRE(dst && src, "hexa_copy_2d: null pointer");
  HEXA_REQUIRE(width_bytes >= 0 && height >= 0 && dst_pitch_bytes >= width_bytes && src_pitch_bytes >= width_bytes,
               "hexa_copy_2d: bad sizes");
  if (width_bytes == 0 || height == 0) return HEXA_OK;
  HEXA_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_pitch_bytes, src, (size_t)src_pitch_bytes, (size_t)width_bytes, (size_t)height,
                              cudaMemcpyDeviceToDevice, (cudaStream_t)stream_));
  return HEXA_OK;
}
