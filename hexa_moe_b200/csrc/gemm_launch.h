// Launchers of the GEMM-shaped operators, one set per kernel family (defined in gemm_tc.cu and gemm_simt.cu,
// selected by the C-ABI entry points in ops_api.cu).  Argument order follows hexa_esmm / hexa_estmm.
#pragma once

#include "hexa_common.cuh"

namespace hexa {
int esmm_simt_launch(const void*, int64_t, const void*, int, int64_t, int64_t, const float*, int64_t, void*, int64_t, void*,
                     int64_t, const int32_t*, const int32_t*, const int32_t*, int, int64_t, int64_t, int64_t, int, int, int,
                     cudaStream_t, int e_begin, int e_end);
int estmm_simt_launch(const void*, int64_t, const void*, int64_t, const int32_t*, int, int64_t, int64_t, void*, int64_t,
                      int64_t, int64_t, int64_t, int, int, int, cudaStream_t);
bool esmm_tc_supported(const void*, int64_t, const void*, int64_t, int64_t, const void*, int64_t, const void*, int64_t,
                       const float*, int64_t, int64_t, int);
int esmm_tc_launch(const void*, int64_t, const void*, int, int64_t, int64_t, const float*, int64_t, void*, int64_t, void*,
                   int64_t, const int32_t*, const int32_t*, const int32_t*, const int32_t*, int, int64_t, int64_t, int64_t, int,
                   int, int, cudaStream_t, int e_begin, int e_end, float* colsum = nullptr);
bool estmm_tc_supported(const void*, int64_t, const void*, int64_t, const void*, int64_t, int64_t, int64_t, int64_t, int, int);
int estmm_tc_launch(const void*, int64_t, const void*, int64_t, const int32_t*, int, int64_t, int64_t, int64_t, void*, int64_t,
                    int64_t, int64_t, int64_t, int, int, int, cudaStream_t, void* const* split_out = nullptr, int n_split = 0,
                    void* workspace = nullptr, size_t workspace_bytes = 0);
size_t estmm_tc_workspace_bytes(int E, int64_t row_cap, int64_t m, int64_t n);
// rows.cu: both passes of ESS, and its second pass alone (per expert, the partial rows of its 128-row blocks added in order)
int ess_launch(const void* src, int64_t src_ld, const int32_t* pad_offsets, int E, int64_t row_cap, int64_t cols, float* out,
               int64_t ldo, int dtype, float* partial, cudaStream_t stream);
int ess_finish(const float* partial, const int32_t* pad_offsets, int E, int64_t cols, float* out, int64_t ldo, cudaStream_t stream);
}  // namespace hexa
