/*
 * hexa_moe_b200 - C ABI of the B200 (sm_100a) expert-specific MoE operators.
 *
 * Every entry point takes plain device pointers, sizes, leading dimensions and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t).  Unless a comment says otherwise an entry point
 * allocates nothing, never synchronises with the host and never exits the process: scratch memory
 * is supplied by the caller (query the size with the matching *_workspace_bytes function).
 * Return value: HEXA_OK or a negative hexa_status; hexa_last_error_string() describes the
 * last failure on the calling thread.
 *
 * Layout shared by all operators ("sorted rows"): the N = T*top_k routed rows of a layer are
 * numbered f = j*T + t (route-major) and stably sorted by expert; expert e owns rows
 * [pad_offsets[e], pad_offsets[e] + counts[e]) and its segment is padded with empty rows up to
 * pad_offsets[e+1], a multiple of `align`.  row_token[r] is the token of row r or -1 for a pad
 * row; token_row[t*top_k + j] is the row of routed row (t,j); tile_expert[r/align] is the expert
 * that owns the `align`-row tile.  Pad rows of every activation buffer hold zeros.
 *
 * Replaces, in the reference (paths inside the UNITES-Lab/HEXA-MoE repository):
 *   hexa_moe_cuda/hexa_moe/include/hexa_moe.h:3-181      (13 raw-pointer launchers)
 *   hexa_moe_cuda/hexa_moe/torch/hexa_moe_ops.cpp:9-301  (pybind11 module hexa_moe_cuda)
 *   hexa_moe_triton/hexa_moe/kernels/{basics,esmm,fused}.py (counter / ESMM / es_fused)
 */
#ifndef HEXA_MOE_B200_H
#define HEXA_MOE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  HEXA_OK = 0,
  HEXA_ERR_INVALID = -1,      /* bad argument (null pointer, size, alignment, enum) */
  HEXA_ERR_CUDA = -2,         /* a CUDA runtime / driver call failed */
  HEXA_ERR_UNSUPPORTED = -3,  /* valid request that this build has no kernel for */
  HEXA_ERR_WORKSPACE = -4,    /* caller-supplied workspace too small */
  HEXA_ERR_DEVICE = -5        /* a kernel reported a failure through its status word */
} hexa_status;

typedef enum { HEXA_F32 = 0, HEXA_F16 = 1, HEXA_BF16 = 2 } hexa_dtype;

/* Activation fused into the ESMM epilogue (HEXA_ACT_NONE: plain linear). */
typedef enum {
  HEXA_ACT_NONE = 0,
  HEXA_ACT_RELU = 1,
  HEXA_ACT_GELU = 2,       /* exact, erf based (torch.nn.functional.gelu default) */
  HEXA_ACT_GELU_TANH = 3,
  HEXA_ACT_SILU = 4
} hexa_act;

/* Layout of the per-expert B operand of hexa_esmm. */
typedef enum {
  HEXA_B_NK = 0, /* b[e] is [n_out, k], k contiguous: c = a * b[e]^T (fc1 forward, fc2 dgrad)   */
  HEXA_B_KN = 1  /* b[e] is [k, n_out], n_out contiguous: c = a * b[e] (fc2 forward, fc1 dgrad) */
} hexa_b_layout;

/* Epilogue of hexa_esmm. */
typedef enum {
  HEXA_EPI_LINEAR = 0, /* c = acc + bias                                                          */
  HEXA_EPI_ACT = 1,    /* aux (if non-null) = acc + bias ; c = act(acc + bias)                    */
  HEXA_EPI_DACT = 2    /* c = acc * act'(aux)   (aux holds the saved pre-activation)              */
} hexa_epilogue;

/* Which kernel family executes a GEMM-shaped operator. */
typedef enum {
  HEXA_ENGINE_AUTO = 0, /* tcgen05 when dtype/alignment allow it, otherwise the CUDA-core kernel  */
  HEXA_ENGINE_TCGEN05 = 1,
  HEXA_ENGINE_SIMT = 2  /* fp32-accumulating CUDA-core kernel (the only one for HEXA_F32)         */
} hexa_engine;

/* Library / error reporting.  Replaces HandleError's printf+exit(1)
 * (hexa_moe_cuda/hexa_moe/kernels/esmm_half.cu:27-36). */
int hexa_version(void);
const char* hexa_last_error_string(void);

/* Device status word for kernels with bounded waits (mbarrier spins in the tcgen05 kernels).
 * `status` points to one zeroed int32 that kernels on the CURRENT device can write: device memory, or pinned host
 * memory (cudaHostAlloc / cudaHostRegister), which the host can read at any time without a copy or a synchronisation.
 * A kernel that gives up a wait stores a non-zero code there (1 = producer waiting for a free ring slot, 2 = MMA
 * issuer waiting for a drained accumulator, 3 = MMA issuer waiting for operands, 4 = epilogue waiting for an
 * accumulator), lets copies in flight land, frees its tensor memory and returns; its outputs are incomplete.
 * One word per device, shared by all host threads (forward and backward of a training step are launched from
 * different threads).  With a word in pinned host memory, hexa_esmm / hexa_estmm / hexa_estmm_scatter return
 * HEXA_ERR_DEVICE without launching while the word is non-zero; the caller zeroes the word to continue.
 * NULL disables reporting (waits stay bounded).  Replaces, as the way a device-side failure reaches the host,
 * HandleError's printf + exit(1) (hexa_moe_cuda/hexa_moe/kernels/esmm_half.cu:27-36). */
int hexa_set_status_word(int32_t* status);
/* Code currently in the current device's status word when that word is host-readable, else 0.  Never synchronises. */
int hexa_pending_device_status(void);
/* Limit of every wait inside the kernels, in nanoseconds of the GPU's global timer (process-wide; default 2 s). */
int hexa_set_wait_limit_ns(uint64_t ns);
/* Measurement / test switches of the tcgen05 kernels (process-wide; initial value: environment variable
 * HEXA_TC_DEBUG, default 0).  bit 0: the TMA producer skips its loads and signals their arrival itself; bit 1: the
 * MMA thread skips the MMAs (both: timing of the remaining pipeline, results are garbage); bit 2: the producer
 * neither loads nor signals, so every wait of the pipeline runs into its limit and the kernel reports through the
 * status word (used with a short hexa_set_wait_limit_ns to exercise the error path without any fault). */
int hexa_set_tc_debug(int flags);

/* Cap on the SMs the persistent GEMM kernels occupy from now on (process-wide; 0 = all SMs).  Their tile
 * schedule is static, so they should not share SMs with long-running kernels of other streams (collectives):
 * set a cap while such kernels may be running.  No counterpart in the reference. */
int hexa_set_sm_limit(int num_sms);

/* ---- routing: replaces launch_count + launch_assign (include/hexa_moe.h:3-22,
 *      kernels/shared_cuda_core.cu:128-182, 285-333) and kernels/basics.py:counter (89-118) ---- */

/* Upper bound on padded rows: T*top_k + E*(align-1), rounded up to a multiple of align. */
int64_t hexa_route_row_capacity(int64_t num_tokens, int top_k, int num_experts, int align);
size_t hexa_route_workspace_bytes(int64_t num_tokens, int top_k, int num_experts);
/* Entries of the optional pair-tile list (align = 128 only): row_capacity/256 + E + 1. */
int64_t hexa_route_pair_capacity(int64_t num_tokens, int top_k, int num_experts);

/* ids: expert id of routed row (t,j) at ids[t*stride_t + j*stride_k]; ids outside [0,E) are
 * skipped (their token_row entry is -1).
 * Outputs (device, int32): counts[E], seg_offsets[E+1] (exclusive scan of counts),
 * pad_offsets[E+1], row_token[row_capacity], token_row[T*top_k], tile_expert[row_capacity/align]
 * (-1 beyond pad_offsets[E]).  Results are deterministic: identical to a stable sort.
 * pair_block (optional, NULL to skip; needs align = 128): for the GEMMs that run on pairs of SMs, the list of
 * 256-row pair tiles, entry = (first 128-row block)*2 + (1 if the next block belongs to the same expert),
 * terminated and padded with -1; hexa_route_pair_capacity entries. */
int hexa_route(const int32_t* ids, int64_t num_tokens, int top_k, int64_t stride_t, int64_t stride_k,
               int num_experts, int align, int32_t* counts, int32_t* seg_offsets, int32_t* pad_offsets,
               int32_t* row_token, int32_t* token_row, int32_t* tile_expert, int32_t* pair_block,
               void* workspace, size_t workspace_bytes, void* stream);

/* ---- row movement between token order and sorted-row order (the reference gathers rows by
 *      tok_ids inside its kernels, kernels/esmm.py:95-101, and sums the k routes in Python,
 *      impls/layers.py:254-258) ---- */

/* dst[r,:] = row_token[r] >= 0 ? src[row_token[r],:] : 0   for r < pad_offsets[E]. */
int hexa_gather_rows(const void* src, int64_t src_ld, const int32_t* row_token, const int32_t* pad_offsets,
                     int num_experts, int64_t row_capacity, int64_t cols, void* dst, int64_t dst_ld,
                     int dtype, void* stream);

/* dst[t,:] = sum_j src[token_row[t*top_k + j],:] (fp32 accumulation, fixed order j = 0..k-1). */
int hexa_combine_rows(const void* src, int64_t src_ld, const int32_t* token_row, int64_t num_tokens,
                      int top_k, int64_t cols, void* dst, int64_t dst_ld, int dtype, void* stream);

/* ---- ESMM: replaces launch_esmm_accum_shared_tensor_{full,mix,half} (include/hexa_moe.h:24-72)
 *      and the ESMM part of launch_fused_grad_* ; kernels/esmm.py:ESMM (249-295),
 *      kernels/fused.py:142-182 ----
 * For every sorted row r < pad_offsets[E] with e = tile_expert[r/128]:
 *   acc[r,:] = a[r,:] (1 x k) times b[e] (layout per b_layout), fp32 accumulation, then `epilogue`.
 * a [row_capacity, k] (lda), c [row_capacity, n_out] (ldc), aux like c (ldaux) or NULL,
 * bias fp32 [E, n_out] (ldbias) or NULL, b expert stride b_estride and row stride ldb in elements.
 * Rows with row_token[r] < 0 are written as zeros.  Segments must be aligned to 128 rows.
 * pair_block: the list hexa_route produced, or NULL; with it (and n_out > 128, 16-bit data) the tcgen05 kernel
 * runs on clusters of two CTAs (256-row tiles, each CTA loading half of the weight tile).
 * The tcgen05 kernel takes 16-bit data with 16-byte aligned pointers and lda, ldb, b_estride, ldc, ldaux multiples
 * of 8 elements, ldbias a multiple of 4; n_out and k themselves may be any size (a rank's slice of an unevenly split
 * hidden dimension) as long as aux rows are padded to a multiple of 8 elements and bias rows to a multiple of 4
 * (ldaux >= roundup(n_out, 8), ldbias >= roundup(n_out, 4)): the epilogue reads them in 16-byte chunks.  Anything
 * else runs on the CUDA-core kernel under HEXA_ENGINE_AUTO and is refused under HEXA_ENGINE_TCGEN05. */
int hexa_esmm(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
              const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
              const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
              const int32_t* pair_block, int num_experts, int64_t row_capacity, int64_t n_out, int64_t k,
              int dtype, int epilogue, int act, int engine, void* stream);

/* hexa_esmm restricted to the rows of experts expert_begin <= e < expert_end; rows of other experts are left untouched.
 * Launching the layer's first GEMM once per group of experts lets it start on the experts whose weights have arrived
 * while the remaining weights of the layer are still being gathered from the other ranks (no counterpart in the
 * reference, which waits for the whole gathered tensor: impls/layers.py:109-124).  The groups of one operator may be
 * launched in any order and together write exactly what one hexa_esmm call writes. */
int hexa_esmm_experts(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                      const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                      const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                      const int32_t* pair_block, int num_experts, int64_t row_capacity, int64_t n_out, int64_t k,
                      int dtype, int epilogue, int act, int engine, int expert_begin, int expert_end, void* stream);

/* ---- ESTMM: replaces task 1 of launch_fused_grad_* (include/hexa_moe.h:74-181),
 *      kernels/fused.py:183-235 (operator definition; the reference kernels mis-handle segments
 *      longer than 16 rows) ----
 * out[e] (m x n, ld ldo, expert stride o_estride) = beta*out[e] + sum over rows r of expert e of
 * p[r,:m]^T (outer) q[r,:n].  Experts without rows get beta*out[e] (zeros for beta = 0).
 * p [row_capacity, m] (ldp), q [row_capacity, n] (ldq) in `dtype`; out in `out_dtype`
 * (HEXA_F32 or `dtype`); beta is 0 or 1.
 * m_split / split_stride: output row i of expert e is written at
 *   out + e*o_estride + (i / m_split)*split_stride + (i % m_split)*ldo,
 * which lets the gradient land directly in the [ranks, E, m/ranks, n] layout a reduce-scatter over the
 * hidden dimension consumes (m_split = m/ranks, split_stride = E*m_split*ldo, o_estride = m_split*ldo).
 * Pass m_split = 0 for the plain [E, m, n] layout.
 * workspace (optional): when the output has few tiles and the segments are long - the weight gradient of a dense FFN
 * run as one expert, or a few experts with a small m x n - one tile per expert's whole segment would leave most SMs
 * idle.  With hexa_estmm_workspace_bytes(...) bytes of 16-byte aligned scratch the tcgen05 kernel cuts every segment
 * into chunks (the count depends only on the static sizes), writes fp32 partial results there and adds them in chunk
 * order in a second kernel: deterministic, same rounding of the final result.  The query returns 0 when no split
 * would be used; NULL / too small a workspace runs the unsplit kernel.  (The reference accumulates a whole segment in
 * one program, kernels/fused.py:183-235.) */
size_t hexa_estmm_workspace_bytes(int num_experts, int64_t row_capacity, int64_t m, int64_t n, int dtype);
int hexa_estmm(const void* p, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets,
               int num_experts, int64_t row_capacity, int64_t m, int64_t n, void* out, int64_t ldo,
               int64_t o_estride, int64_t m_split, int64_t split_stride, int dtype, int out_dtype, int beta,
               int engine, void* workspace, size_t workspace_bytes, void* stream);

/* ESTMM whose output slices go to separate buffers (no reference counterpart; the reference all-reduces the full
 * gradient through torch.distributed, impls/layers.py:431-474): output row i of expert e is written at
 *   split_out[i / m_split] + e*o_estride + (i % m_split)*ldo            (elements of out_dtype)
 * split_out is a HOST array of n_split = ceil(m / m_split) <= 16 device pointers (copied at the call).  Meant for
 * laying a weight gradient out per owner of a hidden slice without a packing pass.  Every destination must be memory of
 * the calling device: a pointer into another GPU's memory is refused with HEXA_ERR_UNSUPPORTED (anything that is not
 * device memory with HEXA_ERR_INVALID).  Stores of this kernel into a peer's IPC-mapped buffer faulted with an illegal
 * address on two B200s in every attempt, with and without cudaDeviceEnablePeerAccess from the storing device; the
 * cause is not known, so the transfer of the reduce-scatter stays with the copy engines.
 * 16-bit inputs only (the tcgen05 kernel); the destination is overwritten (beta = 0). */
int hexa_estmm_scatter(const void* p, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets,
                       int num_experts, int64_t row_capacity, int64_t m, int64_t n, void* const* split_out, int n_split,
                       int64_t ldo, int64_t o_estride, int64_t m_split, int dtype, int out_dtype, void* stream);

/* Strided block copy on the stream (cudaMemcpy2DAsync, device to device): `height` rows of `width_bytes`.
 * Used to move hidden-dimension slices between the gathered [ranks, E, loc, d] staging layout and
 * [E, H, d] without spending SMs on it.  No counterpart in the reference (it builds the same views with
 * cat / permute / contiguous copies, impls/layers.py:112-118). */
int hexa_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes, int64_t width_bytes,
                 int64_t height, void* stream);

/* ---- ESS: replaces task 2 of launch_fused_grad_bias_*, kernels/fused.py:111-141 ----
 * out[e,:] = sum of src rows of expert e, fp32 [E, cols] (ldo).  Deterministic two-pass
 * reduction; workspace holds one fp32 partial row per 128 sorted rows. */
size_t hexa_ess_workspace_bytes(int64_t row_capacity, int64_t cols);
int hexa_ess(const void* src, int64_t src_ld, const int32_t* pad_offsets, int num_experts,
             int64_t row_capacity, int64_t cols, float* out, int64_t ldo, int dtype, void* workspace,
             size_t workspace_bytes, void* stream);

/* ESMM and ESS of its output in one pass.  No counterpart as a single call: the reference computes the hidden
 * gradient and then sums it per expert in its fused backward kernel (task 2 of launch_fused_grad_bias_*,
 * kernels/fused.py:111-141, reading the gradient back).  Arguments up to `engine` are hexa_esmm's.  Additionally
 * sums[e,:] (fp32 [E, n_out], ld_sums) = sum over expert e's rows of c as it was stored (after rounding to the 16-bit
 * type), i.e. what hexa_ess(c, ...) returns up to the order of the fp32 additions.  On the tcgen05 engine the epilogue
 * adds up every 128-row block while it is staged for its store, so c is not read again; otherwise the call runs
 * hexa_esmm and hexa_ess one after the other.  workspace: hexa_ess_workspace_bytes(row_capacity, n_out).
 * Deterministic (fixed order of additions). */
int hexa_esmm_ess(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                  const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                  const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                  const int32_t* pair_block, int num_experts, int64_t row_capacity, int64_t n_out, int64_t k,
                  int dtype, int epilogue, int act, int engine, float* sums, int64_t ld_sums, void* workspace,
                  size_t workspace_bytes, void* stream);

/* ESS without caller-provided scratch.  No counterpart in the reference (its launchers cudaMalloc their
 * own scratch on every call, kernels/shared_cuda_core.cu:304-309).  Same result as hexa_ess, bit for bit,
 * but pass 1's partial sums live in a fixed 32 MiB array inside the library, so the call allocates nothing
 * and needs no workspace argument.  It is meant for callers that cannot get device memory where the call
 * is made: code running inside an allocator-free region (a custom autograd node or a framework callback
 * that must not touch the caching allocator), or a plain-C host that holds only the input and output
 * pointers it was handed.  Limits and caveats:
 *   - ceil(row_capacity/128) * cols * 4 bytes must fit in hexa_ess_static_capacity_bytes(); larger requests
 *     fail with HEXA_ERR_WORKSPACE and a message naming both sizes (use hexa_ess then);
 *   - every GPU that loads the library holds the 32 MiB until the process exits;
 *   - all calls on a device share the one array: two calls that may overlap on the GPU (different streams)
 *     race - serialise them; contents from the previous call are left behind and never read;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call outside any stream capture. */
size_t hexa_ess_static_capacity_bytes(void);
int hexa_ess_static(const void* src, int64_t src_ld, const int32_t* pad_offsets, int num_experts,
                    int64_t row_capacity, int64_t cols, float* out, int64_t ldo, int dtype, void* stream);

/* ---- SM-free collectives over NVLink peer memory (no counterpart in the reference, which calls NCCL through
 *      torch.distributed for everything) ---- */

/* The stream waits until *addr >= value (cuStreamWaitValue32).  With one word per peer, written by the peer with a
 * 4-byte hexa_copy_2d into this GPU's memory, this is a barrier between ranks that needs no kernel. */
int hexa_stream_wait_value(const int32_t* addr, int32_t value, void* stream);

/* out[i] = (local[i] + sum_{s<n_recv} recv[s*elems + i]) / world, fp32 accumulation, 16-byte vectors: the reduction
 * step of a reduce-scatter(AVG) whose transfers were peer copies.  elems must be a multiple of 16/sizeof(dtype). */
int hexa_mean_slices(const void* local, const void* recv, int n_recv, int64_t elems, int world, void* out, int dtype,
                     void* stream);

/* ---- the step before routing: softmax + top-k + GShard auxiliary loss ---------------------------------------------
 * Replaces the reference's chain softmax -> torch.topk -> int64 -> int32 casts -> gshard_loss
 * (hexa_moe_triton/hexa_moe/impls/cascaded_moe.py:568-598, impls/layers.py:480-489, impls/losses.py:12-19) for
 * float32 logits [num_tokens, num_experts] (leading dimension ld), 1 <= num_experts <= hexa_gate_max_experts().
 *   ids          int32 [top_k, num_tokens], route-major: ids[j*num_tokens + t] = expert of token t's j-th choice,
 *                descending score, lowest expert id on ties (what hexa_route reads with stride_k = num_tokens)
 *   mass         float [num_experts]: column sums of softmax(logits)
 *   first_count  int32 [num_experts]: tokens whose first choice is the expert
 *   loss         float [1]: (E/T^2) * sum_e mass_e * first_count_e
 * All four are overwritten.  Every floating-point sum has a fixed order (per-warp, per-block and per-grid partials added
 * by index), so mass and loss are bit-identical from run to run.  A NaN score ranks below every number: a row of
 * NaN / inf logits still yields top_k distinct ids in [0, num_experts) (the lowest free ones) and NaN in mass / loss.
 * workspace: hexa_gate_workspace_bytes() bytes of 16-byte aligned device memory, contents irrelevant. */
int hexa_gate_max_experts(void);
size_t hexa_gate_workspace_bytes(void);
int hexa_gate_topk(const float* logits, int64_t ld, int64_t num_tokens, int num_experts, int top_k, int32_t* ids,
                   float* mass, int32_t* first_count, float* loss, void* workspace, size_t workspace_bytes, void* stream);

/* dlogits[t,e] = d loss / d logits[t,e] * dloss[0] for the loss of hexa_gate_topk: the softmax is recomputed from the
 * logits, first_count is the forward's output, dloss a float in device memory (the upstream gradient).
 * (What autograd derives for impls/losses.py:12-19 through F.softmax.) */
int hexa_gate_loss_grad(const float* logits, int64_t ld, int64_t num_tokens, int num_experts, const int32_t* first_count,
                        const float* dloss, float* dlogits, int64_t ldd, void* stream);

/* The same step for the other auxiliary loss of the reference, the load-importance loss (impls/losses.py:21-43, selected by
 * is_gshard_loss=False; needs gate noise): ids = top-k of the NOISY logits (what torch.topk of softmax(noisy) returns),
 *   importance[e] = sum_t softmax(logits)[t,e],   load[e] = sum_t Phi((softmax(logits)[t,e] - thr_t) / sigma),
 *   thr_t = k-th largest noisy logit of token t, sigma = gate_noise / num_experts,
 *   loss = (cv2(importance) + cv2(load)) / 2 with cv2(v) = var_unbiased(v) / (mean(v)^2 + 1e-10)
 * (the reference compares a score with a logit in `load`; kept as it is).  logits and logits_w_noise are float32
 * [num_tokens, num_experts] with the same leading dimension; sums in fixed order (bit-identical from run to run);
 * workspace as for hexa_gate_topk.  The gradient entry point recomputes softmax, top-k and the normal density from the two
 * logit tensors and the forward's importance / load totals; dloss is a float in device memory. */
int hexa_gate_topk_load_importance(const float* logits, const float* logits_w_noise, int64_t ld, int64_t num_tokens,
                                   int num_experts, int top_k, float sigma, int32_t* ids, float* importance, float* load,
                                   float* loss, void* workspace, size_t workspace_bytes, void* stream);
int hexa_gate_load_importance_grad(const float* logits, const float* logits_w_noise, int64_t ld, int64_t num_tokens,
                                   int num_experts, int top_k, float sigma, const float* importance, const float* load,
                                   const float* dloss, float* dlogits, int64_t ldd, void* stream);

/* Elementwise helper on sorted rows for activations the epilogue does not know:
 * dst[r,:] = row_token[r] >= 0 ? src[r,:] : 0 (restores the zero-pad-row invariant). */
int hexa_mask_pad_rows(void* buf, int64_t ld, const int32_t* row_token, const int32_t* pad_offsets,
                       int num_experts, int64_t row_capacity, int64_t cols, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HEXA_MOE_B200_H */
