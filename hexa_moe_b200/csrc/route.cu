// Routing: segment the T*top_k routed rows into contiguous, padded per-expert segments.
//
// Three launches, no host synchronisation, deterministic (equal to a stable sort by expert):
//   1. route_hist    each warp histograms one chunk of kRowsPerWarp routed rows
//   2. route_scan    one block: per-expert exclusive scan over chunks, per-expert totals, padded
//                    segment offsets, tile -> expert table, -1 in the pad slots
//   3. route_scatter each warp re-reads its chunk and places every row at
//                    pad_offsets[e] + (rows of e in earlier chunks) + (rows of e earlier in the chunk)
// HBM traffic: ids are read twice (8 B per routed row), row_token and token_row written once.
#include <stdarg.h>
#include <stdlib.h>

#include "hexa_common.cuh"

namespace hexa {
namespace {

constexpr int kRowsPerWarp = 512;
constexpr int kMaxExperts = 4096;  // keeps both shared-memory tables under 48 KB

__device__ __forceinline__ int load_id(const int32_t* ids, int64_t f, int64_t T, int64_t stride_t, int64_t stride_k) {
  int64_t j = f / T;
  int64_t t = f - j * T;
  return ids[t * stride_t + j * stride_k];
}

__global__ void route_hist(const int32_t* __restrict__ ids, int64_t T, int64_t n_rows, int64_t stride_t,
                           int64_t stride_k, int E, int32_t* __restrict__ chunk_hist) {
  extern __shared__ int32_t sm[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* h = sm + warp * E;
  for (int e = lane; e < E; e += 32) h[e] = 0;
  __syncwarp();
  const int64_t chunk = (int64_t)blockIdx.x * warps + warp;
  const int64_t begin = chunk * kRowsPerWarp;
  if (begin < n_rows) {
    const int64_t end = min(begin + (int64_t)kRowsPerWarp, n_rows);
    for (int64_t f = begin + lane; f < end; f += 32) {
      int e = load_id(ids, f, T, stride_t, stride_k);
      if (e >= 0 && e < E) atomicAdd(&h[e], 1);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) chunk_hist[chunk * E + e] = h[e];
  }
}

__global__ void __launch_bounds__(1024)
route_scan(int32_t* __restrict__ chunk_hist, int64_t n_chunks, int E, int align, int64_t row_capacity,
           int32_t* __restrict__ counts, int32_t* __restrict__ seg_offsets, int32_t* __restrict__ pad_offsets,
           int32_t* __restrict__ row_token, int32_t* __restrict__ tile_expert, int32_t* __restrict__ pair_off,
           int32_t* __restrict__ pair_block, int64_t pair_cap) {
  extern __shared__ int32_t sm[];
  int32_t* s_cnt = sm;          // [E]
  int32_t* s_pad = sm + E;      // [E + 1]
  // per-expert exclusive scan over chunks (thread per expert: coalesced across experts)
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int32_t run = 0;
    int64_t c = 0;
    for (; c + 4 <= n_chunks; c += 4) {
      int32_t v0 = chunk_hist[(c + 0) * E + e], v1 = chunk_hist[(c + 1) * E + e];
      int32_t v2 = chunk_hist[(c + 2) * E + e], v3 = chunk_hist[(c + 3) * E + e];
      chunk_hist[(c + 0) * E + e] = run; run += v0;
      chunk_hist[(c + 1) * E + e] = run; run += v1;
      chunk_hist[(c + 2) * E + e] = run; run += v2;
      chunk_hist[(c + 3) * E + e] = run; run += v3;
    }
    for (; c < n_chunks; ++c) {
      int32_t v = chunk_hist[c * E + e];
      chunk_hist[c * E + e] = run; run += v;
    }
    s_cnt[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  // exclusive scans over experts (unpadded and padded) by warp 0, 32 experts per step
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int32_t carry_seg = 0, carry_pad = 0, carry_pair = 0;
    for (int base = 0; base < E; base += 32) {
      int e = base + lane;
      int32_t c = e < E ? s_cnt[e] : 0;
      int32_t p = (c + align - 1) / align * align;
      int32_t q = (p / kRowTile + 1) / 2;      // pair tiles: two 128-row blocks each, the last one may be half empty
      int32_t ic = c, ip = p, iq = q;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int32_t tc = __shfl_up_sync(0xffffffffu, ic, o), tp = __shfl_up_sync(0xffffffffu, ip, o);
        int32_t tq = __shfl_up_sync(0xffffffffu, iq, o);
        if (lane >= o) { ic += tc; ip += tp; iq += tq; }
      }
      if (e < E) {
        seg_offsets[e] = carry_seg + ic - c;
        int32_t po = carry_pad + ip - p;
        pad_offsets[e] = po;
        s_pad[e] = po;
        if (pair_block) pair_off[e] = carry_pair + iq - q;
      }
      carry_seg += __shfl_sync(0xffffffffu, ic, 31);
      carry_pad += __shfl_sync(0xffffffffu, ip, 31);
      carry_pair += __shfl_sync(0xffffffffu, iq, 31);
    }
    if (lane == 0) {
      seg_offsets[E] = carry_seg;
      pad_offsets[E] = carry_pad;
      s_pad[E] = carry_pad;
      if (pair_block) pair_off[E] = carry_pair;
    }
  }
  __syncthreads();
  // pair-tile list for CTA-pair GEMMs: entry = (first 128-row block) * 2 + (the next block belongs to the same expert)
  if (pair_block) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int32_t b0 = s_pad[e] / kRowTile, nb = (s_pad[e + 1] - s_pad[e]) / kRowTile;
      int32_t o = pair_off[e];
      for (int32_t i = 0; i < nb; i += 2, ++o)
        if (o < pair_cap) pair_block[o] = (b0 + i) * 2 + (i + 1 < nb ? 1 : 0);
    }
    const int32_t total = pair_off[E];
    for (int64_t i = total + threadIdx.x; i < pair_cap; i += blockDim.x) pair_block[i] = -1;
  }
  // tile -> expert: binary search for the segment that holds the tile's first row
  const int64_t n_tiles = row_capacity / align;
  const int32_t n_pad = s_pad[E];
  for (int64_t i = threadIdx.x; i < n_tiles; i += blockDim.x) {
    int32_t row = (int32_t)(i * align);
    int32_t val = -1;
    if (row < n_pad) {
      int lo = 0, hi = E;  // largest e with s_pad[e] <= row (empty experts share an offset: take the last)
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (s_pad[mid] <= row) lo = mid; else hi = mid;
      }
      val = lo;
    }
    tile_expert[i] = val;
  }
  // pad slots of every segment
  for (int64_t i = threadIdx.x; i < (int64_t)E * align; i += blockDim.x) {
    int e = (int)(i / align), o = (int)(i % align);
    int32_t slot = s_pad[e] + s_cnt[e] + o;
    if (slot < s_pad[e + 1]) row_token[slot] = -1;
  }
}

__global__ void route_scatter(const int32_t* __restrict__ ids, int64_t T, int top_k, int64_t n_rows, int64_t stride_t,
                              int64_t stride_k, int E, const int32_t* __restrict__ chunk_base,
                              const int32_t* __restrict__ pad_offsets, int32_t* __restrict__ row_token,
                              int32_t* __restrict__ token_row) {
  extern __shared__ int32_t sm[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int32_t* cur = sm + warp * E;
  const int64_t chunk = (int64_t)blockIdx.x * warps + warp;
  const int64_t begin = chunk * kRowsPerWarp;
  if (begin >= n_rows) return;  // whole warp leaves together
  for (int e = lane; e < E; e += 32) cur[e] = pad_offsets[e] + chunk_base[chunk * E + e];
  __syncwarp();
  const int64_t end = min(begin + (int64_t)kRowsPerWarp, n_rows);
  for (int64_t f0 = begin; f0 < end; f0 += 32) {
    const int64_t f = f0 + lane;
    int e = -1;
    int64_t j = 0, t = 0;
    if (f < end) {
      j = f / T; t = f - j * T;
      e = ids[t * stride_t + j * stride_k];
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int32_t pos = -1;
    if (e >= 0) pos = cur[e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) cur[e] += __popc(peers);
    __syncwarp();
    if (f < end) {
      token_row[t * top_k + j] = pos;
      if (pos >= 0) row_token[pos] = (int32_t)t;
    }
  }
}

}  // namespace

// ---- error plumbing shared by every translation unit ------------------------------------------
static thread_local char g_err[512] = "no error";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

// Status words are per device, not per host thread: the kernels of one training step are launched from the
// Python thread (forward) and from the autograd engine's thread (backward), and both must report to the same word.
struct StatusSlot {
  int32_t* word;        // where kernels store their code (device-accessible)
  int host_readable;    // the word lives in pinned host memory: entry points can look at it before they launch
};
static StatusSlot g_status[64];
static uint64_t g_wait_limit_ns = 2000000000ull;
static int g_tc_debug = -1;

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  return dev;
}
int32_t* status_word() {
  const int dev = current_device();
  return dev < 0 ? nullptr : __atomic_load_n(&g_status[dev].word, __ATOMIC_ACQUIRE);
}
int status_pending() {
  const int dev = current_device();
  if (dev < 0) return 0;
  int32_t* w = __atomic_load_n(&g_status[dev].word, __ATOMIC_ACQUIRE);
  if (!w || !g_status[dev].host_readable) return 0;
  return (int)*reinterpret_cast<volatile int32_t*>(w);
}
uint64_t wait_limit_ns() { return g_wait_limit_ns; }
int tc_debug_flags() {
  if (g_tc_debug < 0) {
    const char* s = getenv("HEXA_TC_DEBUG");
    g_tc_debug = s ? atoi(s) : 0;
  }
  return g_tc_debug;
}

static int g_sm_limit = 0;
int sm_limit() { return g_sm_limit; }

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace hexa

using namespace hexa;

extern "C" int hexa_version(void) { return 100; }
extern "C" int hexa_set_sm_limit(int n) {
  hexa::g_sm_limit = n > 0 ? n : 0;
  return HEXA_OK;
}
extern "C" const char* hexa_last_error_string(void) { return hexa::g_err; }
extern "C" int hexa_set_status_word(int32_t* status) {
  const int dev = hexa::current_device();
  HEXA_REQUIRE(dev >= 0, "hexa_set_status_word: no current CUDA device (or ordinal >= 64)");
  int host = 0;
  if (status) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, status) == cudaSuccess) host = at.type == cudaMemoryTypeHost;
    else (void)cudaGetLastError();
  }
  hexa::g_status[dev].host_readable = host;
  __atomic_store_n(&hexa::g_status[dev].word, status, __ATOMIC_RELEASE);
  return HEXA_OK;
}
extern "C" int hexa_pending_device_status(void) { return hexa::status_pending(); }
extern "C" int hexa_set_wait_limit_ns(uint64_t ns) {
  HEXA_REQUIRE(ns >= 1000, "hexa_set_wait_limit_ns: the limit must be at least 1000 ns");
  hexa::g_wait_limit_ns = ns;
  return HEXA_OK;
}
extern "C" int hexa_set_tc_debug(int flags) {
  HEXA_REQUIRE(flags >= 0 && flags < 64, "hexa_set_tc_debug: flags must be a combination of bits 0..5");
  hexa::g_tc_debug = flags;
  return HEXA_OK;
}

extern "C" int64_t hexa_route_row_capacity(int64_t T, int top_k, int E, int align) {
  if (T < 0 || top_k <= 0 || E <= 0 || align <= 0) return -1;
  int64_t cap = T * top_k + (int64_t)E * (align - 1);
  return ceil_div(cap, align) * align;
}

extern "C" size_t hexa_route_workspace_bytes(int64_t T, int top_k, int E) {
  if (T < 0 || top_k <= 0 || E <= 0) return 0;
  int64_t chunks = ceil_div(T * top_k, kRowsPerWarp);
  if (chunks < 1) chunks = 1;
  return ((size_t)chunks * (size_t)E + (size_t)E + 1) * sizeof(int32_t);   // per-chunk histograms + pair-tile offsets
}

extern "C" int64_t hexa_route_pair_capacity(int64_t T, int top_k, int E) {
  const int64_t cap = hexa_route_row_capacity(T, top_k, E, kRowTile);
  if (cap < 0) return -1;
  return cap / (2 * kRowTile) + E + 1;   // every expert may end on a half-filled pair; one terminator
}

extern "C" int hexa_route(const int32_t* ids, int64_t T, int top_k, int64_t stride_t, int64_t stride_k, int E,
                          int align, int32_t* counts, int32_t* seg_offsets, int32_t* pad_offsets,
                          int32_t* row_token, int32_t* token_row, int32_t* tile_expert, int32_t* pair_block,
                          void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  HEXA_REQUIRE(T >= 0 && top_k > 0 && E > 0 && E <= kMaxExperts && align > 0, "hexa_route: bad sizes T=%lld k=%d E=%d align=%d",
               (long long)T, top_k, E, align);
  HEXA_REQUIRE(T * top_k + (int64_t)E * align < (int64_t)INT32_MAX, "hexa_route: too many rows for int32 indices");
  HEXA_REQUIRE(counts && seg_offsets && pad_offsets && row_token && token_row && tile_expert && workspace,
               "hexa_route: null output or workspace pointer");
  HEXA_REQUIRE(T == 0 || ids, "hexa_route: null ids");
  const size_t need = hexa_route_workspace_bytes(T, top_k, E);
  if (workspace_bytes < need) {
    set_error("hexa_route: workspace %zu bytes < required %zu", workspace_bytes, need);
    return HEXA_ERR_WORKSPACE;
  }
  const int64_t n_rows = T * top_k;
  const int64_t n_chunks = ceil_div(n_rows, kRowsPerWarp);
  const int64_t row_cap = hexa_route_row_capacity(T, top_k, E, align);
  int32_t* chunk_hist = (int32_t*)workspace;
  int warps = (int)(48 * 1024 / (4 * (int64_t)E));
  warps = warps < 1 ? 1 : (warps > 8 ? 8 : warps);
  const size_t smem = (size_t)warps * E * sizeof(int32_t);
  if (n_chunks > 0) {
    route_hist<<<(unsigned)ceil_div(n_chunks, warps), warps * 32, smem, stream>>>(ids, T, n_rows, stride_t, stride_k, E,
                                                                                chunk_hist);
    HEXA_LAUNCH_CHECK("route_hist");
  }
  HEXA_REQUIRE(pair_block == nullptr || align == kRowTile, "hexa_route: the pair-tile list needs align = %d", kRowTile);
  int32_t* pair_off = chunk_hist + (size_t)(n_chunks > 0 ? n_chunks : 1) * E;
  route_scan<<<1, 1024, (2 * (size_t)E + 1) * sizeof(int32_t), stream>>>(
      chunk_hist, n_chunks, E, align, row_cap, counts, seg_offsets, pad_offsets, row_token, tile_expert, pair_off, pair_block,
      pair_block ? hexa_route_pair_capacity(T, top_k, E) : 0);
  HEXA_LAUNCH_CHECK("route_scan");
  if (n_chunks > 0) {
    route_scatter<<<(unsigned)ceil_div(n_chunks, warps), warps * 32, smem, stream>>>(
        ids, T, top_k, n_rows, stride_t, stride_k, E, chunk_hist, pad_offsets, row_token, token_row);
    HEXA_LAUNCH_CHECK("route_scatter");
  }
  return HEXA_OK;
}
