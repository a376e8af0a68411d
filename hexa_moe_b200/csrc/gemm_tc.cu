// tcgen05 / TMEM / TMA grouped GEMMs on the sorted-row layout (sm_100a only):
//   ESMM   c[r,:]  = a[r,:] x b[expert(r)]   (b K-major "NK" or N-major "KN"), fused bias / activation /
//                    activation-derivative epilogue, pad rows written as zeros
//   ESTMM  out[e]  = p_e^T x q_e             (contraction over the expert's ragged row segment; both
//                    operands are MN-major in shared memory, no transposed copy is ever made)
//
// Persistent kernel, static tile list.  Two flavours of the same code (template parameter CTAS):
//   CTAS = 1  one CTA per SM computes a 128 x BN tile (tcgen05 cta_group::1)
//   CTAS = 2  a cluster of two CTAs on neighbouring SMs computes a 256 x 256 tile (cta_group::2): each CTA
//             loads its own 128 rows of A and only HALF of the B tile, the pair's MMA reads both halves, and
//             each CTA keeps its 128 x 256 accumulator in its own TMEM.  Shared-memory fill traffic per MMA
//             drops from 48 KB to 32 KB per SM per 64-deep k-block, which is what bounds the 1-CTA kernel.
//             No TMA multicast is used.
// Warp roles in every CTA:
//   warp 0      TMA producer: 128B-swizzled k-blocks of A and B into a ring of shared-memory stages
//   warp 1      MMA issuer (only in the pair's leader CTA when CTAS = 2): one thread issues tcgen05.mma
//               (K = 16 per instruction) into one of two TMEM accumulators; tcgen05.commit frees ring slots
//               and publishes finished accumulators (multicast to both CTAs of a pair)
//   warps 2..   epilogue (EW = 16 or 8 warps, template parameter): tcgen05.ld of the accumulator (lane quadrant =
//               warp % 4, each group of four warps owns a column range), fused epilogue math; ESMM results go through
//               a 64B-swizzled staging tile and one TMA store per 128x32 block, ESTMM stores from registers.  The
//               MMA and producer threads share their issue slots with the epilogue warps of their sub-partition:
//               16 warps finish a tile's epilogue sooner (short k-loops), 8 leave the role threads more slots
// so the epilogue of tile i overlaps the MMAs of tile i+1.  Every mbarrier wait is bounded: after ~2 s a CTA
// raises an abort flag, records a code in the status word and drains; both CTAs of a pair always reach the
// closing cluster barrier.
//
// Segments are aligned to 128 rows, so an ESMM row block never straddles two experts and an ESTMM k-block
// (64 rows) never reads another expert's rows; pad rows hold zeros and add nothing.  A pair tile takes two
// consecutive row blocks of the same expert (list built by the routing step); an expert with an odd number of
// blocks leaves the second CTA of its last pair without rows to store.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdlib.h>

#include "gemm_launch.h"
#include "hexa_common.cuh"

namespace hexa {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;   // one 128-byte swizzle span of 16-bit elements
constexpr int UMMA_K = 16;
constexpr uint32_t kABytes = BLOCK_M * BLOCK_K * 2;  // 16 KB

enum Mode { ESMM_NK = 0, ESMM_KN = 1, ESTMM = 2 };

struct Params {
  const int32_t* tile_expert;
  const int32_t* pad_offsets;
  const int32_t* row_token;
  const int32_t* pair_block;   // CTAS = 2, ESMM: per pair tile (first 128-row block) * 2 + (second block belongs to the same expert), -1 ends the list
  int64_t max_pairs;
  const float* bias;
  int64_t ldbias;
  void* aux;
  int64_t ldaux;
  void* c;          // ESMM: c ; ESTMM: out
  int64_t ldc;
  int64_t c_estride;  // ESTMM only
  int64_t m_split, split_stride;  // ESTMM: output row m lives at (m / m_split) * split_stride + (m % m_split) * ldc
  void* c_split[16];  // ESTMM, n_split > 0: slice m / m_split of the output goes to this base instead (it may be
  int n_split;        // another GPU's memory: the reduce-scatter layout written straight into the owners' buffers)
  int64_t n;        // output columns
  int64_t k;        // ESMM: contraction length ; ESTMM: unused
  int64_t m;        // ESTMM: output rows per expert
  int E;
  uint32_t nt;          // tile columns of the output: ceil(n / BN)
  uint32_t per_expert;  // ESTMM: tiles per expert = tile rows x tile columns x splits
  uint32_t total_tiles; // ESTMM: E x per_expert ; ESMM single-CTA: unused (the row count is device-side)
  int e_begin, e_end;   // ESMM: only tiles of experts in [e_begin, e_end) are computed by this launch
  int epilogue, act;
  int is_bf16;      // 16-bit flavour of the inputs (and of 16-bit outputs)
  int out_f32;      // ESTMM: fp32 output
  int beta;         // ESTMM: accumulate into out
  int splits;       // ESTMM: > 1 = every expert's row segment is cut into this many chunks, each its own tile, whose fp32
  float* partial;   //        partial results [splits, E, m, n] go here and are added in chunk order by estmm_reduce_kernel
  float* colsum;    // ESMM, optional: fp32 [row_capacity / 128, n]; row b receives the column sums of the 128 output rows
                    // of block b, taken from the values as they are stored (after rounding to the 16-bit type)
  int debug;        // measurement / test aid (HEXA_TC_DEBUG, hexa_set_tc_debug): bit 0 = the producer skips the TMA loads and
                    // arrives in their place, bit 1 = the MMA thread skips the MMAs, bit 2 = the producer neither loads
                    // nor arrives, so that every wait of the pipeline runs into its limit
  int32_t* status;
  uint64_t wait_limit_ns;   // limit of every mbarrier wait (hexa_set_wait_limit_ns; default 2 s)
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that lets the hardware park the thread for up to ~`hint_ns` before it reports "not yet"
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The status word may live in device memory or in pinned host memory (where the host can poll it without a copy), so
// it is written with plain stores: the first code to arrive stays, and which of two simultaneous codes wins is immaterial.
__device__ __forceinline__ void report_status(int32_t* status, int code) {
  if (status) {
    volatile int32_t* s = status;
    if (*s == 0) *s = code;
    __threadfence_system();
  }
}

// Bounded wait.  Returns false when this CTA is aborting (its own limit ran out or another role's did).
__device__ __noinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status, int code,
                                       uint64_t limit_ns) {
  uint32_t spins = 0;
  uint64_t t0 = 0;
  while (!mbar_try_wait_hint(bar, parity, 4000u)) {
    if ((++spins & 0xF) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        report_status(status, code);
        return false;
      }
    }
  }
  return true;
}

// Fast path of a bounded wait: one try_wait inline, the timed loop only when the barrier is not ready yet.
__device__ __forceinline__ bool mbar_wait_fast(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status, int code,
                                               uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait(bar, parity, abort_flag, status, code, limit_ns);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
// bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
// [46,48) version, [61,64) layout type (2 = SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int is_bf16) {
  if (is_bf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float unpack_lo(uint32_t w, int is_bf16) {
  if (is_bf16) return __uint_as_float(w << 16);
  return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
}
__device__ __forceinline__ float unpack_hi(uint32_t w, int is_bf16) {
  if (is_bf16) return __uint_as_float(w & 0xFFFF0000u);
  return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}


// ---- cluster / cta_group::2 helpers -------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: data lands in the issuing CTA's shared memory, the byte count is credited to the
// mbarrier at `bar_cluster_addr` (the leader CTA's).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* dst, const CUtensorMap* tm, uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

template <int BN, int CTAS, int EW, int MODE> struct Cfg {
  static constexpr int kThreads = 32 * (2 + EW);
  // ESTMM stores from registers and needs no staging tile: its ring gets the space (one more 32 KB slot), which is what
  // a loop bounded by the latency of a ring slot's round trip (MMA done -> slot refilled) converts into throughput
#ifndef HEXA_TC_RING_SLOTS      // build-time override for experiments with the ring depth (0 = the defaults below)
#define HEXA_TC_RING_SLOTS 0
#endif
#ifndef HEXA_TC_SMEM_SLACK      // bytes kept for aligning the dynamic shared memory base to 1 KB by hand
#define HEXA_TC_SMEM_SLACK 1024
#endif
  static constexpr int kStages = (BN == 256 && CTAS == 1) ? 4 : (HEXA_TC_RING_SLOTS ? HEXA_TC_RING_SLOTS : (MODE == ESTMM ? 7 : 6));
  static constexpr uint32_t kBBytes = (BN / CTAS) * BLOCK_K * 2;   // this CTA's share of the B tile
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators; 256 or 512, a power of two
  static constexpr uint32_t kStoreBufBytes = 128 * 64;   // [128 rows x 32 16-bit columns]
  static constexpr uint32_t kStoreBytes = MODE == ESTMM ? 0 : (EW / 4) * kStoreBufBytes;  // one buffer per group of four epilogue warps
  static constexpr size_t kSmemBytes = HEXA_TC_SMEM_SLACK + (size_t)kStages * kStageBytes + kStoreBytes + 256 /*barriers*/;
  static_assert(kSmemBytes <= 232448, "more shared memory than one CTA can have (227 KB)");
};

struct Tile {
  int e;          // expert
  int row0;       // ESMM: first sorted row of this CTA's block ; ESTMM: first row of the expert's segment
  int col0;       // first output column of the tile
  int m0;         // ESTMM: first output row of this CTA's block
  int num_kb;     // k-blocks to accumulate
  int valid;      // this CTA has rows to store (the second CTA of a pair may not)
  int skip;       // ESMM: the tile's expert is outside the launch's expert range (every role skips it alike)
  int split;      // ESTMM with splits > 1: which chunk of the segment this tile covers
};

// Tile t of the static list, as seen by CTA `rank` of its pair (rank = 0 when CTAS = 1).  Returns false past the end.
// The tile index and every quantity it is divided by are 32-bit (the host checks the tile count): the lookup runs once
// per tile in each of the three roles, two of which are single threads that the tensor pipe waits for, and a 64-bit
// division is a ~100-instruction sequence.
template <int BN, int MODE, int CTAS>
__device__ __forceinline__ bool get_tile(const Params& p, uint32_t t, int rank, Tile& tile) {
  if (MODE == ESTMM) {
    if (t >= p.total_tiles) return false;
    const uint32_t S = (uint32_t)p.splits;
    const uint32_t e = t / p.per_expert;
    const uint32_t in_e = t - e * p.per_expert;
    const uint32_t rem = in_e / S;
    const uint32_t c = in_e - rem * S;
    const uint32_t mrow = rem / p.nt;
    tile.e = (int)e;
    tile.m0 = ((int)mrow * CTAS + rank) * BLOCK_M;
    tile.col0 = (int)(rem - mrow * p.nt) * BN;
    const int seg0 = p.pad_offsets[e];
    const int kb_all = (p.pad_offsets[e + 1] - seg0) / BLOCK_K;
    const int kb_per = (kb_all + (int)S - 1) / (int)S;       // chunks of equal length, the last ones may be short or empty
    const int kb0 = (int)c * kb_per;
    tile.row0 = seg0 + kb0 * BLOCK_K;
    tile.num_kb = max(0, min(kb_per, kb_all - kb0));
    tile.split = (int)c;
    tile.skip = 0;
    tile.valid = tile.m0 < p.m;
    return true;
  } else {
    const uint32_t row_tile = t / p.nt;          // pair index (CTAS = 2) or 128-row block
    uint32_t mb;
    if (CTAS == 2) {
      if (row_tile >= (uint32_t)p.max_pairs) return false;
      const int pb = p.pair_block[row_tile];
      if (pb < 0) return false;
      mb = (uint32_t)(pb >> 1);
      tile.e = p.tile_expert[mb];
      tile.valid = rank == 0 || (pb & 1);
      mb += (uint32_t)rank;
    } else {
      const uint32_t mblocks = (uint32_t)(p.pad_offsets[p.E] / BLOCK_M);
      if (row_tile >= mblocks) return false;
      mb = row_tile;
      tile.e = p.tile_expert[mb];
      tile.valid = 1;
    }
    tile.row0 = (int)(mb * BLOCK_M);
    tile.col0 = (int)(t - row_tile * p.nt) * BN;
    tile.m0 = 0;
    tile.num_kb = (int)((p.k + BLOCK_K - 1) / BLOCK_K);
    tile.skip = tile.e < p.e_begin || tile.e >= p.e_end;
    return tile.e >= 0;
  }
}

// ---- epilogue staging: registers -> 64B-swizzled shared memory -> TMA store ------------------------
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tm), "r"(smem_u32(src)),
               "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One thread's row (32 columns = 64 B = four 16-byte chunks) into a [128 x 64 B] staging tile laid out
// as TMA's 64-byte swizzle expects: chunk c of row r lives at chunk c ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage_row(uint8_t* buf, int r, const uint32_t (&w)[16]) {
  uint8_t* row = buf + r * 64;
  const int x = (r >> 1) & 3;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(row + ((c ^ x) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

// Values of 16 columns of one row for the two possible outputs of the ESMM epilogue: y = acc + bias packed as it
// is (the saved pre-activation), o = the layer output of this GEMM.  Rows that are padding come out as zeros without a
// select per element: their accumulator is exactly zero (the A operand's pad rows are zeros), the caller has masked
// their bias, and every activation here maps 0 to 0 (the derivative epilogue multiplies the zero accumulator).  Working
// on 16 columns at a time keeps few enough values live for the compiler to interleave the independent activations.
template <int EPI, int ACT, int is_bf16>
__device__ __forceinline__ void epi_values16(const float (&f)[16], const uint16_t* xp, int ncols, uint32_t* y, uint32_t* o) {
  if (EPI == HEXA_EPI_DACT) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      // columns at or beyond ncols do not exist (the TMA store clips them): do not read aux there
      const uint4 a = g * 8 < ncols ? *reinterpret_cast<const uint4*>(xp + g * 8) : make_uint4(0, 0, 0, 0);
      const uint32_t* ap = reinterpret_cast<const uint32_t*>(&a);
#pragma unroll
      for (int i = 0; i < 4; ++i)
        o[4 * g + i] = pack2(f[8 * g + 2 * i] * act_grad_fast<ACT>(unpack_lo(ap[i], is_bf16)),
                             f[8 * g + 2 * i + 1] * act_grad_fast<ACT>(unpack_hi(ap[i], is_bf16)), is_bf16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (EPI == HEXA_EPI_ACT) {
        y[i] = pack2(f[2 * i], f[2 * i + 1], is_bf16);
        o[i] = pack2(act_fast<ACT>(f[2 * i]), act_fast<ACT>(f[2 * i + 1]), is_bf16);
      } else {
        o[i] = pack2(f[2 * i], f[2 * i + 1], is_bf16);
      }
    }
  }
}

template <int BN, int MODE, int CTAS, int EW>
__global__ void __launch_bounds__(32 * (2 + EW), 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX, const Params p) {
  using C = Cfg<BN, CTAS, EW, MODE>;
  constexpr int kEpiWarps = EW;
  constexpr int kStages = C::kStages;
  constexpr int BNH = BN / CTAS;          // B columns this CTA loads
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  if (HEXA_TC_SMEM_SLACK < 1024 && smem != smem_raw) {      // without slack the base itself must be 1 KB aligned
    if (threadIdx.x == 0) report_status(p.status, 9);
    return;                                                  // uniform: every thread of every CTA sees the same base offset
  }
  uint8_t* store_bufs = smem + (size_t)kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_bufs + C::kStoreBytes);
  uint64_t* full = bars;                  // [kStages]  producers -> MMA     (used in the leader CTA)
  uint64_t* empty = bars + kStages;       // [kStages]  MMA -> producer      (one per CTA, multicast commit)
  uint64_t* acc_full = bars + 2 * kStages;        // [2] MMA -> epilogue     (one per CTA, multicast commit)
  uint64_t* acc_empty = bars + 2 * kStages + 2;   // [2] epilogues -> MMA    (used in the leader CTA)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* group_abort = abort_flag + 1;   // [4]: one per group of four epilogue warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = CTAS == 2 ? (int)cluster_ctarank() : 0;    // 0 = leader of the pair
  const uint32_t tile_first = CTAS == 2 ? (blockIdx.x >> 1) : blockIdx.x;
  const uint32_t tile_step = CTAS == 2 ? (gridDim.x >> 1) : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], kEpiWarps * CTAS); }
    *abort_flag = 0;
    for (int g = 0; g < kEpiWarps / 4; ++g) group_abort[g] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the allocating warp also frees; with CTAS = 2 the same warp of both CTAs takes part
    if (CTAS == 2) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::kTmemCols) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (every CTA)
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      const uint32_t lead_full0 = CTAS == 2 ? map_to_cta(&full[0], 0) : 0u;   // the leader CTA's first full barrier
      for (uint32_t t = tile_first; ok && get_tile<BN, MODE, CTAS>(p, t, rank, tile); t += tile_step) {
        if (MODE != ESTMM && tile.skip) continue;
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!(ok = mbar_wait_fast(&empty[stage], phase ^ 1, abort_flag, p.status, 1, p.wait_limit_ns))) break;
          uint8_t* sA = smem + (size_t)stage * C::kStageBytes;
          uint8_t* sB = sA + kABytes;
          const int bcol = tile.col0 + rank * BNH;     // this CTA's share of the B columns
          if (p.debug & 4) {
            // nothing is loaded and nobody arrives: the consumers' waits run into their limit (error-path test)
          } else if (p.debug & 1) {   // results are garbage; only the timing of the remaining pipeline is of interest
            if (rank == 0) mbar_arrive(&full[stage]);
          } else if (CTAS == 2) {
            // bytes of both CTAs are credited to the leader's barrier; only the leader arms it
            const uint32_t lead_full = lead_full0 + 8u * (uint32_t)stage;
            if (rank == 0) mbar_expect_tx(&full[stage], 2 * C::kStageBytes);
            if (MODE == ESTMM) {
              const int r = tile.row0 + kb * BLOCK_K;
#pragma unroll
              for (int c = 0; c < BLOCK_M / 64; ++c) tma_load_2d_pair(sA + c * 8192, &tmA, lead_full, tile.m0 + c * 64, r);
#pragma unroll
              for (int c = 0; c < BNH / 64; ++c) tma_load_2d_pair(sB + c * 8192, &tmB, lead_full, bcol + c * 64, r);
            } else {
              tma_load_2d_pair(sA, &tmA, lead_full, kb * BLOCK_K, tile.row0);
              if (MODE == ESMM_NK) {
                tma_load_3d_pair(sB, &tmB, lead_full, kb * BLOCK_K, bcol, tile.e);
              } else {
#pragma unroll
                for (int c = 0; c < BNH / 64; ++c) tma_load_3d_pair(sB + c * 8192, &tmB, lead_full, bcol + c * 64, kb * BLOCK_K, tile.e);
              }
            }
          } else {
            mbar_expect_tx(&full[stage], C::kStageBytes);
            if (MODE == ESTMM) {
              const int r = tile.row0 + kb * BLOCK_K;
#pragma unroll
              for (int c = 0; c < BLOCK_M / 64; ++c) tma_load_2d(sA + c * 8192, &tmA, &full[stage], tile.m0 + c * 64, r);
#pragma unroll
              for (int c = 0; c < BNH / 64; ++c) tma_load_2d(sB + c * 8192, &tmB, &full[stage], bcol + c * 64, r);
            } else {
              tma_load_2d(sA, &tmA, &full[stage], kb * BLOCK_K, tile.row0);
              if (MODE == ESMM_NK) {
                tma_load_3d(sB, &tmB, &full[stage], kb * BLOCK_K, bcol, tile.e);
              } else {
#pragma unroll
                for (int c = 0; c < BNH / 64; ++c) tma_load_3d(sB + c * 8192, &tmB, &full[stage], bcol + c * 64, kb * BLOCK_K, tile.e);
              }
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr bool kAMn = (MODE == ESTMM), kBMn = (MODE != ESMM_NK);
      // instruction descriptor: fp32 accumulate, A/B format (0 = f16, 1 = bf16), majors, N>>3, M>>4
      // (M is 256 for a CTA pair: 128 rows from each CTA's shared memory into each CTA's TMEM)
      const uint32_t fmt = p.is_bf16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((kAMn ? 1u : 0u) << 15) | ((kBMn ? 1u : 0u) << 16) |
                             ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((BLOCK_M * CTAS) >> 4) << 24);
      // K-major: 8-row groups 1024 B apart (SBO), LBO unused (1).  MN-major: 64-element column chunks
      // BLOCK_K*128 B apart (LBO), 8-k groups 1024 B apart (SBO).
      const uint32_t a_lbo = kAMn ? BLOCK_K * 128 : 16, b_lbo = kBMn ? BLOCK_K * 128 : 16;
      // start-address advance per K=16 step, in 16-byte units: 32 B inside the swizzle row (K-major)
      // or two 8-k groups = 2048 B (MN-major)
      const uint32_t a_step = kAMn ? (2048u >> 4) : (32u >> 4);
      const uint32_t b_step = kBMn ? (2048u >> 4) : (32u >> 4);
      // The issuing thread is the pacemaker of the whole kernel: everything loop-invariant is hoisted so that a
      // k-block costs one try_wait, two 64-bit adds, four MMAs and one commit.
      const uint32_t s0 = smem_u32(smem);
      const uint64_t adesc0 = make_smem_desc(s0, a_lbo, 1024);
      const uint64_t bdesc0 = make_smem_desc(s0 + kABytes, b_lbo, 1024);
      constexpr uint64_t kStageDesc = C::kStageBytes >> 4;    // descriptor start-address units per ring slot
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      Tile tile;
      int it = -1;
      for (uint32_t t = tile_first; ok && get_tile<BN, MODE, CTAS>(p, t, rank, tile); t += tile_step) {
        if (MODE != ESTMM && tile.skip) continue;
        ++it;
        const int acc = it & 1;
        const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
        if (!(ok = mbar_wait_fast(&acc_empty[acc], acc_phase ^ 1, abort_flag, p.status, 2, p.wait_limit_ns))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < tile.num_kb; ++kb) {
          if (!(ok = mbar_wait_fast(&full[stage], phase, abort_flag, p.status, 3, p.wait_limit_ns))) break;
          const uint64_t adesc = adesc0 + (uint64_t)stage * kStageDesc;
          const uint64_t bdesc = bdesc0 + (uint64_t)stage * kStageDesc;
          if (!(p.debug & 2)) {
#pragma unroll
            for (int j = 0; j < BLOCK_K / UMMA_K; ++j) {
              if (CTAS == 2) umma_f16_pair(d_tmem, adesc + (uint64_t)(j * a_step), bdesc + (uint64_t)(j * b_step), idesc, j == 0 ? accumulate : 1u);
              else umma_f16(d_tmem, adesc + (uint64_t)(j * a_step), bdesc + (uint64_t)(j * b_step), idesc, j == 0 ? accumulate : 1u);
            }
          }
          accumulate = 1;
          // slot reusable (in both CTAs) once these MMAs have read it
          if (CTAS == 2) umma_commit_pair(&empty[stage]); else umma_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (tile.num_kb > 0) {
          if (CTAS == 2) umma_commit_pair(&acc_full[acc]); else umma_commit(&acc_full[acc]);
        } else {  // empty segment: nothing to wait for, the epilogues write zeros
          mbar_arrive(&acc_full[acc]);
          if (CTAS == 2) mbar_arrive_cluster(map_to_cta(&acc_full[acc], 1));
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (every CTA, its own 128 rows)
    constexpr int kParts = kEpiWarps / 4;   // groups of four warps; each group owns BN / kParts columns of every tile
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int part = (warp - 2) >> 2;
    const int is_bf16 = p.is_bf16;
    const bool leader = (q == 2) && lane == 0;   // the first warp of every group of four issues the group's TMA stores
    uint8_t* buf = store_bufs + (size_t)part * C::kStoreBufBytes;
    bool ok = true;
    Tile tile;
    int it = -1;
    for (uint32_t t = tile_first; ok && get_tile<BN, MODE, CTAS>(p, t, rank, tile); t += tile_step) {
      if (MODE != ESTMM && tile.skip) continue;
      ++it;
      const int acc = it & 1;
      const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
      // The four warps of a group meet at named barriers inside the tile, so they must leave together: each warp
      // publishes a failed wait, the group synchronises, and all four read the same verdict.
      if (!mbar_wait(&acc_full[acc], acc_phase, abort_flag, p.status, 4, p.wait_limit_ns) && lane == 0) group_abort[part] = 1;
      group_sync(1 + part);
      if (group_abort[part]) { ok = false; break; }
      tc_fence_after();
      const int rloc = q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int cc = 0; cc < BN / kParts / 32; ++cc) {
        const int cloc = part * (BN / kParts) + cc * 32;
        const int64_t gcol = (int64_t)tile.col0 + cloc;
        if (gcol >= p.n || !tile.valid) break;  // uniform across the four warps of a group
        if (MODE == ESTMM) {
          uint32_t v[32];
          if (tile.num_kb > 0) {
            tmem_ld32(t_row + (uint32_t)cloc, v);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          const int64_t mrow = (int64_t)tile.m0 + rloc;
          if (mrow < p.m && p.splits > 1) {
            // a chunk's partial result: plain fp32 [splits, E, m, n]
            float* o = p.partial + (((int64_t)tile.split * p.E + tile.e) * p.m + mrow) * p.n + gcol;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              if (gcol + g * 4 < p.n)
                *reinterpret_cast<float4*>(o + g * 4) = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]),
                                                                    __uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3]));
            }
          } else if (mrow < p.m) {
            if (p.out_f32) {
              float* o = (p.n_split ? reinterpret_cast<float*>(p.c_split[mrow / p.m_split])
                                    : reinterpret_cast<float*>(p.c) + (mrow / p.m_split) * p.split_stride) +
                         (int64_t)tile.e * p.c_estride + (mrow % p.m_split) * p.ldc + gcol;
#pragma unroll
              for (int g = 0; g < 8; ++g) {
                if (gcol + g * 4 < p.n) {
                  float4 w = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]),
                                         __uint_as_float(v[4 * g + 2]), __uint_as_float(v[4 * g + 3]));
                  if (p.beta) {
                    float4 old = *reinterpret_cast<float4*>(o + g * 4);
                    w.x += old.x; w.y += old.y; w.z += old.z; w.w += old.w;
                  }
                  *reinterpret_cast<float4*>(o + g * 4) = w;
                }
              }
            } else {
              uint16_t* o = (p.n_split ? reinterpret_cast<uint16_t*>(p.c_split[mrow / p.m_split])
                                       : reinterpret_cast<uint16_t*>(p.c) + (mrow / p.m_split) * p.split_stride) +
                            (int64_t)tile.e * p.c_estride + (mrow % p.m_split) * p.ldc + gcol;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (gcol + g * 8 < p.n) {
                  uint4 w;
                  uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
                  if (p.beta) {
                    uint4 old = *reinterpret_cast<uint4*>(o + g * 8);
                    const uint32_t* op = reinterpret_cast<const uint32_t*>(&old);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                      wp[i] = pack2(__uint_as_float(v[8 * g + 2 * i]) + unpack_lo(op[i], is_bf16),
                                    __uint_as_float(v[8 * g + 2 * i + 1]) + unpack_hi(op[i], is_bf16), is_bf16);
                  } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                      wp[i] = pack2(__uint_as_float(v[8 * g + 2 * i]), __uint_as_float(v[8 * g + 2 * i + 1]), is_bf16);
                  }
                  *reinterpret_cast<uint4*>(o + g * 8) = w;
                }
              }
            }
          }
        } else {
          const int64_t r = (int64_t)tile.row0 + rloc;
          // a pad row skips the bias, which is the only thing that could make it non-zero
          const bool live = p.row_token == nullptr || p.row_token[r] >= 0;
          uint32_t yv[16], ov[16];
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const int64_t hcol = gcol + hf * 16;
            const int ncols = (int)min((int64_t)16, p.n - hcol);   // <= 0: nothing of this half exists
            uint32_t v[16];
            tmem_ld16(t_row + (uint32_t)(cloc + hf * 16), v);      // ESMM tiles always have k-blocks
            float f[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) f[i] = __uint_as_float(v[i]);
            if (p.bias && ncols > 0 && live) {
              const float* bp = p.bias + (int64_t)tile.e * p.ldbias + hcol;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (g * 4 < ncols) {
                  const float4 bv = __ldg(reinterpret_cast<const float4*>(bp + g * 4));
                  f[4 * g] += bv.x; f[4 * g + 1] += bv.y; f[4 * g + 2] += bv.z; f[4 * g + 3] += bv.w;
                }
              }
            }
            const uint16_t* xp = p.aux ? reinterpret_cast<const uint16_t*>(p.aux) + r * p.ldaux + hcol : nullptr;
            uint32_t* yh = yv + hf * 8;
            uint32_t* oh = ov + hf * 8;
            // one specialisation per (epilogue, activation, 16-bit flavour): no per-element branches
#define HEXA_EPI_CASE(E_, A_)                                                                          \
  case E_ * 8 + A_:                                                                                    \
    if (is_bf16) epi_values16<E_, A_, 1>(f, xp, ncols, yh, oh);                                        \
    else epi_values16<E_, A_, 0>(f, xp, ncols, yh, oh);                                                \
    break;
            switch ((p.debug & 8) ? 99 : p.epilogue * 8 + p.act) {
              HEXA_EPI_CASE(HEXA_EPI_ACT, HEXA_ACT_RELU)
              HEXA_EPI_CASE(HEXA_EPI_ACT, HEXA_ACT_GELU)
              HEXA_EPI_CASE(HEXA_EPI_ACT, HEXA_ACT_GELU_TANH)
              HEXA_EPI_CASE(HEXA_EPI_ACT, HEXA_ACT_SILU)
              HEXA_EPI_CASE(HEXA_EPI_ACT, HEXA_ACT_NONE)
              HEXA_EPI_CASE(HEXA_EPI_DACT, HEXA_ACT_RELU)
              HEXA_EPI_CASE(HEXA_EPI_DACT, HEXA_ACT_GELU)
              HEXA_EPI_CASE(HEXA_EPI_DACT, HEXA_ACT_GELU_TANH)
              HEXA_EPI_CASE(HEXA_EPI_DACT, HEXA_ACT_SILU)
              default:
                if (is_bf16) epi_values16<HEXA_EPI_LINEAR, HEXA_ACT_NONE, 1>(f, xp, ncols, yh, oh);
                else epi_values16<HEXA_EPI_LINEAR, HEXA_ACT_NONE, 0>(f, xp, ncols, yh, oh);
                break;
            }
#undef HEXA_EPI_CASE
          }
          // registers -> swizzled staging tile -> one TMA store per 128x32 block (full 128-byte lines to L2)
          const bool two = (p.epilogue == HEXA_EPI_ACT) && p.aux != nullptr && !(p.debug & 16);
          for (int o = (p.debug & 32) ? 2 : (two ? 0 : 1); o < 2; ++o) {
            if (leader) bulk_wait_read<0>();   // the previous store has finished reading the buffer
            group_sync(1 + part);
            stage_row(buf, rloc, o == 0 ? yv : ov);
            fence_async_smem();
            group_sync(1 + part);
            if (leader) {
              tma_store_2d(o == 0 ? &tmX : &tmC, buf, (int)gcol, tile.row0);
              bulk_commit();
            }
          }
          if (p.colsum != nullptr && !(p.debug & 32)) {
            // Column sums of the block that now sits in the staging tile (the output as stored).  The warp whose TMEM
            // quadrant is q takes the 16-byte chunk q of every row: lane = (row mod 8) * 4 + 32-bit word within the
            // chunk (two columns), 16 rows per lane, then the eight row classes meet through three shuffles.  The eight
            // rows of one load fall into eight different groups of four banks (rows r, r+1 differ by 64 bytes, rows
            // r, r+2 by the swizzle): one conflict-free 128-byte wavefront per load.  Nothing else is synchronised:
            // every thread has finished reading before it arrives at the barrier that precedes the next write of the buffer.
            const int w4 = lane & 3, ro = lane >> 2;
            const uint8_t* src = buf + ro * 64 + ((q ^ ((ro >> 1) & 3)) << 4) + w4 * 4;   // (r >> 1) & 3 == (ro >> 1) & 3 for r = 8 i + ro
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t v = *reinterpret_cast<const uint32_t*>(src + i * 512);
              s0 += unpack_lo(v, is_bf16);
              s1 += unpack_hi(v, is_bf16);
            }
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) {
              s0 += __shfl_xor_sync(0xffffffffu, s0, d);
              s1 += __shfl_xor_sync(0xffffffffu, s1, d);
            }
            const int64_t col = gcol + q * 8 + w4 * 2;
            if (ro == 0 && col < p.n) {
              float* dst = p.colsum + (int64_t)(tile.row0 / BLOCK_M) * p.n + col;
              dst[0] = s0;
              if (col + 1 < p.n) dst[1] = s1;
            }
          }
        }
      }
      // accumulator drained: hand it back to the (leader's) MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2 && rank != 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
        else mbar_arrive(&acc_empty[acc]);
      }
    }
    if (leader) bulk_wait_all();   // staging buffers must outlive the stores that read them
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();   // no CTA leaves while its peer may still signal its barriers or read its shared memory
  if (warp == 1) {
    if (*abort_flag) {  // error path: give copies / MMAs in flight a bounded moment to land
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    if (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
  }
}

// Second pass of a split ESTMM: out = beta * out + sum over chunks (in chunk order) of the fp32 partial results, stored
// in the output's own type and layout.  One thread per four adjacent columns.
__global__ void __launch_bounds__(256)
estmm_reduce_kernel(const float* __restrict__ partial, int splits, int E, int64_t m, int64_t n, void* __restrict__ out, int64_t ldc,
                    int64_t c_estride, int64_t m_split, int64_t split_stride, int out_f32, int is_bf16, int beta) {
  const int64_t n4 = n / 4;
  const int64_t total = (int64_t)E * m * n4;
  const int64_t plane = (int64_t)E * m * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c4 = i % n4, row = i / n4;          // row = e * m + mrow
    const int64_t e = row / m, mrow = row - e * m;
    const float* src = partial + row * n + c4 * 4;
    float4 acc = *reinterpret_cast<const float4*>(src);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(src + (int64_t)s * plane);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const int64_t off = (mrow / m_split) * split_stride + e * c_estride + (mrow % m_split) * ldc + c4 * 4;
    if (out_f32) {
      float* o = reinterpret_cast<float*>(out) + off;
      if (beta) { const float4 old = *reinterpret_cast<float4*>(o); acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w; }
      *reinterpret_cast<float4*>(o) = acc;
    } else {
      uint16_t* o = reinterpret_cast<uint16_t*>(out) + off;
      if (beta) {
        const uint2 old = *reinterpret_cast<uint2*>(o);
        acc.x += unpack_lo(old.x, is_bf16); acc.y += unpack_hi(old.x, is_bf16);
        acc.z += unpack_lo(old.y, is_bf16); acc.w += unpack_hi(old.y, is_bf16);
      }
      *reinterpret_cast<uint2*>(o) = make_uint2(pack2(acc.x, acc.y, is_bf16), pack2(acc.z, acc.w, is_bf16));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// rank-2 or rank-3 map over 16-bit elements, 128-byte swizzle unless told otherwise, zero fill out of bounds
int make_map(CUtensorMap* tm, const void* base, int is_bf16, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
             const uint32_t* box, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  auto fn = encode_fn();
  if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return HEXA_ERR_CUDA; }
  cuuint64_t d[3]; cuuint64_t s[2]; cuuint32_t b[3]; cuuint32_t es[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
  for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
  CUresult r = fn(tm, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                  const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d dims %llu,%llu box %u,%u)", (int)r, rank,
              (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return HEXA_ERR_CUDA;
  }
  return HEXA_OK;
}

template <int BN, int MODE, int CTAS, int EW>
int launch_ew(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmX, const Params& p,
              int64_t max_tiles, cudaStream_t stream) {
  using C = Cfg<BN, CTAS, EW, MODE>;
  static bool attr_set[64] = {false};
  static int max_clusters[64] = {0};
  auto kernel = gemm_tc_kernel<BN, MODE, CTAS, EW>;
  int dev = 0;
  HEXA_CUDA(cudaGetDevice(&dev));
  HEXA_REQUIRE(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
  if (!attr_set[dev]) {
    HEXA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes));
    attr_set[dev] = true;
  }
  if (max_tiles <= 0) return HEXA_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (CTAS == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (max_clusters[dev] == 0) {   // how many CTA pairs the device can hold at once (one CTA per SM)
      cfg.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); n = sm_count() / 2; }
      max_clusters[dev] = n;
    }
    int64_t pairs = max_tiles < max_clusters[dev] ? max_tiles : max_clusters[dev];
    if (sm_limit() > 0 && pairs > sm_limit() / 2) pairs = sm_limit() / 2;
    cfg.gridDim = dim3((unsigned)(2 * (pairs > 0 ? pairs : 1)));
  } else {
    int64_t ctas = max_tiles < sm_count() ? max_tiles : sm_count();
    if (sm_limit() > 0 && ctas > sm_limit()) ctas = sm_limit();
    cfg.gridDim = dim3((unsigned)ctas);
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmA, tmB, tmC, tmX, p);
  if (e != cudaSuccess) {
    set_error("launch of gemm_tc_kernel<%d,%d,%d,%d> failed: %s", BN, MODE, CTAS, EW, cudaGetErrorString(e));
    return HEXA_ERR_CUDA;
  }
  return HEXA_OK;
}

int env_int(const char* name, int dflt) {
  const char* s = getenv(name);
  return s ? atoi(s) : dflt;
}

// Epilogue warps of a launch: HEXA_TC_EPI_WARPS (8 or 16, read at every launch so that one process can compare the two)
// or, by default, 8 for long k-loops and 16 for short ones, where the epilogue of a tile has to keep pace with few MMAs.
int epi_warps_for(int64_t num_kb_typical) {
  const int forced = env_int("HEXA_TC_EPI_WARPS", 0);
  if (forced == 4 || forced == 8 || forced == 16) return forced;
  const int64_t threshold = env_int("HEXA_TC_EPI_WARPS_KB", 0);     // 0: always 16 (the faster setting at K = 768 and, for the
                                                                     // launches with an activation, at K = 2048 as well)
  return (threshold > 0 && num_kb_typical >= threshold) ? 8 : 16;
}

template <int BN, int MODE, int CTAS>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmX, const Params& p,
           int64_t max_tiles, cudaStream_t stream, int epi_warps) {
  if (epi_warps == 4) return launch_ew<BN, MODE, CTAS, 4>(tmA, tmB, tmC, tmX, p, max_tiles, stream);
  if (epi_warps == 8) return launch_ew<BN, MODE, CTAS, 8>(tmA, tmB, tmC, tmX, p, max_tiles, stream);
  return launch_ew<BN, MODE, CTAS, 16>(tmA, tmB, tmC, tmX, p, max_tiles, stream);
}
// HEXA_TC_CTAS=1 keeps every GEMM on single-CTA tiles (for A/B measurements); default: CTA pairs where they apply.
bool pairs_enabled() { static int v = -1; if (v < 0) v = env_int("HEXA_TC_CTAS", 2) == 1 ? 0 : 1; return v == 1; }

}  // namespace

bool esmm_tc_supported(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t b_estride, const void* aux,
                       int64_t ldaux, const void* c, int64_t ldc, const float* bias, int64_t ldbias, int64_t n_out,
                       int dtype) {
  if (dtype != HEXA_F16 && dtype != HEXA_BF16) return false;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || (aux && !aligned16(aux)) || (bias && !aligned16(bias))) return false;
  if (lda % 8 || ldb % 8 || b_estride % 8 || ldc % 8 || (aux && ldaux % 8) || (bias && ldbias % 4)) return false;
  // n_out itself may be any size (a rank's slice of an unevenly split hidden dimension): the TMA stores clip at
  // n_out, but the epilogue's 16-byte reads of bias and saved pre-activation run to the end of the last chunk, so
  // those rows must be padded to whole chunks
  const int64_t n8 = (n_out + 7) / 8 * 8, n4 = (n_out + 3) / 4 * 4;
  if ((aux && ldaux < n8) || (bias && ldbias < n4)) return false;
  return true;
}

int esmm_tc_launch(const void* a, int64_t lda, const void* b, int b_layout, int64_t ldb, int64_t b_estride,
                   const float* bias, int64_t ldbias, void* aux, int64_t ldaux, void* c, int64_t ldc,
                   const int32_t* tile_expert, const int32_t* pad_offsets, const int32_t* row_token,
                   const int32_t* pair_block, int E, int64_t row_cap, int64_t n_out, int64_t k, int dtype, int epilogue,
                   int act, cudaStream_t stream, int e_begin, int e_end, float* colsum) {
  if (row_cap == 0 || e_begin >= e_end) return HEXA_OK;
  const int is_bf16 = dtype == HEXA_BF16;
  const int BN = n_out > 128 ? 256 : 128;
  const int ctas = (BN == 256 && pair_block != nullptr && pairs_enabled()) ? 2 : 1;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {(uint64_t)k, (uint64_t)row_cap};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {BLOCK_K, BLOCK_M};
    int rc = make_map(&tmA, a, is_bf16, 2, dims, str, box);
    if (rc) return rc;
  }
  if (b_layout == HEXA_B_NK) {
    uint64_t dims[3] = {(uint64_t)k, (uint64_t)n_out, (uint64_t)E};
    uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)b_estride * 2};
    uint32_t box[3] = {BLOCK_K, (uint32_t)(BN / ctas), 1};   // each CTA of a pair loads half of the B rows
    int rc = make_map(&tmB, b, is_bf16, 3, dims, str, box);
    if (rc) return rc;
  } else {
    uint64_t dims[3] = {(uint64_t)n_out, (uint64_t)k, (uint64_t)E};
    uint64_t str[2] = {(uint64_t)ldb * 2, (uint64_t)b_estride * 2};
    uint32_t box[3] = {64, BLOCK_K, 1};
    int rc = make_map(&tmB, b, is_bf16, 3, dims, str, box);
    if (rc) return rc;
  }
  // output maps for the epilogue's TMA stores: [128 rows x 32 columns] boxes, 64-byte swizzle
  CUtensorMap tmC, tmX;
  {
    uint64_t dims[2] = {(uint64_t)n_out, (uint64_t)row_cap};
    uint32_t box[2] = {32, BLOCK_M};
    uint64_t str[1] = {(uint64_t)ldc * 2};
    int rc = make_map(&tmC, c, is_bf16, 2, dims, str, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;
    tmX = tmC;
    if (aux && epilogue == HEXA_EPI_ACT) {
      uint64_t strx[1] = {(uint64_t)ldaux * 2};
      rc = make_map(&tmX, aux, is_bf16, 2, dims, strx, box, CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
    }
  }
  Params p{};
  p.tile_expert = tile_expert; p.pad_offsets = pad_offsets; p.row_token = row_token;
  p.pair_block = pair_block; p.max_pairs = row_cap / (2 * BLOCK_M) + E;
  p.bias = bias; p.ldbias = ldbias; p.aux = aux; p.ldaux = ldaux; p.c = c; p.ldc = ldc;
  p.n = n_out; p.k = k; p.m = 0; p.E = E; p.e_begin = e_begin; p.e_end = e_end;
  p.epilogue = epilogue; p.act = act; p.is_bf16 = is_bf16; p.colsum = colsum;
  p.status = status_word(); p.debug = tc_debug_flags(); p.wait_limit_ns = wait_limit_ns();
  const int64_t NT = ceil_div(n_out, BN);
  HEXA_REQUIRE((row_cap / BLOCK_M + E + 1) * NT < (int64_t)0x7fffffff, "hexa_esmm: too many output tiles for a 32-bit tile index");
  p.nt = (uint32_t)NT;
  const int ew = epi_warps_for(ceil_div(k, BLOCK_K));
  if (ctas == 2) {
    const int64_t max_tiles = p.max_pairs * NT;
    return b_layout == HEXA_B_NK ? launch<256, ESMM_NK, 2>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew)
                                 : launch<256, ESMM_KN, 2>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew);
  }
  const int64_t max_tiles = (row_cap / BLOCK_M) * NT;
  if (b_layout == HEXA_B_NK)
    return BN == 256 ? launch<256, ESMM_NK, 1>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew)
                     : launch<128, ESMM_NK, 1>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew);
  return BN == 256 ? launch<256, ESMM_KN, 1>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew)
                   : launch<128, ESMM_KN, 1>(tmA, tmB, tmC, tmX, p, max_tiles, stream, ew);
}

bool estmm_tc_supported(const void* p, int64_t ldp, const void* q, int64_t ldq, const void* out, int64_t ldo,
                        int64_t o_estride, int64_t split_stride, int64_t n, int dtype, int out_dtype) {
  if (dtype != HEXA_F16 && dtype != HEXA_BF16) return false;
  if (out_dtype != HEXA_F32 && out_dtype != dtype) return false;
  if (!aligned16(p) || !aligned16(q) || !aligned16(out)) return false;
  const int ov = out_dtype == HEXA_F32 ? 4 : 8;
  if (ldp % 8 || ldq % 8 || ldo % ov || o_estride % ov || split_stride % ov || n % 8) return false;
  return true;
}

// How many chunks a split ESTMM cuts every expert's segment into (1 = no split).  Only static sizes enter: the tile
// count without a split against the CTA pairs (or CTAs) of the device, and the average segment length, so that a chunk
// keeps at least 8 k-blocks.  Few, long segments - the dense FFN's weight gradient (one "expert" owning every row), or a
// handful of experts with a small d x H - would otherwise leave most SMs idle behind a few serial k-loops.
int estmm_tc_splits(int E, int64_t row_cap, int64_t m, int64_t n) {
  static int forced = -2;
  if (forced == -2) forced = env_int("HEXA_ESTMM_SPLITS", -1);       // A/B switch: 1 = never split
  if (n % 4) return 1;
  const int BN = n > 128 ? 256 : 128;
  const int ctas = (BN == 256 && m > BLOCK_M && pairs_enabled()) ? 2 : 1;
  const int64_t tiles = (int64_t)E * ceil_div(m, BLOCK_M * ctas) * ceil_div(n, BN);
  const int64_t slots = ctas == 2 ? sm_count() / 2 : sm_count();
  const int64_t avg_kb = row_cap / BLOCK_K / E;
  int64_t s = 1;
  if (tiles < 2 * slots) s = ceil_div(2 * slots, tiles);
  if (s > avg_kb / 8) s = avg_kb / 8;
  if (forced > 0) s = forced;
  if (s > 32) s = 32;
  return s < 1 ? 1 : (int)s;
}

size_t estmm_tc_workspace_bytes(int E, int64_t row_cap, int64_t m, int64_t n) {
  const int s = estmm_tc_splits(E, row_cap, m, n);
  return s > 1 ? (size_t)s * (size_t)E * (size_t)m * (size_t)n * sizeof(float) : 0;
}

int estmm_tc_launch(const void* pp, int64_t ldp, const void* q, int64_t ldq, const int32_t* pad_offsets, int E,
                    int64_t row_cap, int64_t m, int64_t n, void* out, int64_t ldo, int64_t o_estride, int64_t m_split,
                    int64_t split_stride, int dtype, int out_dtype, int beta, cudaStream_t stream, void* const* split_out,
                    int n_split, void* workspace, size_t workspace_bytes) {
  const int is_bf16 = dtype == HEXA_BF16;
  const int BN = n > 128 ? 256 : 128;
  const int ctas = (BN == 256 && m > BLOCK_M && pairs_enabled()) ? 2 : 1;
  int splits = n_split > 0 ? 1 : estmm_tc_splits(E, row_cap, m, n);
  if (splits > 1 && (!workspace || workspace_bytes < (size_t)splits * E * m * n * sizeof(float) || !aligned16(workspace)))
    splits = 1;      // without scratch the operator still runs, one tile per expert's whole segment
  CUtensorMap tmA, tmB;
  // the maps need at least one row even when no token was routed
  const uint64_t rows = row_cap > 0 ? (uint64_t)row_cap : 1;
  {
    uint64_t dims[2] = {(uint64_t)m, rows};
    uint64_t str[1] = {(uint64_t)ldp * 2};
    uint32_t box[2] = {64, BLOCK_K};
    int rc = make_map(&tmA, pp, is_bf16, 2, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)n, rows};
    uint64_t str[1] = {(uint64_t)ldq * 2};
    uint32_t box[2] = {64, BLOCK_K};
    int rc = make_map(&tmB, q, is_bf16, 2, dims, str, box);
    if (rc) return rc;
  }
  Params p{};
  p.pad_offsets = pad_offsets; p.c = out; p.ldc = ldo; p.c_estride = o_estride; p.n = n; p.m = m; p.E = E;
  p.m_split = m_split; p.split_stride = split_stride;
  p.n_split = n_split;
  for (int i = 0; i < n_split && i < 16; ++i) p.c_split[i] = split_out[i];
  p.is_bf16 = is_bf16; p.out_f32 = out_dtype == HEXA_F32; p.beta = beta;
  p.splits = splits; p.partial = static_cast<float*>(workspace);
  p.status = status_word(); p.debug = tc_debug_flags(); p.wait_limit_ns = wait_limit_ns();
  const int64_t max_tiles = (int64_t)E * ceil_div(m, BLOCK_M * ctas) * ceil_div(n, BN) * splits;
  HEXA_REQUIRE(max_tiles < (int64_t)0x7fffffff, "hexa_estmm: too many output tiles for a 32-bit tile index");
  p.nt = (uint32_t)ceil_div(n, BN);
  p.per_expert = (uint32_t)(ceil_div(m, BLOCK_M * ctas) * ceil_div(n, BN) * splits);
  p.total_tiles = (uint32_t)max_tiles;
  // ESTMM stores straight from registers; the two output maps are unused placeholders
  int rc;
  const int ew = epi_warps_for(row_cap / BLOCK_K / (E * (int64_t)splits));
  if (ctas == 2) rc = launch<256, ESTMM, 2>(tmA, tmB, tmA, tmA, p, max_tiles, stream, ew);
  else rc = BN == 256 ? launch<256, ESTMM, 1>(tmA, tmB, tmA, tmA, p, max_tiles, stream, ew)
                      : launch<128, ESTMM, 1>(tmA, tmB, tmA, tmA, p, max_tiles, stream, ew);
  if (rc != HEXA_OK || splits == 1) return rc;
  const int64_t total = (int64_t)E * m * (n / 4);
  int64_t blocks = ceil_div(total, 256);
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  estmm_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.partial, splits, E, m, n, out, ldo, o_estride, p.m_split, p.split_stride,
                                                          p.out_f32, is_bf16, beta);
  HEXA_LAUNCH_CHECK("estmm_reduce_kernel");
  return HEXA_OK;
}

}  // namespace hexa
