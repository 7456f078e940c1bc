// TMA-fed tcgen05 / TMEM GEMM skeleton for sm_100a.
//
// A GEMM-shaped Kernel (Mul of two loads under an f32 Add reduction, the form the reference's
// `jitRules[Dot]` builds, src/frontend/jit.ts:639-648) runs here when its operands can be
// described by TMA tensor maps.  The reference tiles the same kernel for WebGPU with 4x4
// register tiles and no shared memory (src/tuner.ts:284-383) and for Wasm with a 128x128x64
// plan (src/backend/wasm/tilePlan.ts:38-45); on Blackwell the tile lives in tensor memory:
//
//   warp 0      TMA producer: 128-byte-swizzled tiles of A and B into a ring of shared-memory
//               stages (cp.async.bulk.tensor, one CTA, no multicast), mbarrier expect_tx
//   warp 1      MMA issuer: tcgen05.mma (cta_group::1, M=128, N=BN) from shared-memory
//               descriptors into one of two TMEM accumulators; tcgen05.commit frees the stage
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator, apply the Kernel's spliced
//               epilogue (Cast, bias, ReLU ...) and store, while warp 1 fills the other one
//   then        3xTF32 with LO_IN_KERNEL: four warps that derive the remainder tiles from the loaded
//               operands inside the stage (after the gather warps, when there are any)
//   warps 6+    convolutions only (B_GATHER): evaluate the Kernel's patch expression for the stage's
//               [BK x BN] slice of the B operand and write it (and its 3xTF32 remainder) straight
//               into the stage in the swizzled layout a TMA box would have, so that the patch
//               operand never exists in global memory (implicit GEMM); TMA then loads A only
//
// The kernel is persistent (one CTA per SM, static tile schedule).  float16 operands use
// kind::f16 with f32 accumulation.  float32 operands use kind::tf32 three times per k-step on
// the operand (whose low 13 mantissa bits the tensor core ignores) and a remainder plane
// lo = x - tf32(x) (3xTF32: lo*hi + hi*lo + hi*hi),
// which keeps f32 accuracy; plain TF32 is never used.  Every mbarrier wait is bounded: on a
// time-out the kernel records a code in `status` and winds down instead of hanging the GPU.
#include "gemm_tc.hpp"

#include <cstdlib>
#include <cstring>
#include <sstream>

#include "prelude.hpp"

namespace jaxcuda {

namespace {

const char* const kTcSource = R"TCGEMM(
struct __align__(64) CUtensorMap { unsigned long long opaque[16]; };

// SPIN_LIMIT (polls of a pipeline wait before it gives up, about a second at the default) and
// FAULT_SKIP_LOAD (tests of the wind-down only) are defined by the planner.

__device__ __forceinline__ u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(u32 bar, u32 count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(u32 bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u32 bar, u32 bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: polls without blocking (test_wait), backs off with nanosleep, and gives up after
// SPIN_LIMIT polls (about a second) or as soon as another role has reported a failure.
__device__ __forceinline__ bool mbar_wait(u32 bar, u32 parity, volatile int* status) {
  for (int spin = 0; spin < SPIN_LIMIT; spin++) {
    u32 done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if (spin > 64) __nanosleep(40);
    if ((spin & 1023) == 1023 && *status != 0) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_3d(u32 dst, const CUtensorMap* map, u32 bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// CTA_PAIR: two CTAs of a cluster work on one 256 x BN tile (tcgen05 cta_group::2).  Each CTA loads
// its own 128 rows of A and its own half of the columns of B; the MMAs, issued by the even CTA alone,
// read B from both.  Per output a CTA so fetches a third less (f16, BN = 256) through L2 and shared
// memory, which is what bounds the single-CTA kernel.  The loads carry no multicast: each CTA's own
// TMA (cta_group::2 form) reports to the even CTA's mbarrier, whose address is the own one with the
// rank bit cleared.
__device__ __forceinline__ void tma_load_3d_pair(u32 dst, const CUtensorMap* map, u32 bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(u32 bar) {   // arrives on the barrier at this offset in both CTAs
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_at(u32 bar, u32 cta_rank) {   // arrive on CTA cta_rank's barrier at this offset
  asm volatile("{\n\t.reg .b32 r;\n\tmapa.shared::cluster.u32 r, %0, %1;\n\t"
               "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [r];\n\t}" ::"r"(bar), "r"(cta_rank) : "memory");
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma(u32 d_tmem, u64 adesc, u64 bdesc, u32 idesc, u32 accumulate) {
#if CTA_PAIR && KIND == 1
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#elif CTA_PAIR
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#elif KIND == 1
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#else
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
#endif
}
__device__ __forceinline__ void umma_commit(u32 bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(u32 taddr, u32* v) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr));
}

__device__ __forceinline__ uint4 ld_shared_16(u32 addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_16(u32 addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Where byte `o` (row * 128 + byte in row) of a [rows][128 bytes] TMA box lands inside the box:
// the 128-byte swizzle in 16-byte units (16-bit elements) or in 32-byte units (32-bit elements).
__device__ __forceinline__ u32 box_swizzle(u32 o) {
  return ELEM == 4 ? (o ^ (((o >> 7) & 3u) << 5)) : (o ^ (((o >> 7) & 7u) << 4));
}

// Shared-memory matrix descriptor (sm_100): start address, leading / stride byte offsets in
// 16-byte units, descriptor version 1, 128-byte swizzle.
// layout: 2 = 128-byte swizzle in 16-byte units; 1 = 128-byte swizzle in 32-byte units, the only
// layout tensor cores accept for MN-major 32-bit (TF32) operands.
__device__ __forceinline__ u64 make_desc(u32 addr, u32 lbo_bytes, u32 sbo_bytes, u32 layout) {
  return (u64)((addr >> 4) & 0x3fff) | ((u64)((lbo_bytes >> 4) & 0x3fff) << 16) |
         ((u64)((sbo_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) | ((u64)layout << 61);
}

// Per k-step (32 bytes of K) descriptor of an operand tile that starts at `base`.
//   K-major : rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart; advance 32 bytes per step
//   MN-major: boxes of [BK rows of k][128 bytes of m/n], BOX_BYTES apart; a step covers KROWS k-rows
#define KROWS (32 / ELEM)             /* k elements per MMA: 16 (f16) or 8 (tf32) */
#define BK (128 / ELEM)               /* k elements per stage */
#define BOX_BYTES (BK * 128)
//             (4-byte elements: swizzle atoms are 4 k-rows = 512 bytes, in 32-byte units)
__device__ __forceinline__ u64 operand_desc(u32 base, int kk, int mn_major) {
  if (!mn_major) return make_desc(base + kk * 32, 16, 1024, 2);
  return ELEM == 4 ? make_desc(base + kk * KROWS * 128, BOX_BYTES, 512, 1)
                   : make_desc(base + kk * KROWS * 128, BOX_BYTES, 1024, 2);
}

#define TILE_M (CTA_PAIR ? 2 * BM : BM)     /* rows of a tile: a CTA pair covers 256 */
#define B_COLS (CTA_PAIR ? BN / 2 : BN)     /* columns of B a CTA holds per stage */
#define WORKER ((int)blockIdx.x / (CTA_PAIR ? 2 : 1))   /* index of this CTA (pair) in the tile schedule */
#define WORKERS ((int)gridDim.x / (CTA_PAIR ? 2 : 1))
#define A_BYTES (BM * 128)
#define B_BYTES (B_COLS * 128)
#define NPLANES (KIND == 2 ? 2 : 1)
#define STAGE_BYTES (NPLANES * (A_BYTES + B_BYTES))
#define TILES_M ((GM + TILE_M - 1) / TILE_M)
#define TILES_N ((GN + BN - 1) / BN)
#define NUM_TILES (TILES_M * TILES_N * GBATCH)
#define K_BLOCKS ((GK + BK - 1) / BK)
#define TMEM_COLS (2 * ACC_STRIDE)     /* a power of two; the two accumulators start ACC_STRIDE columns apart */
#define NCHUNK ((K_BLOCKS + CHUNK_KB - 1) / CHUNK_KB)
#define IDESC ((1u << 4) | ((KIND == 2 ? 2u : 0u) << 7) | ((KIND == 2 ? 2u : 0u) << 10) | ((u32)A_MN << 15) | \
               ((u32)B_MN << 16) | ((u32)(BN >> 3) << 17) | ((u32)(TILE_M >> 4) << 24))
#define IDESC_N(bn) (HALF_LAST ? ((IDESC & ~(0x3fu << 17)) | ((u32)((bn) >> 3) << 17)) : IDESC)

__device__ __forceinline__ void tile_coords(int t, int& b, int& m_blk, int& n_blk) {
  const int per_batch = TILES_M * TILES_N;
  b = t / per_batch;
  const int rem = t - b * per_batch;
  const int GROUP = 8;                       // M-tiles sharing a sweep over N: keeps B tiles hot in L2
  const int span = GROUP * TILES_N;
  const int first_m = (rem / span) * GROUP;
  const int gsz = (TILES_M - first_m) < GROUP ? (TILES_M - first_m) : GROUP;
  const int in = rem % span;
  m_blk = first_m + in % gsz;
  n_blk = in / gsz;
}

// Work of one CTA, in order: whole tiles t = blockIdx.x, + gridDim.x, ... while full waves last.  The
// R < gridDim.x tiles that are left over would occupy R CTAs for a whole tile's time; with SPLITK
// each of them is cut along K into S = gridDim.x / R slices (at most 8) that run side by side, so the
// last wave takes 1 / S of a tile's time (and an output with fewer tiles than SMs uses S times as
// many of them).  CTA c takes slice c / R of left-over tile c % R: CTAs that run at the same time
// work at the same depth of K in different tiles and so still share operand panels through L2.
// (Sharing the left-over k-blocks out evenly instead, each CTA continuing where its neighbour
// stops, was measured 20 to 40 % slower than no split at all: neighbours then read different
// k-ranges of the same panels and every operand byte comes from DRAM.)  A slice's accumulators go to
// scratch; the CTA that delivers a tile's last slice adds them up in k order and runs the epilogue.
struct Seg { int tile, kb0, kb1, partial, slot, n_off, bn; };   // n_off, bn: the columns of the tile this segment covers
__device__ __forceinline__ int sk_tiles_full() {
  const int full = (NUM_TILES / WORKERS) * WORKERS;
  if (HALF_LAST) return 2 * (NUM_TILES - full) <= WORKERS ? full : NUM_TILES;   // (the grid may be smaller than planned)
  return STREAMK ? full : NUM_TILES;
}
__device__ __forceinline__ int sk_slices() {
  const int rest = NUM_TILES - sk_tiles_full();
  int s = rest > 0 ? WORKERS / rest : 1;
  s = s > 8 ? 8 : s;
  return s > K_BLOCKS ? K_BLOCKS : s;
}
__device__ __forceinline__ bool get_segment(int i, Seg& s) {
  const int P = WORKERS, c = WORKER;
  const int tiles_full = sk_tiles_full();
  const int n_static = tiles_full > c ? (tiles_full - c + P - 1) / P : 0;
  s.n_off = 0; s.bn = BN;
  if (i < n_static) { s.tile = c + i * P; s.kb0 = 0; s.kb1 = K_BLOCKS; s.partial = 0; s.slot = 0; return true; }
#if HALF_LAST
  // CTA pairs: the tiles left over behind the whole waves, at most half as many as pairs, are cut
  // in two along N and run as 256 x BN/2 tiles on twice as many pairs, every pair still walking the
  // whole K in step with the others and nothing to add up afterwards.  A half tile takes about 0.7
  // of a whole tile's time (its CTA stores a quarter of B per stage instead of a half).
  {
    const int rest_h = NUM_TILES - tiles_full;
    if (rest_h == 0 || i > n_static || c >= 2 * rest_h) return false;
    s.tile = tiles_full + c / 2; s.kb0 = 0; s.kb1 = K_BLOCKS; s.partial = 0; s.slot = 0;
    s.bn = BN / 2; s.n_off = (c & 1) * (BN / 2);
    return true;
  }
#endif
  const int rest = NUM_TILES - tiles_full;
  if (!STREAMK || rest == 0 || i > n_static) return false;
  const int S = sk_slices();
  if (c >= rest * S) return false;
  const int slice = c / rest;
  s.tile = tiles_full + c % rest;
  s.kb0 = (int)((i64)K_BLOCKS * slice / S);
  s.kb1 = (int)((i64)K_BLOCKS * (slice + 1) / S);
  s.partial = S > 1;
  s.slot = c;
  return true;
}

#if B_GATHER
// Emitted behind this source from the Kernel's patch expression: fills rows k0 .. k0 + BK of the B
// tile whose first column is n_tile (batch entry b) at shared address sb; gt is the calling thread's
// index among the GROUP_WARPS * 32 threads that fill this stage.
__device__ __forceinline__ void jx_gather_tile(JX_PARAMS, u32 sb, int b, int n_tile, int k0, int gt);
#endif
// LO_IN_KERNEL (3xTF32): TMA brings only the operands themselves and signals raw(s); XFORM_WARPS
// warps then write the remainder tiles lo = x - tf32(x) beside them, chunk for chunk at the same
// offsets (so the swizzle needs no thought), and arrive on full(s).  No split pass over global
// memory, half the TMA traffic.
#define TMA_PLANES (LO_IN_KERNEL ? 1 : NPLANES)
#define TX_BYTES (B_GATHER ? TMA_PLANES * A_BYTES : TMA_PLANES * (A_BYTES + B_BYTES))
// EPI_SPLIT groups of four epilogue warps share a tile's columns (2 for the 256-column 3xTF32 pairs,
// whose partial sums would not fit one thread's registers); they sit behind warps 0 and 1, and the
// gather and remainder-tile warps, which never coexist with a second group, behind the first group.
#define EPI_COLS (BN / EPI_SPLIT)
#define NTHREADS (64 + 128 * EPI_SPLIT + 32 * (GATHER_WARPS + XFORM_WARPS))
#define GROUP_WARPS (GATHER_WARPS / GATHER_GROUPS)
#if HALF_LAST && (!CTA_PAIR || BN < 256)
#error "half tiles in the last wave: CTA pairs on 256-column tiles"
#endif
#if EPI_SPLIT > 1 && (STREAMK || B_GATHER || LO_IN_KERNEL)
#error "a second group of epilogue warps takes the place of the gather and remainder-tile warps"
#endif
#if CTA_PAIR && (STREAMK || B_GATHER || LO_IN_KERNEL)
#error "CTA pairs run whole tiles with TMA-loaded operands only"
#endif
#if B_GATHER && (GATHER_GROUPS > STAGES || GATHER_WARPS % GATHER_GROUPS)
#error "gather groups must divide the gather warps and not outnumber the stages"
#endif

extern "C" __global__ void __launch_bounds__(NTHREADS, 1)
jx_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA2,
        const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2,
        JX_PARAMS, int* status_ptr) {
  extern __shared__ unsigned char smem_raw[];
  volatile int* status = status_ptr;
  // the slices' accumulators and their arrival counters live at SK_OFFSET of the scratch (counters first)
  int* sk_counters = reinterpret_cast<int*>(reinterpret_cast<char*>(scratch) + SK_OFFSET);
  float* sk_pieces = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + SK_OFFSET + SK_COUNTER_BYTES);
  (void)sk_counters; (void)sk_pieces;
  const u32 smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;     // swizzle atoms are 1024-byte aligned
  const u32 bars = smem_base + STAGES * STAGE_BYTES;                // full[STAGES], empty[STAGES], tfull[2], tempty[2]
  const u32 tmem_slot = bars + (2 * STAGES + 4 + (LO_IN_KERNEL ? STAGES : 0)) * 8;
  auto full = [&](int s) { return bars + s * 8; };
  auto empty = [&](int s) { return bars + (STAGES + s) * 8; };
  auto tfull = [&](int a) { return bars + (2 * STAGES + a) * 8; };
  auto tempty = [&](int a) { return bars + (2 * STAGES + 2 + a) * 8; };
  auto raw = [&](int s) { return bars + (2 * STAGES + 4 + s) * 8; };   // LO_IN_KERNEL only
  auto tma_bar = [&](int s) { return LO_IN_KERNEL ? raw(s) : full(s); };
  (void)raw;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  u32 rank = 0;                              // CTA_PAIR: 0 for the even CTA of the pair, which issues the MMAs
  if (CTA_PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full(s), (LO_IN_KERNEL ? XFORM_WARPS : 1) + (B_GATHER ? GROUP_WARPS : 0));
      mbar_init(empty(s), 1);
      if (LO_IN_KERNEL) mbar_init(raw(s), 1);
    }
    for (int a = 0; a < 2; a++) { mbar_init(tfull(a), 1); mbar_init(tempty(a), 4 * EPI_SPLIT * (CTA_PAIR ? 2 : 1)); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
#if CTA_PAIR
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((u32)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
#else
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"((u32)TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
#endif
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CTA_PAIR) cluster_sync();              // the peer's barriers exist before anything is signalled across
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  u32 tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  bool failed = false;
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int it = 0;
      Seg sg;
      for (int si = 0; !failed && get_segment(si, sg); si++) {
        int b, m_blk, n_blk;
        tile_coords(sg.tile, b, m_blk, n_blk);
        for (int kb = sg.kb0; kb < sg.kb1; kb++, it++) {
          const int s = it % STAGES;
          if (it >= STAGES && !mbar_wait(empty(s), ((it / STAGES) + 1) & 1, status)) { atomicCAS((int*)status_ptr, 0, 1); failed = true; break; }
          if (!CTA_PAIR) mbar_expect_tx(tma_bar(s), TX_BYTES);
          else if (rank == 0)   // both CTAs' loads report to the even CTA's barrier
            mbar_expect_tx(full(s), 2 * (TX_BYTES - ((HALF_LAST && B_MN) ? (BN - sg.bn) / 2 * 128 * TMA_PLANES : 0)));   // (a K-major box of B is always B_COLS rows: a half tile uses the first half of it)
#if FAULT_SKIP_LOAD
          // test of the wind-down: CTA 0 announces its second stage and never loads it, so the MMA
          // role's bounded wait on that stage runs out
          if (blockIdx.x == 0 && it == 1) continue;
#endif
          const u32 sa = smem_base + s * STAGE_BYTES, sb = sa + NPLANES * A_BYTES;
          const int k0 = kb * BK;
          const int ba = A_SHARED ? 0 : b, bb = B_SHARED ? 0 : b;   // an operand all batches share has one plane
          const int b_cols = HALF_LAST ? sg.bn / 2 : B_COLS;   // columns of B this CTA loads (a pair's half tile: a quarter of BN)
          const int m0 = m_blk * TILE_M + (int)rank * BM, n0 = n_blk * BN + sg.n_off + (int)rank * b_cols;   // this CTA's rows of A and columns of B
#if CTA_PAIR
#define TMA_LOAD tma_load_3d_pair
#else
#define TMA_LOAD tma_load_3d
#endif
#if A_MN
          for (int j = 0; j < BM / BK; j++) {
            TMA_LOAD(sa + j * BOX_BYTES, &tmA, tma_bar(s), m0 + j * BK, k0, ba);
            if (KIND == 2 && !LO_IN_KERNEL) TMA_LOAD(sa + A_BYTES + j * BOX_BYTES, &tmA2, tma_bar(s), m0 + j * BK, k0, ba);
          }
#else
          TMA_LOAD(sa, &tmA, tma_bar(s), k0, m0, ba);
          if (KIND == 2 && !LO_IN_KERNEL) TMA_LOAD(sa + A_BYTES, &tmA2, tma_bar(s), k0, m0, ba);
#endif
#if B_GATHER
          (void)sb; (void)bb; (void)n0;
#elif B_MN
          for (int j = 0; j < b_cols / BK; j++) {
            TMA_LOAD(sb + j * BOX_BYTES, &tmB, tma_bar(s), n0 + j * BK, k0, bb);
            if (KIND == 2 && !LO_IN_KERNEL) TMA_LOAD(sb + B_BYTES + j * BOX_BYTES, &tmB2, tma_bar(s), n0 + j * BK, k0, bb);
          }
#else
          TMA_LOAD(sb, &tmB, tma_bar(s), k0, n0, bb);
          if (KIND == 2 && !LO_IN_KERNEL) TMA_LOAD(sb + B_BYTES, &tmB2, tma_bar(s), k0, n0, bb);
#endif
#undef TMA_LOAD
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // A tile's K loop is cut into NCHUNK chunks of CHUNK_KB k-blocks; every chunk starts a fresh
    // accumulator (alternating between the two TMEM buffers) that the epilogue warps fold into
    // registers.  Tensor cores add into the accumulator with truncation, a bias that grows with the
    // length of the chain; short chains joined by round-to-nearest f32 adds keep f32 accuracy.
    if (lane == 0 && rank == 0) {            // of a CTA pair only the even CTA issues MMAs
      int it = 0, cc = 0;
      Seg sg;
      for (int si = 0; !failed && get_segment(si, sg); si++) {
        const int nch = (sg.kb1 - sg.kb0 + CHUNK_KB - 1) / CHUNK_KB;
        for (int ch = 0; ch < nch && !failed; ch++, cc++) {
          const int acc = cc & 1;
          if (cc >= 2 && !mbar_wait(tempty(acc), ((cc >> 1) + 1) & 1, status)) { atomicCAS((int*)status_ptr, 0, 2); failed = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const u32 d = tmem_base + acc * ACC_STRIDE;
          const int kb_first = sg.kb0 + ch * CHUNK_KB;
          const int kb_end = kb_first + CHUNK_KB < sg.kb1 ? kb_first + CHUNK_KB : sg.kb1;
          for (int kb = kb_first; kb < kb_end; kb++, it++) {
            const int s = it % STAGES;
            if (LO_IN_KERNEL && !mbar_wait(raw(s), (it / STAGES) & 1, status)) { atomicCAS((int*)status_ptr, 0, 3); failed = true; break; }
            if (!mbar_wait(full(s), (it / STAGES) & 1, status)) { atomicCAS((int*)status_ptr, 0, 3); failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const u32 sa = smem_base + s * STAGE_BYTES, sb = sa + NPLANES * A_BYTES;
            #pragma unroll
            for (int kk = 0; kk < 4; kk++) {
              const u32 first = (kb != kb_first || kk) ? 1u : 0u;
#if KIND == 1
              umma(d, operand_desc(sa, kk, A_MN), operand_desc(sb, kk, B_MN), IDESC_N(sg.bn), first);
#else
              // 3xTF32: small cross terms first, then the main product
              umma(d, operand_desc(sa + A_BYTES, kk, A_MN), operand_desc(sb, kk, B_MN), IDESC_N(sg.bn), first);
              umma(d, operand_desc(sa, kk, A_MN), operand_desc(sb + B_BYTES, kk, B_MN), IDESC_N(sg.bn), 1u);
              umma(d, operand_desc(sa, kk, A_MN), operand_desc(sb, kk, B_MN), IDESC_N(sg.bn), 1u);
#endif
            }
            // the stage is free once these MMAs have read it (in both CTAs of a pair)
            if (CTA_PAIR) umma_commit_pair(empty(s)); else umma_commit(empty(s));
          }
          if (!failed) { if (CTA_PAIR) umma_commit_pair(tfull(acc)); else umma_commit(tfull(acc)); }  // this chunk's accumulator is complete
        }
      }
    }
#if B_GATHER
  } else if (warp >= 6 && warp < 6 + GATHER_WARPS) {
    // ---------------------------------------------------------------- patch gatherers (convolutions)
    // GATHER_GROUPS groups of GROUP_WARPS warps take the stages in turn, so that as many stages are
    // being filled at a time: one group's pass over a stage is a chain of address arithmetic, loads
    // that mostly come from L2 and stores, longer than the MMAs of a stage take.  GATHER_GROUPS <=
    // STAGES (the planner sees to it): the parity wait below cannot tell a stage that is two uses
    // behind from one that is free.
    const int grp = (threadIdx.x - 192) / (GROUP_WARPS * 32), gt = (threadIdx.x - 192) % (GROUP_WARPS * 32);
    int it = 0;
    Seg sg;
    for (int si = 0; !failed && get_segment(si, sg); si++) {
      int b, m_blk, n_blk;
      tile_coords(sg.tile, b, m_blk, n_blk);
      for (int kb = sg.kb0; kb < sg.kb1; kb++, it++) {
        if (it % GATHER_GROUPS != grp) continue;
        const int s = it % STAGES;
        if (it >= STAGES && !mbar_wait(empty(s), ((it / STAGES) + 1) & 1, status)) { atomicCAS((int*)status_ptr, 0, 5); failed = true; break; }
        jx_gather_tile(JX_PARAM_NAMES, smem_base + s * STAGE_BYTES + NPLANES * A_BYTES, b, n_blk * BN, kb * BK, gt);
        // the tensor core reads shared memory through the async proxy: order these writes before it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full(s));
      }
    }
#endif
#if LO_IN_KERNEL
  } else if (warp >= 6 + GATHER_WARPS) {
    // ---------------------------------------------------------------- remainder tiles (3xTF32)
    const int xt = threadIdx.x - 192 - 32 * GATHER_WARPS;
    auto lo_of = [](uint4 v) {
      uint4 r;
      r.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(v.x & 0xffffe000u));
      r.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(v.y & 0xffffe000u));
      r.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(v.z & 0xffffe000u));
      r.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(v.w & 0xffffe000u));
      return r;
    };
    int it = 0;
    Seg sg;
    for (int si = 0; !failed && get_segment(si, sg); si++) {
      for (int kb = sg.kb0; kb < sg.kb1; kb++, it++) {
        const int s = it % STAGES;
        // the TMA of this use of the stage was issued after the MMAs of the previous use had
        // finished, so once it has landed the remainder tiles are free to overwrite as well
        if (!mbar_wait(raw(s), (it / STAGES) & 1, status)) { atomicCAS((int*)status_ptr, 0, 6); failed = true; break; }
        const u32 sa = smem_base + s * STAGE_BYTES;
        #pragma unroll 4
        for (int c = xt; c < A_BYTES / 16; c += XFORM_WARPS * 32) st_shared_16(sa + A_BYTES + c * 16, lo_of(ld_shared_16(sa + c * 16)));
#if !B_GATHER
        const u32 sb = sa + 2 * A_BYTES;
        #pragma unroll 4
        for (int c = xt; c < B_BYTES / 16; c += XFORM_WARPS * 32) st_shared_16(sb + B_BYTES + c * 16, lo_of(ld_shared_16(sb + c * 16)));
#endif
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(full(s));
      }
    }
#endif
  } else {
    // ---------------------------------------------------------------- epilogue warps 2..5
    const int q = warp & 3;                 // TMEM lane quarter this warp may access
    const int cg0 = ((warp - 2) / 4) * (EPI_COLS / 16);   // first 16-column group of this warp's share of the tile
    int cc = 0;
    Seg sg;
    for (int si = 0; !failed && get_segment(si, sg); si++) {
      int b, m_blk, n_blk;
      tile_coords(sg.tile, b, m_blk, n_blk);
      const int m = m_blk * TILE_M + (int)rank * BM + q * 32 + lane;
      // epilogue and store of 16 consecutive outputs of this thread's row, from their accumulators
      auto finish16 = [&](int c, const float* accv) {
        const int n0 = n_blk * BN + sg.n_off + c * 16;
        if (m < GM && n0 < GN) {
          __align__(16) JX_OUT_T res[16];
          const int g0 = (int)(((i64)b * GM + m) * GN + n0);
          (void)g0;
          JX_EPI_PRELOAD
          #pragma unroll
          for (int j = 0; j < 16; j++) {
            const int n = n0 + j;
            const int gidx = (int)(((i64)b * GM + m) * GN + (n < GN ? n : GN - 1));
            const float acc = accv[j];
#define JX_DST res[j]
JX_EPILOGUE
#undef JX_DST
          }
          JX_OUT_T* dst = out + (((i64)b * GM + m) * GN + n0);
          if (n0 + 16 <= GN && (GN * sizeof(JX_OUT_T)) % 16 == 0) {
            #pragma unroll
            for (int j = 0; j < 16; j += 16 / sizeof(JX_OUT_T))
              *reinterpret_cast<jx_vec<16>*>(dst + j) = *reinterpret_cast<const jx_vec<16>*>(&res[j]);
          } else {
            for (int j = 0; j < 16 && n0 + j < GN; j++) dst[j] = res[j];
          }
        }
      };
      const int nch = (sg.kb1 - sg.kb0 + CHUNK_KB - 1) / CHUNK_KB;
#if NCHUNK > 1
      float sum[EPI_COLS];
      #pragma unroll
      for (int j = 0; j < EPI_COLS; j++) sum[j] = 0.0f;
      for (int ch = 0; ch < nch - 1 && !failed; ch++, cc++) {
        const int acc_i = cc & 1;
        if (!mbar_wait(tfull(acc_i), (cc >> 1) & 1, status)) { atomicCAS((int*)status_ptr, 0, 4); failed = true; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const u32 trow = tmem_base + ((u32)(q * 32) << 16) + acc_i * ACC_STRIDE;
        #pragma unroll
        for (int c = 0; c < EPI_COLS / 16; c++) {
          if (HALF_LAST && (cg0 + c) * 16 >= sg.bn) break;   // a half tile has no columns for the second group
          u32 v[16];
          tmem_ld16(trow + (cg0 + c) * 16, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          #pragma unroll
          for (int j = 0; j < 16; j++) sum[c * 16 + j] += __uint_as_float(v[j]);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) { if (CTA_PAIR) mbar_arrive_at(tempty(acc_i), 0); else mbar_arrive(tempty(acc_i)); }
      }
      if (failed) break;
#endif
      const int acc_i = cc & 1;
      if (!mbar_wait(tfull(acc_i), (cc >> 1) & 1, status)) { atomicCAS((int*)status_ptr, 0, 4); failed = true; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const u32 trow = tmem_base + ((u32)(q * 32) << 16) + acc_i * ACC_STRIDE;
      // a piece is laid out [16-column group][row][16]: a warp's 32 rows of one group are 2 KB in a row
      float* piece = sk_pieces + (size_t)sg.slot * BM * BN + (size_t)(q * 32 + lane) * 16;
#if NCHUNK > 1
      #pragma unroll
#else
      #pragma unroll 1
#endif
      for (int c = 0; c < EPI_COLS / 16; c++) {
        if (HALF_LAST && (cg0 + c) * 16 >= sg.bn) break;
        u32 v[16];
        tmem_ld16(trow + (cg0 + c) * 16, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        float accv[16];
        #pragma unroll
        for (int j = 0; j < 16; j++) {
#if NCHUNK > 1
          accv[j] = sum[c * 16 + j] + __uint_as_float(v[j]);
#else
          accv[j] = __uint_as_float(v[j]);
#endif
        }
        if (!sg.partial) {
          finish16(cg0 + c, accv);
        } else {
          #pragma unroll
          for (int j = 0; j < 16; j += 4)
            __stcg(reinterpret_cast<float4*>(piece + (size_t)c * BM * 16 + j), make_float4(accv[j], accv[j + 1], accv[j + 2], accv[j + 3]));
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) { if (CTA_PAIR) mbar_arrive_at(tempty(acc_i), 0); else mbar_arrive(tempty(acc_i)); }
      cc++;
#if STREAMK
      if (sg.partial) {
        // Every quarter of the tile (32 rows: one epilogue warp in each of the S CTAs that hold a
        // slice) is finished by the warp that arrives last.
        const int rest = NUM_TILES - sk_tiles_full(), S = sk_slices();
        const int sk_tile = sg.tile - sk_tiles_full();
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) last = atomicAdd(sk_counters + sk_tile * 4 + q, 1) == S - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
          #pragma unroll 1
          for (int c = 0; c < BN / 16; c++) {
            float accv[16];
            const size_t at = (size_t)c * BM * 16 + (size_t)(q * 32 + lane) * 16;
            #pragma unroll
            for (int j = 0; j < 16; j++) accv[j] = 0.0f;
            #pragma unroll 1
            for (int p0 = 0; p0 < S; p0 += 4) {      // four slices' loads in flight at a time, added in k order
              float4 f[4][4];
              #pragma unroll
              for (int p = 0; p < 4; p++)
                if (p0 + p < S) {
                  const float* src = sk_pieces + (size_t)((p0 + p) * rest + sk_tile) * BM * BN + at;   // slice p is CTA p * rest + sk_tile
                  #pragma unroll
                  for (int j = 0; j < 4; j++) f[p][j] = __ldcg(reinterpret_cast<const float4*>(src) + j);
                }
              #pragma unroll
              for (int p = 0; p < 4; p++)
                if (p0 + p < S) {
                  #pragma unroll
                  for (int j = 0; j < 4; j++) { accv[4 * j] += f[p][j].x; accv[4 * j + 1] += f[p][j].y; accv[4 * j + 2] += f[p][j].z; accv[4 * j + 3] += f[p][j].w; }
                }
            }
            finish16(c, accv);
          }
          if (lane == 0) sk_counters[sk_tile * 4 + q] = 0;   // ready for the next launch
        }
      }
#endif
    }
  }
  if (*status != 0) {
    // Wind-down after a time-out: give copies that are still in flight time to land before the
    // shared memory and the tensor memory of this CTA are released.
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (CTA_PAIR) cluster_sync();              // neither CTA frees tensor memory the other's MMAs or loads still use
  if (warp == 1) {
#if CTA_PAIR
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((u32)TMEM_COLS) : "memory");
#else
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((u32)TMEM_COLS) : "memory");
#endif
  }
}

#if KIND == 2
// Remainder planes of the f32 operands: lo = x - hi, hi = x with the low 13 mantissa bits cleared.
// The hi planes themselves are never materialised: a kind::tf32 MMA reads f32 words and ignores
// those 13 bits (verified on B200: results are bit-identical with explicit hi planes), so the
// original operand serves as hi.  Planes keep the operand's own indexing.
extern "C" __global__ void __launch_bounds__(256) jx_split(const float* __restrict__ a, const float* __restrict__ b,
                                                          float* __restrict__ plane_a, float* __restrict__ plane_b,
                                                          int do_a, int do_b) {
  // do_a / do_b: a plane that an earlier GEMM of the same step list already wrote is not written again
  const i64 na4 = do_a ? (i64)LEN_A / 4 : 0, nb4 = do_b ? (i64)LEN_B / 4 : 0;
  const i64 total4 = na4 + nb4;
  for (i64 i = (i64)blockIdx.x * 256 + threadIdx.x; i < total4; i += (i64)gridDim.x * 256) {
    const bool is_a = i < na4;
    const i64 j = is_a ? i : i - na4;
    const float4 v = reinterpret_cast<const float4*>(is_a ? a : b)[j];
    float4 lo;
    lo.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
    lo.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
    lo.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
    lo.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
    reinterpret_cast<float4*>(is_a ? plane_a : plane_b)[j] = lo;
  }
  if (blockIdx.x == 0 && threadIdx.x < 8) {     // the up to three trailing elements of each operand
    const bool is_a = threadIdx.x < 4;
    const i64 len = is_a ? (i64)LEN_A : (i64)LEN_B;
    const i64 j = (len / 4) * 4 + (threadIdx.x & 3);
    if (j < len && (is_a ? do_a : do_b)) {
      const float v = (is_a ? a : b)[j];
      (is_a ? plane_a : plane_b)[j] = v - __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    }
  }
}
#endif
)TCGEMM";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*LaunchFn)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                             void**, void**);

int64_t pad64(int64_t n) { return (n + 63) / 64 * 64; }  // planes start on 256-byte boundaries

}  // namespace

bool plan_gemm_tc(const KernelIR& k, const GemmDesc& g, const Options& opt, Plan& plan,
                  const std::string& epilogue_body, const std::string& params_decl, const std::string& epilogue_preload,
                  const std::string& gather_source) {
  if (g.dtA != g.dtB) return false;
  const int kind = g.dtA == JAXCUDA_F16 ? 1 : g.dtA == JAXCUDA_F32 ? 2 : 0;
  if (!kind) return false;
  const int e = kind == 1 ? 2 : 4;
  const bool a_mn = g.sAm == 1 && g.sAk != 1, b_mn = g.sBn == 1 && g.sBk != 1;
  if (!a_mn && g.sAk != 1) return false;
  if (!b_mn && g.sBk != 1) return false;
  const int64_t a_outer = a_mn ? g.sAk : g.sAm, b_outer = b_mn ? g.sBk : g.sBn;
  auto ok16 = [&](int64_t elems) { return elems > 0 && (elems * e) % 16 == 0; };
  if (!ok16(a_outer) || !ok16(b_outer)) return false;
  if ((g.offA * e) % 16 || (g.offB * e) % 16 || g.offA < 0 || g.offB < 0) return false;
  if (g.batch > 1 && (!ok16(g.sAb == 0 ? 16 : g.sAb) || !ok16(g.sBb == 0 ? 16 : g.sBb) || g.sAb < 0 || g.sBb < 0)) return false;
  if (g.M < 64 || g.N < 32 || g.K < 32) return false;
  if (g.N < 64 && (g.M < 256 || kind == 1)) return false;   // 32-column tiles: tall f32 outputs only (an MN-major f16 box is 64 columns wide)
  if ((uint64_t)g.lenA >= (1ull << 31) || (uint64_t)g.lenB >= (1ull << 31)) return false;

  const int BM = 128;
  const int bk = 128 / e;
  int BN = 64;
  for (int cand : {256, 128, 64}) {
    if (kind == 2 && cand == 256) continue;  // two planes per operand: 256 columns would leave two stages
    const int64_t tiles = ((g.M + BM - 1) / BM) * ((g.N + cand - 1) / cand) * g.batch;
    if (cand <= g.N && (tiles >= (int64_t)opt.sm_count * 3 / 4 || cand == 64)) { BN = cand; break; }
  }
  if (BN > g.N) BN = g.N >= 64 ? 64 : 32;   // 32 columns: one 128-byte box of f32, half a box of f16 columns (a vmapped batch of 32)
  // 3xTF32 on CTA pairs takes 256 columns after all: a CTA then holds half of B's columns per stage
  // (64 KB a stage, three stages), and two groups of epilogue warps split the columns so that each
  // thread keeps 128 partial sums.  Per k-block a CTA moves 208 KB through shared memory (TMA writes
  // plus the MMAs' operand reads, B's half served to both CTAs) for twice the products of a
  // 128 x 128 tile's 160 KB: that traffic, at 128 bytes a clock, is what bounds this kernel.
  const bool wide_pairs = kind == 2 && opt.tc_pair != 0 && opt.tc_bn == 0 && !g.b_gathered && g.M >= 2 * BM && g.N >= 256 &&
                          ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + 255) / 256) * g.batch * 2 >= opt.sm_count * 3 / 4;   // 1.5 times the work per byte is worth a quarter of the SMs idle
  if (wide_pairs) BN = 256;
  // A 192-column tile would shorten the static schedule of f16 4096^3 (512 tiles of 256 columns are
  // 3.46 waves of 148 CTAs), but measured slower (124 us against 108): narrower tiles re-read A from
  // shared memory more often per flop, and the MMA pipe is already fed at its limit with 256 columns.
  // The width stays selectable (Options::tc_bn) for experiments.
  if (opt.tc_bn == 64 || opt.tc_bn == 128 || (kind == 1 && (opt.tc_bn == 192 || opt.tc_bn == 256))) BN = std::min<int>(opt.tc_bn, (int)(g.N / 64 * 64));
  // Split-K (see get_segment in the kernel).  Measured on B200: an output with at most half as many
  // tiles as SMs and a long K gains (f32 512 x 512 x 4096: 80 -> 44 us); a last wave behind full waves
  // does not (f16 4096^3: 108 -> 121 us, f32 1024^3 at 128 x 128 tiles: 30 -> 33 us), because the warp
  // that adds a tile's slices up does so at the very end of the kernel in a chain of dependent L2
  // reads that costs more than the part of a wave it saves.  So only the first case is split; the
  // kernel handles both (JAXCUDA_TC_STREAMK=2 splits whenever at most half a wave is left over).
  const int64_t kb_total = (g.K + bk - 1) / bk;
  auto tiles_for = [&](int bn) { return ((g.M + BM - 1) / BM) * ((g.N + bn - 1) / bn) * g.batch; };
  bool streamk = opt.tc_streamk != 0;
  if (streamk && opt.tc_bn == 0 && kb_total >= 64) {
    for (int cand : {256, 128}) {   // few tiles anyway: take the widest that still leaves two slices per tile
      if (kind == 2 && cand == 256) continue;
      if (cand > g.N || cand <= BN) continue;
      if (tiles_for(cand) * 2 <= opt.sm_count) { BN = cand; break; }
    }
  }
  {
    const int64_t tiles = tiles_for(BN), rest = tiles % opt.sm_count;
    if (rest == 0 || rest * 2 > opt.sm_count || kb_total < 4) streamk = false;
    if (opt.tc_streamk != 2 && (tiles >= opt.sm_count || kb_total < 64)) streamk = false;
  }
  const int planes = kind == 2 ? 2 : 1;
  // CTA pairs (cta_group::2) on 256 x BN tiles: each CTA loads half of the B columns, so a third less
  // (BN = 256) or a quarter less (BN = 128) comes through L2 and shared memory per output.  Whole
  // tiles only, operands from TMA, and enough tiles to fill the 74 pairs.
  const int64_t pair_tiles = ((g.M + 2 * BM - 1) / (2 * BM)) * ((g.N + BN - 1) / BN) * g.batch;
  // Measured (B200): f16 4096^3 109 -> 104 us (1318 TFLOP/s); with K = 1024 or less the pair's extra
  // set-up costs more than it saves (23.0 -> 24.5 us), and 3xTF32 neither gains nor loses (its tiles
  // stay 128 columns wide per CTA), so by default pairs run f16 GEMMs with at least 32 k-blocks.
  // JAXCUDA_TC_PAIR: 0 never, 2 whenever the shape allows.
  const bool pair = !streamk && !g.b_gathered && g.M >= 2 * BM && BN >= 128 && (wide_pairs || pair_tiles * 2 >= opt.sm_count) &&
                    (opt.tc_pair == 2 || wide_pairs || (opt.tc_pair == 1 && kind == 1 && kb_total >= 32));
  const int epi_split = (pair && kind == 2 && BN == 256) ? 2 : 1;
  if (kind == 2 && BN == 256 && !pair) return false;   // (cannot happen: wide_pairs implies the pair conditions)
  const int stage_bytes = planes * (BM + (pair ? BN / 2 : BN)) * 128;
  int stages = (227 * 1024 - 2048) / stage_bytes;
  stages = std::max(2, std::min(stages, pair ? 8 : 6));
  const int64_t tiles = pair ? pair_tiles : ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) * g.batch;

  std::ostringstream os;
  os << kPrelude;
  os << "#define KIND " << kind << "\n#define ELEM " << e << "\n#define BM " << BM << "\n#define BN " << BN << "\n";
  os << "#define ACC_STRIDE " << (BN > 128 ? 256 : BN) << "\n";
  os << "#define A_SHARED " << ((g.batch > 1 && g.sAb == 0) ? 1 : 0) << "\n#define B_SHARED " << ((g.batch > 1 && g.sBb == 0) ? 1 : 0) << "\n";
  // CTA pairs on 256-column tiles whose last wave is at most half full run it as half-width tiles
  // (see get_segment; JAXCUDA_TC_HALF_LAST=0 keeps whole tiles)
  const int64_t pairs_in_grid = std::min<int64_t>(tiles, opt.sm_count / 2);
  // Measured: 3xTF32 8192 x 2048 x 2048 296 -> 284 us; f16 4096^3 103 -> 106 us (there a half tile
  // costs 0.8 of a whole one and the tensor pipe, not shared memory, is the bound), so 3xTF32 only
  // unless the option is 2.
  const bool half_last = pair && BN == 256 && (opt.tc_half_last == 2 || (opt.tc_half_last == 1 && kind == 2)) && tiles > pairs_in_grid &&
                         tiles % pairs_in_grid != 0 && 2 * (tiles % pairs_in_grid) <= pairs_in_grid;
  os << "#define STREAMK " << (streamk ? 1 : 0) << "\n#define CTA_PAIR " << (pair ? 1 : 0) << "\n#define EPI_SPLIT " << epi_split
     << "\n#define HALF_LAST " << (half_last ? 1 : 0) << "\n";
  os << "#define SPIN_LIMIT " << std::max(1024, opt.tc_spin_limit) << "\n#define FAULT_SKIP_LOAD " << (opt.tc_fault == 1 ? 1 : 0) << "\n";
  // Gather warps of a convolution (B_GATHER): groups of four warps, each group filling every
  // gather_groups-th stage.  Never more groups than stages: a group waits for "stage free" by phase
  // parity, which only tells apart two consecutive phases, and the wait of one group for a stage's
  // next use is behind the previous use's completion only while groups <= stages (with four groups
  // on three stages a group ran two phases ahead, passed its wait at once and overwrote a stage that
  // was still being read: "unspecified launch failure").  Measured for N=32, 64 -> 128 channels,
  // 56 x 56, 3 x 3: f32 8 warps in 2 groups 132 us (12 in 3: 140), f16 12 warps in 3 groups 69 us (8 in 2: 74).
  const int gather_groups = g.b_implicit ? std::min(stages, kind == 2 ? 2 : 3) : 1;
  const int gather_warps = g.b_implicit ? 4 * gather_groups : 0;
  // Remainder tiles made in the kernel save the split pass (a launch and a round trip of both
  // operands through global memory) but add a read and a write of every stage to the shared-memory
  // traffic that already bounds the 3xTF32 main loop.  Measured: 1024^3 (one wave of tiles) 30.1 ->
  // 27.2 us, 8192 x 2048 x 2048 320 -> 339 us, the convolution 131 -> 149 us, one wave of tiles over a long K
  // (784 x 2048 x 65536) 1427 -> 1501 us.  So: outputs of at most one wave of tiles and at most 64
  // k-blocks (JAXCUDA_TC_LO_IN_KERNEL = 0 never, 2 always).
  const bool lo_in_kernel = kind == 2 && !(g.b_gathered && !g.b_implicit) &&
                            !pair && (opt.tc_lo_in_kernel == 2 || (opt.tc_lo_in_kernel == 1 && !g.b_gathered && tiles <= opt.sm_count && kb_total <= 64));
  const int xform_warps = lo_in_kernel ? 4 : 0;
  os << "#define LO_IN_KERNEL " << (lo_in_kernel ? 1 : 0) << "\n#define XFORM_WARPS " << xform_warps << "\n";
  os << "#define B_GATHER " << (g.b_implicit ? 1 : 0) << "\n#define GATHER_WARPS " << gather_warps << "\n#define GATHER_GROUPS " << gather_groups << "\n";
  os << "#define STAGES " << stages << "\n#define A_MN " << (a_mn ? 1 : 0) << "\n#define B_MN " << (b_mn ? 1 : 0) << "\n";
  os << "#define GM " << g.M << "\n#define GN " << g.N << "\n#define GK " << g.K << "\n#define GBATCH " << g.batch << "\n";
  // k-blocks accumulated in tensor memory before the partial sum is folded into registers with a
  // rounded f32 add: 256 elements of K for 3xTF32; the whole K for f16 (its f16 result absorbs the bias)
  const int64_t k_blocks = (g.K + bk - 1) / bk;
  os << "#define CHUNK_KB " << (kind == 2 ? 8 : k_blocks) << "\n";
  // a gathered B operand arrives with its remainder plane already written: only A is split
  os << "#define LEN_A " << g.lenA << "LL\n#define LEN_B " << (g.b_gathered ? 0 : g.lenB) << "LL\n";
  os << "#define LEN_A_PAD " << pad64(g.lenA) << "LL\n#define LEN_B_PAD " << pad64(g.lenB) << "LL\n";
  // scratch: [gathered B and its remainder plane][remainder planes of the operands][stream-K counters][stream-K pieces]
  size_t sk_offset = 0;
  if (g.b_gathered && !g.b_implicit) sk_offset += (size_t)pad64(g.lenB) * e * planes;
  if (kind == 2 && !lo_in_kernel) sk_offset += (size_t)(pad64(g.lenA) + (g.b_gathered ? 0 : pad64(g.lenB))) * 4;
  sk_offset = (sk_offset + 255) / 256 * 256;
  const size_t sk_counter_bytes = 4096;   // 4 counters per left-over tile, fewer than 148 of them
  const size_t sk_bytes = streamk ? sk_counter_bytes + (size_t)opt.sm_count * BM * BN * 4 : 0;   // one slice per CTA
  os << "#define SK_OFFSET " << sk_offset << "ULL\n#define SK_COUNTER_BYTES " << sk_counter_bytes << "ULL\n";
  const char* out_t = k.out_dtype() == JAXCUDA_F16 ? "jx_half" : k.out_dtype() == JAXCUDA_F64 ? "double"
                      : k.out_dtype() == JAXCUDA_U32 ? "u32" : k.out_dtype() == JAXCUDA_F32 ? "float" : "int";
  os << "#define JX_OUT_T " << out_t << "\n";
  os << "#define JX_PARAMS " << params_decl << "\n";
  {  // the same parameters by name, for calls that pass them on
    std::string names, decl = params_decl + ",";
    size_t start = 0;
    for (size_t i = 0; i < decl.size(); i++) {
      if (decl[i] != ',') continue;
      size_t end = i;
      while (end > start && isspace((unsigned char)decl[end - 1])) end--;
      size_t b0 = end;
      while (b0 > start && (isalnum((unsigned char)decl[b0 - 1]) || decl[b0 - 1] == '_')) b0--;
      names += (names.empty() ? "" : ", ") + decl.substr(b0, end - b0);
      start = i + 1;
    }
    os << "#define JX_PARAM_NAMES " << names << "\n";
  }
  std::string body = epilogue_body;  // newlines inside a macro need continuation
  std::string escaped;
  for (char c : body) { if (c == '\n') escaped += " \\\n"; else escaped += c; }
  os << "#define JX_EPILOGUE " << escaped << "\n";
  // loads of the epilogue that are contiguous over a thread's 16 outputs, fetched as 128-bit vectors
  // ahead of the per-element code (empty when there are none or rows are not a multiple of 16 wide)
  std::string pre;
  for (char c : epilogue_preload) { if (c == '\n') pre += " \\\n"; else pre += c; }
  os << "#define JX_EPI_PRELOAD " << pre << "\n";
  os << kTcSource;
  if (g.b_gathered) os << gather_source;
  plan.source = os.str();
  plan.skeleton = SK_GEMM_TC;
  plan.tc_kind = kind;
  plan.tc_bm = BM; plan.tc_bn = BN; plan.tc_bk = bk; plan.tc_stages = stages;
  plan.stages.clear();
  plan.scratch_bytes = 0;
  if (g.b_gathered && !g.b_implicit) {   // scratch: [B][B remainder plane (3xTF32)][A remainder plane (3xTF32)]
    Stage ga;
    ga.entry = "jx_gather_b";
    ga.grid[0] = (unsigned)std::max<int64_t>(1, (g.b_pitch / 4 * g.batch + 255) / 256);  // a thread per four pixels ...
    ga.grid[1] = (unsigned)std::max<int64_t>(1, (g.K + 31) / 32);                         // ... and 32 values of k (emit.cpp: kGatherKChunk)
    ga.block[0] = 256;
    plan.stages.push_back(ga);
    plan.scratch_bytes = (size_t)pad64(g.lenB) * e * planes;
  }
  plan.tc_lo_in_kernel = lo_in_kernel;
  if (kind == 2 && !lo_in_kernel) {
    Stage sp;
    sp.entry = "jx_split";
    const int64_t split_len = g.lenA + (g.b_gathered ? 0 : g.lenB);
    sp.grid[0] = (unsigned)std::max<int64_t>(1, std::min<int64_t>((split_len / 4 + 255) / 256, (int64_t)opt.sm_count * 32));
    sp.block[0] = 256;
    plan.stages.push_back(sp);
    plan.scratch_bytes += (size_t)(pad64(g.lenA) + (g.b_gathered ? 0 : pad64(g.lenB))) * 4;
  }
  if (streamk) plan.scratch_bytes = sk_offset + sk_bytes;
  plan.tc_sk_offset = streamk ? sk_offset : 0;
  plan.tc_sk_counter_bytes = streamk ? sk_counter_bytes : 0;
  Stage st;
  st.entry = "jx_gemm";
  st.grid[0] = streamk ? (unsigned)opt.sm_count
               : pair  ? (unsigned)std::min<int64_t>(2 * tiles, opt.sm_count & ~1)
                       : (unsigned)std::min<int64_t>(tiles, opt.sm_count);
  st.cluster = pair ? 2 : 1;
  plan.tc_pair = pair;
  st.block[0] = 64 + 128 * epi_split + 32 * (gather_warps + xform_warps);
  st.smem = (unsigned)(stages * stage_bytes + 1024 + (3 * stages + 4) * 8 + 16);
  plan.stages.push_back(st);
  plan.describe = std::string("gemm-tcgen05 ") + (kind == 1 ? "f16" : "3xtf32") + " " + std::to_string(g.batch) + "x" +
                  std::to_string(g.M) + "x" + std::to_string(g.N) + "x" + std::to_string(g.K) + " tile " + (pair ? "256x" : "128x") +
                  std::to_string(BN) + "x" + std::to_string(bk) + " stages=" + std::to_string(stages) + " A:" +
                  (a_mn ? "MN" : "K") + " B:" + (b_mn ? "MN" : "K") + " ctas=" + std::to_string(st.grid[0]) +
                  (pair ? " cta-pairs" : "") + (half_last ? " half-tiles-last" : "") + (lo_in_kernel ? " lo-in-kernel" : "") +
                  (streamk ? " split-k" : "");
  return true;
}

int launch_gemm_tc(void* encode_fn, void* launch_fn, void* launch_ex_fn, const Plan& plan, const std::vector<CUfunction>& fns,
                   const std::vector<void*>& inputs, void* out, void* scratch, cudaStream_t stream,
                   int* status_dev, std::string& err, int max_ctas, const LoPlanes* lo) {
  auto encode = (EncodeTiledFn)encode_fn;
  auto launch = (LaunchFn)launch_fn;
  const GemmDesc& g = plan.gemm;
  const int kind = plan.tc_kind;
  const int e = kind == 1 ? 2 : 4;
  const bool a_mn = g.sAm == 1 && g.sAk != 1, b_mn = g.sBn == 1 && g.sBk != 1;
  int launches = 0;
  size_t stage_i = 0;
  const char* baseA = (const char*)inputs[g.gidA];
  const char* baseB = g.b_implicit ? (const char*)inputs[g.gidA] : g.b_gathered ? (const char*)scratch : (const char*)inputs[g.gidB];
  const char* baseA2 = baseA;
  const char* baseB2 = baseB;
  char* split_planes = (char*)scratch;
  if (g.b_gathered && !g.b_implicit) {
    // the gather kernel takes the Kernel's own parameters (inputs, out, scratch) and fills B (and its
    // remainder plane) at the start of the scratch
    std::vector<void*> gp(inputs.begin(), inputs.end());
    gp.push_back(out);
    gp.push_back(scratch);
    std::vector<void*> gargs;
    for (auto& p : gp) gargs.push_back(&p);
    const Stage& ga = plan.stages[stage_i];
    CUresult r = launch(fns[stage_i], ga.grid[0], ga.grid[1], 1, ga.block[0], 1, 1, 0, (CUstream)stream, gargs.data(), nullptr);
    if (r != CUDA_SUCCESS) { err = "launch of the operand gather kernel failed"; return -1; }
    launches++;
    stage_i++;
    const size_t plane_bytes = (size_t)pad64(g.lenB) * e;
    baseB2 = baseB + plane_bytes;
    split_planes = (char*)scratch + plane_bytes * (kind == 2 ? 2 : 1);
  }
  if (kind == 2 && !plan.tc_lo_in_kernel) {
    // remainder planes: in the scratch, or where the caller keeps them across the GEMMs of a step list
    float* plane_a = (lo && lo->a) ? lo->a : (float*)split_planes;
    float* plane_b = (lo && lo->b) ? lo->b : (float*)split_planes + pad64(g.lenA);
    int do_a = !(lo && lo->a && !lo->compute_a), do_b = !(lo && lo->b && !lo->compute_b);
    const char* split_b = g.b_gathered ? baseA : baseB;   // not read when LEN_B is 0
    if (do_a || (do_b && !g.b_gathered)) {
      void* args[] = {(void*)&baseA, (void*)&split_b, (void*)&plane_a, (void*)&plane_b, (void*)&do_a, (void*)&do_b};
      const Stage& sp = plan.stages[stage_i];
      CUresult r = launch(fns[stage_i], sp.grid[0], 1, 1, sp.block[0], 1, 1, 0, (CUstream)stream, args, nullptr);
      if (r != CUDA_SUCCESS) { err = "launch of the TF32 split kernel failed"; return -1; }
      launches++;
    }
    stage_i++;
    baseA2 = (const char*)plane_a;                    // lo planes; the operands themselves are the hi terms
    if (!g.b_gathered) baseB2 = (const char*)plane_b;
  }
  const CUtensorMapDataType dt = kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  const cuuint32_t inner_box = 128 / e;
  auto make_map = [&](CUtensorMap* m, const char* base, int64_t off, bool mn, int64_t mn_extent, int64_t k_extent,
                      int64_t outer_stride, int64_t batch_stride, int rows_box) -> bool {
    // dim 0 is the contiguous one: k for a K-major operand, m/n for an MN-major one
    // an operand every batch shares (batch stride 0) is described as a single plane; the kernel reads it at batch 0
    cuuint64_t dims[3] = {(cuuint64_t)(mn ? mn_extent : k_extent), (cuuint64_t)(mn ? k_extent : mn_extent),
                          (cuuint64_t)((g.batch > 1 && batch_stride == 0) ? 1 : g.batch)};
    cuuint64_t bs = batch_stride > 0 ? (cuuint64_t)batch_stride * e : dims[1] * (cuuint64_t)outer_stride * e;
    cuuint64_t strides[2] = {(cuuint64_t)outer_stride * e, bs};
    cuuint32_t box[3] = {inner_box, (cuuint32_t)rows_box, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    // MN-major 32-bit operands must sit in shared memory in the 128-byte swizzle with 32-byte atoms
    const CUtensorMapSwizzle sw = (mn && e == 4) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    CUresult r = encode(m, dt, 3, (void*)(base + off * e), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
  };
  alignas(64) CUtensorMap tmA, tmA2, tmB, tmB2;
  const int bk = plan.tc_bk;
  const int b_rows = plan.tc_pair ? plan.tc_bn / 2 : plan.tc_bn;   // columns of B one CTA loads per stage
  const int64_t a_outer = a_mn ? g.sAk : g.sAm, b_outer = b_mn ? g.sBk : g.sBn;
  bool ok = make_map(&tmA, baseA, g.offA, a_mn, g.M, g.K, a_outer, g.sAb, a_mn ? bk : plan.tc_bm) &&
            make_map(&tmA2, baseA2, g.offA, a_mn, g.M, g.K, a_outer, g.sAb, a_mn ? bk : plan.tc_bm) &&
            (g.b_implicit || (make_map(&tmB, baseB, g.offB, b_mn, g.N, g.K, b_outer, g.sBb, b_mn ? bk : b_rows) &&
                              make_map(&tmB2, baseB2, g.offB, b_mn, g.N, g.K, b_outer, g.sBb, b_mn ? bk : b_rows)));
  if (g.b_implicit) { tmB = tmA; tmB2 = tmA; }   // not read: the kernel fills the B stages itself
  if (!ok) { err = "cuTensorMapEncodeTiled rejected a GEMM operand"; return -1; }
  std::vector<void*> ptrs(inputs.begin(), inputs.end());
  ptrs.push_back(out);
  ptrs.push_back(scratch);
  std::vector<void*> args;
  args.push_back(&tmA); args.push_back(&tmA2); args.push_back(&tmB); args.push_back(&tmB2);
  for (auto& p : ptrs) args.push_back(&p);
  args.push_back(&status_dev);
  if (plan.tc_sk_counter_bytes) {   // arrival counters of the stream-K pieces start every launch at zero
    if (cudaMemsetAsync((char*)scratch + plan.tc_sk_offset, 0, plan.tc_sk_counter_bytes, stream) != cudaSuccess) {
      err = "clearing the stream-K counters failed";
      return -1;
    }
  }
  const Stage& st = plan.stages.back();
  unsigned grid = max_ctas > 0 ? std::min<unsigned>(st.grid[0], (unsigned)max_ctas) : st.grid[0];
  CUresult r;
  if (st.cluster > 1) {
    typedef CUresult (*LaunchExFn)(const CUlaunchConfig*, CUfunction, void**, void**);
    auto launch_ex = (LaunchExFn)launch_ex_fn;
    if (!launch_ex) { err = "cuLaunchKernelEx is unavailable"; return -1; }
    grid = std::max(st.cluster, grid / st.cluster * st.cluster);
    CUlaunchAttribute attr;
    memset(&attr, 0, sizeof attr);
    attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr.value.clusterDim.x = st.cluster;
    attr.value.clusterDim.y = 1;
    attr.value.clusterDim.z = 1;
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = grid; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = st.block[0]; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = st.smem;
    cfg.hStream = (CUstream)stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    r = launch_ex(&cfg, fns.back(), args.data(), nullptr);
  } else {
    r = launch(fns.back(), grid, 1, 1, st.block[0], 1, 1, st.smem, (CUstream)stream, args.data(), nullptr);
  }
  if (r != CUDA_SUCCESS) { err = "launch of the tcgen05 GEMM kernel failed"; return -1; }
  launches++;
  return launches;
}

}  // namespace jaxcuda
