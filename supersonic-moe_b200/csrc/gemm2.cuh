// Two-CTA (cta_group::2) variant of the MXFP8 grouped GEMM: a pair of CTAs on
// neighbouring SMs computes one 256 x BN tile.  Each CTA stages its own 128 rows
// of A and its own half of the B tile (no multicast loads anywhere); the leader
// CTA issues tcgen05.mma for both, each CTA keeps its 128 x BN accumulator in
// its own TMEM (two stages, so the epilogue of tile i overlaps the main loop of
// tile i+1) and drains it with eight epilogue warps.  Outputs go through a
// swizzled shared-memory staging buffer and TMA stores / TMA reduce-adds.
#pragma once
#include "gemm.cuh"

namespace smoe {

constexpr int kEpiWarps2 = 8;
constexpr int kThreads2 = 32 * (2 + kEpiWarps2);
constexpr int kMaxExperts2 = 256;   // expert offsets cached in shared memory by the two-CTA kernel
constexpr int kDefaultL2Prefetch = 0;
constexpr int kSfGroup2 = 4;        // K tiles whose scales travel in one TMA copy (box rows of the scale tensor maps)

// ---- cluster helpers -------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address of this CTA -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The same without memory-ordering semantics, for hand-overs that pass no data through memory: an epilogue warp that
// has read its accumulator columns out of TMEM (tcgen05.wait::ld + tcgen05.fence::before_thread_sync order those
// reads) tells the MMA issuer so.  The releasing form makes the arrival wait for every earlier store of the thread
// - the staging stores of the previous tile among them - to become visible cluster-wide: 1700 cycles in the
// 256 x 384 kernel, at every tile boundary, with the tensor pipe idle.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Releasing at CTA scope (the form without qualifiers): orders this thread's earlier writes to ITS OWN shared memory
// - which is where the data the arrival announces lies - without the cluster-wide flush.
__device__ __forceinline__ void mbar_arrive_cluster_cta_release(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Loads of a CTA pair: data lands in the issuing CTA, the byte count is
// credited to the barrier named by a shared::cluster address (the leader's).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_gather4_pair(uint32_t dst, const void* tmap, uint32_t bar_cluster, int c0, int r0,
                                                 int r1, int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
      : "memory");
}
// Operand tile -> L2 only (no shared memory, no barrier): warms the line the ring will ask for a few K tiles later.
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void mma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// The same with the shared-memory descriptors given as (low word, high word): the high words are constants of the
// kernel, only the low words (start address) move, so the issuing warp carries 32-bit values only.
__device__ __forceinline__ void mma_mxf8_pair_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                 uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %4, [%6], [%7], p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair_lo(uint32_t dst_tmem, uint32_t src_lo, uint32_t src_hi) {
  asm volatile(
      "{\n\t.reg .b64 d;\n\t"
      "mov.b64 d, {%1, %2};\n\t"
      "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}"
      ::"r"(dst_tmem), "r"(src_lo), "r"(src_hi)
      : "memory");
}
// completion of all MMAs issued so far -> one arrival on the barrier at this
// offset in every CTA of `mask`
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t dst_tmem, uint64_t src_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(src_desc) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// sigmoid with two MUFU ops (ex2 + rcp); relative error ~1e-7, far below the
// bf16 / e4m3 resolution of everything it feeds
__device__ __forceinline__ float fast_sigmoid(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return r;
}

// element-wise max of two bf16 pairs
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// max |x| over the warp, delivered to every lane
__device__ __forceinline__ float warp_max_abs(float x) {
  float r;
  asm volatile("redux.sync.max.abs.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(x));
  return r;
}

// CPG: the rows of A are gathered by index inside the kernel with cp.async (four extra load warps per CTA) instead of
// arriving as TMA tiles of a pre-gathered copy.
template <int BN, int MODE, bool CPG = false>
struct Gemm2Smem {
  static constexpr int GATHER_WARPS = CPG ? 4 : 0;        // load warps; one more warp forwards "rows have landed"
  static constexpr int EXTRA_WARPS = CPG ? GATHER_WARPS + 1 : 0;
  static constexpr int A_BYTES = BM * BK;                 // this CTA's 128 rows
  static constexpr int B_BYTES = (BN / 2) * BK;           // this CTA's half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SFB_TILES = (BN == 128) ? 1 : 2;   // 128-row scale tiles covering the BN window
  // Scales travel in their own ring: one slot holds the scales of SF_GROUP consecutive K tiles (A: SF_GROUP x 512 B,
  // B: SF_GROUP x 512 B per 128-row tile), fetched with one TMA copy per operand tile instead of one per K tile.
  // (A deeper ring of smaller groups - 5 slots of 2 K tiles - measured 10 % slower: the extra TMA copies and
  // barrier traffic cost more than the longer prefetch distance gains.)
  static constexpr int SF_GROUP = kSfGroup2;
  static constexpr int SF_SLOT_BYTES = SF_GROUP * 512 * (1 + SFB_TILES);
  // output staging per epilogue warp: PLAIN 2 KB (bf16 32x32), WGRAD 2 KB (f32 32x16),
  // DGATED 4 KB (dz) + 2 KB (y1s), GATED 2 KB (z e4m3 32x64) + 1 KB (y1 e4m3 32x32)
  // DGATEDQ 2 KB (dz e4m3 32x64) + 1 KB (y1s e4m3 32x32)
  static constexpr int EPI_BYTES_PER_WARP = MODE == GATED ? 3072 : (MODE == DGATED ? 6144 : (MODE == DGATEDQ ? 3072 : 2048));
  // epilogue warps: four TMEM lane quadrants x COL_GROUPS column groups.  (Three groups of 64 columns on the
  // 192-column gated tiles measured slower than two: 646 vs 619 us up-projection, 412 vs 385 us fused dgated.)
  static constexpr int COL_GROUPS = 2;
  static constexpr int EPI_WARPS = 4 * COL_GROUPS;
  // the last warp brings the scales: a producer of its own, so that they are requested as soon as a slot of their
  // ring is free (up to two groups of K tiles ahead of the MMAs) instead of when the operand ring gets there
  static constexpr int SF_WARP = 2 + EPI_WARPS + EXTRA_WARPS;
  static constexpr int THREADS = 32 * (SF_WARP + 1);
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BYTES_PER_WARP;
  static constexpr int AUX_BYTES = 512 + 2 * (kMaxExperts2 + 1) * 4 + 8;      // barriers etc. + expert offsets
  static constexpr int BUDGET = 227 * 1024 - 1024 - AUX_BYTES - EPI_BYTES;    // 1024: alignment slack
  static constexpr int SF_SLOTS = 2;
  static constexpr int STAGES_RAW = (BUDGET - SF_SLOTS * SF_SLOT_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int SF_BYTES = SF_SLOTS * SF_SLOT_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + SF_BYTES + EPI_BYTES + AUX_BYTES + 1024;
  static_assert(TOTAL <= 227 * 1024, "shared memory budget");
  static_assert((3 * STAGES + 4 + 2 * SF_SLOTS) * 8 <= 496, "barrier storage");
  static constexpr int ACC_STAGES = (BN == 256) ? 1 : 2;  // TMEM: 512 columns
  static constexpr int SF_COLS = 4 + 4 * SFB_TILES;
  static constexpr int SF_COL0 = ACC_STAGES * BN;
  static_assert(SF_COL0 + STAGES * SF_COLS <= 512, "TMEM budget");
  // bytes the TMA copies of one stage credit to the full barrier: both CTAs' B, and A unless the load warps bring it
  static constexpr uint32_t TX_BYTES = 2u * ((CPG ? 0 : A_BYTES) + B_BYTES);
  static constexpr uint32_t FULL_ARRIVALS = CPG ? 3 : 1;    // the producer's expect_tx (+ both CTAs' forwarders)
  static constexpr uint32_t SF_TX_BYTES = 2u * SF_SLOT_BYTES;            // both CTAs' scales per group
};

struct PairTile {
  int m0;       // first row of this CTA's 128 rows (A' / C rows; WGRAD: output rows)
  int n0;       // first output column
  int e;        // expert
  int kt0, nkt; // K-tile range
  int valid;    // 0: this CTA's half lies beyond its expert's rows - compute, store nothing
  int prob;     // WGRAD with two products in one launch: which one this tile belongs to
};

// varlen-M: experts own ceil(n_e / 2) row pairs; s_pairs = exclusive prefix of that.
template <int BN, int MODE>
__device__ __forceinline__ PairTile pair_tile(int tile, int rank, const GemmParams& p, const int* s_efo,
                                              const int* s_pairs) {
  PairTile t;
  const int n_tiles = (p.N + BN - 1) / BN;     // DGATEDQ may run a ragged last column tile
  t.prob = 0;
  if (MODE == WGRAD) {
    int m_pairs = p.rows / (2 * BM);
    int per_e = m_pairs * n_tiles;
    if (p.rows2 > 0 && tile >= p.E * per_e) {       // tiles of the second product follow those of the first
      tile -= p.E * per_e;
      t.prob = 1;
      m_pairs = p.rows2 / (2 * BM);
      per_e = m_pairs * n_tiles;
    }
    t.e = tile / per_e;
    const int r = tile - t.e * per_e;
    t.m0 = (r / n_tiles) * 2 * BM + rank * BM;
    t.n0 = (r % n_tiles) * BN;
    t.kt0 = s_efo[t.e] / BK;
    t.nkt = (s_efo[t.e + 1] - s_efo[t.e]) / BK;
    t.valid = 1;
  } else {
    const int pr = tile / n_tiles;
    t.n0 = (tile - pr * n_tiles) * BN;
    int lo = 0, hi = p.E;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_pairs[mid + 1] <= pr) lo = mid + 1; else hi = mid;
    }
    t.e = lo;
    const int j = pr - s_pairs[lo];
    t.m0 = s_efo[lo] + (2 * j + rank) * BM;
    t.valid = t.m0 < s_efo[lo + 1];
    t.kt0 = 0;
    t.nkt = p.K / BK;
  }
  return t;
}

template <int BN, int MODE, bool CPG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((Gemm2Smem<BN, MODE, CPG>::THREADS), 1)
gemm2_mxf8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                  const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_c2,
                  const __grid_constant__ CUtensorMap tmap_c3, const GemmParams p) {
  using S = Gemm2Smem<BN, MODE, CPG>;
  const bool GATHER = !CPG && p.a_idx != nullptr;   // rows of A fetched by index with TMA gather4 vs. a plain tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sfring = smem + S::STAGES * S::STAGE_BYTES;
  uint8_t* epi = sfring + S::SF_BYTES;
  uint8_t* aux = epi + S::EPI_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux);     // full[S], empty[S], tfull[2], tempty[2], sffull[2], sfempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 496);
  volatile int* s_abort = reinterpret_cast<volatile int*>(aux + 500);
  int* s_efo = reinterpret_cast<int*>(aux + 512);
  int* s_pairs = s_efo + (kMaxExperts2 + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs_grid = gridDim.x >> 1;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * S::STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * S::STAGES;
  const uint32_t bar_tempty = bar_tfull + 8 * 2;
  const uint32_t bar_sffull = bar_tempty + 8 * 2;
  const uint32_t bar_sfempty = bar_sffull + 8 * S::SF_SLOTS;
  const uint32_t bar_landed = bar_sfempty + 8 * S::SF_SLOTS;    // CPG: this CTA's gathered rows of a stage are in place

  for (int i = threadIdx.x; i <= p.E; i += blockDim.x) s_efo[i] = p.efo[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.E; ++e) {
      s_pairs[e] = acc;
      acc += ((s_efo[e + 1] - s_efo[e]) / BM + 1) >> 1;
    }
    s_pairs[p.E] = acc;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, S::FULL_ARRIVALS);   // leader's: its producer arms it, both CTAs' copies credit it
      mbar_init(bar_empty + 8 * s, 1);       // one commit arrival per use, in each CTA
      if (CPG) mbar_init(bar_landed + 8 * s, 32 * S::GATHER_WARPS);   // one arrival per load thread
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);                   // commit arrival, in each CTA
      mbar_init(bar_tempty + 8 * s, 2 * S::EPI_WARPS);     // leader's: the epilogue warps of both CTAs
    }
    for (int s = 0; s < S::SF_SLOTS; ++s) {
      mbar_init(bar_sffull + 8 * s, 1);                  // leader's: armed by its producer, credited by both CTAs
      mbar_init(bar_sfempty + 8 * s, 1);                 // commit arrival, in each CTA
    }
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc2(smem_u32(tmem_slot), 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t sf_base = smem_u32(sfring);
  const int n_col_tiles = (p.N + BN - 1) / BN;
  const int n_total = (MODE == WGRAD) ? p.E * (p.rows / (2 * BM)) * n_col_tiles : s_pairs[p.E] * n_col_tiles;
  const int nst = S::STAGES - p.dbg_stage_cut;       // ring stages in use (all of them outside timing experiments)

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    // Warp-uniform loops, one elected lane issues (see the MMA issuer below for why); only the gather path keeps
    // per-lane state (four row indices each).
    if (lane == 0) {
      prefetch_tmap(&tmap_a); prefetch_tmap(&tmap_b);
    }
    const uint32_t full0 = map_to_cta(bar_full, 0);      // the leader's full barriers
    const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
    // MN-major operands: both of a weight gradient, or the B of a PLAIN product whose weights lie [E, K, N]
    const bool a_mn = MODE == WGRAD && p.a_mn, b_mn = (MODE == WGRAD || MODE == PLAIN) && p.b_mn;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    const bool dbg_noload = (p.debug_skip_store & 4) != 0;   // timing experiment: operands fetched for one ring pass only
    int dbg_filled = 0;
    for (int tile = pair_id; tile < n_total_u && ok; tile += n_pairs_grid) {
      const PairTile tl = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      const int nkt = __shfl_sync(0xffffffffu, tl.nkt, 0);
      if (nkt == 0) continue;
      const int kt0 = __shfl_sync(0xffffffffu, tl.kt0, 0);
      const int valid = __shfl_sync(0xffffffffu, tl.valid, 0);
      const int m0 = __shfl_sync(0xffffffffu, tl.m0, 0);
      const int n0 = __shfl_sync(0xffffffffu, tl.n0, 0);
      const int te = __shfl_sync(0xffffffffu, tl.e, 0);
      int4 rows4 = make_int4(0, 0, 0, 0);
      if (GATHER && valid) rows4 = *reinterpret_cast<const int4*>(p.a_idx + m0 + 4 * lane);
      const int b_base = (MODE == WGRAD) ? n0 : te * p.N + n0;
      const bool b_mn_plain = MODE == PLAIN && b_mn;       // B of expert te = rows [te*K, (te+1)*K) of an [E*K, N] matrix
      const int b_row = (b_mn_plain ? n0 : b_base) + rank * (BN / 2);
      const int b_k0 = b_mn_plain ? te * p.K : 0;
      const int a_row = valid ? m0 : 0;
      for (int kt = kt0; kt < kt0 + nkt; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1));
        if (!ok) break;
        const uint32_t full = full0 + 8 * stage;
        const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
        const uint32_t b_dst = a_dst + S::A_BYTES;
        if (!CPG && dbg_noload && dbg_filled >= nst) {
          if (rank == 0 && elect_one()) mbar_arrive(bar_full + 8 * stage);
        } else {
          ++dbg_filled;
          if (elect_one()) {
            if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, S::TX_BYTES);
            if (a_mn) tma_load_2d_pair(a_dst, &tmap_a, full, m0, kt * BK);
            else if (!GATHER && !CPG) tma_load_2d_pair(a_dst, &tmap_a, full, kt * BK, a_row);
            if (b_mn) tma_load_2d_pair(b_dst, &tmap_b, full, b_row, b_k0 + kt * BK);
            else tma_load_2d_pair(b_dst, &tmap_b, full, kt * BK, b_row);
            const int kp = kt + p.l2_prefetch;
            if (p.l2_prefetch > 0 && kp < kt0 + nkt) {
              if (a_mn) tma_prefetch_l2_2d(&tmap_a, m0, kp * BK);
              else if (!GATHER && !CPG) tma_prefetch_l2_2d(&tmap_a, kp * BK, a_row);
              if (b_mn) tma_prefetch_l2_2d(&tmap_b, b_row, b_k0 + kp * BK);
              else tma_prefetch_l2_2d(&tmap_b, kp * BK, b_row);
            }
          }
          if (GATHER) {
            __syncwarp();
            tma_gather4_pair(a_dst + lane * 4 * BK, &tmap_a, full, kt * BK, rows4.x, rows4.y, rows4.z, rows4.w);
          }
        }
        if (++stage == nst) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 201); }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    // The whole warp walks the loops in lock step and one elected lane issues.  Every loop-carried value (stage,
    // phases, descriptor words) is then the same in all lanes, which lets the compiler keep the operands of the
    // tcgen05 instructions in uniform registers; with the loops inside a single-lane branch each operand had to be
    // moved over per instruction, and the issue rate of this one thread - not the tensor pipe, the operand loads or
    // the accumulator drain - bounded the kernel (900-1000 clocks per K tile where the MMAs need 512).
    if (rank == 0) {
      // WGRAD may take either operand MN-major: [K rows, M or N bytes] tiles instead of [M or N rows, K bytes]
      const bool a_mn = MODE == WGRAD && p.a_mn, b_mn = (MODE == WGRAD || MODE == PLAIN) && p.b_mn;
      const uint32_t idesc = make_idesc_mxf8(2 * BM, BN) | (a_mn ? 1u << 15 : 0u) | (b_mn ? 1u << 16 : 0u);
      const uint32_t idesc_kb[4] = {idesc_with_sf_ids(idesc, 0, 0), idesc_with_sf_ids(idesc, 1, 1),
                                    idesc_with_sf_ids(idesc, 2, 2), idesc_with_sf_ids(idesc, 3, 3)};
      // operand descriptors (see make_desc_kmajor_sw128 / make_desc_mnmajor_sw128): the high word - 1024-byte group
      // stride, version, 128-byte swizzle - is a constant; the low word is the start address in 16-byte units plus
      // the leading byte offset field, and moves by 32 bytes (K-major) or 4096 bytes (MN-major) per 32-wide K block
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);
      const uint32_t a_step = a_mn ? 256u : 2u, b_step = b_mn ? 256u : 2u;
      const uint32_t a_lo0 = ((smem_base & 0x3FFFF) >> 4) | ((a_mn ? (uint32_t)(S::A_BYTES >> 4) : 1u) << 16);
      const uint32_t b_lo0 = (((smem_base + S::A_BYTES) & 0x3FFFF) >> 4) | ((b_mn ? (uint32_t)(S::B_BYTES >> 4) : 1u) << 16);
      const uint32_t sf_lo0 = (sf_base & 0x3FFFF) >> 4;
      const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
      const bool skip_sf_cp = (p.debug_skip_store & 16) != 0;
      int stage = 0, as = 0, sfs = 0;
      uint32_t phase = 0, aphase = 0, sfphase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < n_total_u && ok; tile += n_pairs_grid) {
        const PairTile t = pair_tile<BN, MODE>(tile, 0, p, s_efo, s_pairs);
        const int nkt = __shfl_sync(0xffffffffu, t.nkt, 0);
        if (nkt == 0) continue;
        const int n0 = __shfl_sync(0xffffffffu, t.n0, 0);
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * as, aphase ^ 1));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        // BN = 192: an odd column tile starts 64 rows into its first 128-row scale tile
        const uint32_t sfb_shift = (BN == 192) ? (((n0 / BN) & 1) ? 2u : 0u) : 0u;
        for (int k = 0; k < nkt; ++k) {
          const int kg = k & (S::SF_GROUP - 1);
          if (kg == 0) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_sffull + 8 * sfs, sfphase));
            if (!ok) break;
          }
          ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase));
          if (!ok) break;
          const uint32_t a_lo = a_lo0 + stage * (S::STAGE_BYTES >> 4);
          const uint32_t b_lo = b_lo0 + stage * (S::STAGE_BYTES >> 4);
          const uint32_t sf_lo = sf_lo0 + ((sfs * S::SF_SLOT_BYTES + kg * 512) >> 4);
          const uint32_t sfa_t = tmem_base + S::SF_COL0 + stage * S::SF_COLS;
          const uint32_t sfb_t = sfa_t + 4;
          const bool sf_done = (kg == S::SF_GROUP - 1 || k == nkt - 1);      // last use of this scale slot
          if (elect_one()) {
            if (!skip_sf_cp) {
              tc_cp_sf_pair_lo(sfa_t, sf_lo, sf_hi);
#pragma unroll
              for (int j = 0; j < S::SFB_TILES; ++j)
                tc_cp_sf_pair_lo(sfb_t + 4 * j, sf_lo + ((S::SF_GROUP * 512 * (1 + j)) >> 4), sf_hi);
            }
#pragma unroll
            for (int kb = 0; kb < BK / 32; ++kb)
              mma_mxf8_pair_lo(d_tmem, a_lo + a_step * kb, b_lo + b_step * kb, desc_hi, idesc_kb[kb], sfa_t,
                               sfb_t + sfb_shift, (k | kb) != 0);
            tc_commit_pair(bar_empty + 8 * stage, 3);
            if (sf_done) tc_commit_pair(bar_sfempty + 8 * sfs, 3);
          }
          if (++stage == nst) { stage = 0; phase ^= 1; }
          if (sf_done) {
            if (++sfs == S::SF_SLOTS) { sfs = 0; sfphase ^= 1; }
          }
        }
        if (!ok) break;
        if (elect_one()) tc_commit_pair(bar_tfull + 8 * as, 3);
        if (++as == S::ACC_STAGES) { as = 0; aphase ^= 1; }
      }
      if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 202); }
    }
    __syncwarp();
  } else if (CPG && warp >= 2 + S::EPI_WARPS && warp < 2 + S::EPI_WARPS + S::GATHER_WARPS) {
    // ------------------------------------------------------------ A-row load warps (both CTAs)
    // Four warps bring this CTA's 128 rows of A, row r of the tile = row a_idx[m0 + r] of the un-gathered e4m3
    // activation, with 16-byte cp.async copies into the 128-byte-swizzled stage (chunk c of row r lands at chunk
    // c ^ (r & 7)).  A warp instruction covers four rows x 128 bytes = four full cache lines.  A thread never waits
    // for its copies: cp.async.mbarrier.arrive makes the stage's "landed" barrier count it once they are done, so
    // the warps run ahead as far as the ring has free stages.
    const int gw = warp - (2 + S::EPI_WARPS);           // rows [32 gw, 32 gw + 32) of the tile
    const int sub = lane >> 3, ch = lane & 7;
    const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
    const uint8_t* xq = reinterpret_cast<const uint8_t*>(p.a_src);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < n_total_u && ok; tile += n_pairs_grid) {
      const PairTile tl = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      const int nkt = __shfl_sync(0xffffffffu, tl.nkt, 0);
      if (nkt == 0) continue;
      const int valid = __shfl_sync(0xffffffffu, tl.valid, 0);
      const int m0 = __shfl_sync(0xffffffffu, tl.m0, 0);
      const uint8_t* src[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = gw * 32 + i * 4 + sub;
        const int64_t row = valid ? (int64_t)p.a_idx[m0 + r] : 0;
        src[i] = xq + row * p.K + ch * 16;
      }
      for (int kt = 0; kt < nkt; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1));
        if (!ok) break;
        const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES + gw * 32 * BK;
        if (valid) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = i * 4 + sub;                   // row within this warp's 32; (gw * 32 + rr) & 7 == rr & 7
            const uint32_t dst = a_dst + rr * BK + ((ch ^ (rr & 7)) << 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src[i] + (size_t)kt * BK)
                         : "memory");
          }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_landed + 8 * stage) : "memory");
        if (++stage == nst) { stage = 0; phase ^= 1; }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");      // nothing of this thread is in flight when the CTA exits
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 204); }
  } else if (CPG && warp == 2 + S::EPI_WARPS + S::GATHER_WARPS) {
    // ------------------------------------------------------------ forwarder (both CTAs): when this CTA's rows of a
    // stage have landed, make them visible to the async proxy (the MMA reads shared memory through it) and count
    // this CTA in on the leader's full barrier of that stage
    // Lane l serves ring stage l: the stages are forwarded independently of one another, so the wake-up, the proxy
    // fence and the remote arrival of one stage overlap those of the others (a single thread walking the stages in
    // order forwarded one K tile per ~0.8 us and throttled the whole kernel).
    const uint32_t full0 = map_to_cta(bar_full, 0);
    const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
    int total_kt = 0;                                     // K tiles this CTA pair will run
    for (int tile = pair_id; tile < n_total_u; tile += n_pairs_grid) {
      const PairTile tl = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      total_kt += __shfl_sync(0xffffffffu, tl.nkt, 0);
    }
    bool ok = true;
    if (lane < nst) {
      uint32_t ph = 0;
      for (int n = lane; n < total_kt; n += nst) {
        ok = mbar_wait(bar_landed + 8 * lane, ph);
        if (!ok) break;
        fence_proxy_async_smem();
        mbar_arrive_cluster_cta_release(full0 + 8 * lane);
        ph ^= 1;
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 205); }
  } else if (warp == S::SF_WARP) {
    // ------------------------------------------------------------ scale producer (both CTAs)
    if (lane == 0) { prefetch_tmap(&tmap_sfa); prefetch_tmap(&tmap_sfb); }
    const uint32_t sffull0 = map_to_cta(bar_sffull, 0);
    const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
    int sfs = 0;
    uint32_t sfphase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < n_total_u && ok; tile += n_pairs_grid) {
      const PairTile tl = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      const int nkt = __shfl_sync(0xffffffffu, tl.nkt, 0);
      if (nkt == 0) continue;
      const int kt0 = __shfl_sync(0xffffffffu, tl.kt0, 0);
      const int valid = __shfl_sync(0xffffffffu, tl.valid, 0);
      const int m0 = __shfl_sync(0xffffffffu, tl.m0, 0);
      const int n0 = __shfl_sync(0xffffffffu, tl.n0, 0);
      const int te = __shfl_sync(0xffffffffu, tl.e, 0);
      const int b_base = (MODE == WGRAD) ? n0 : te * p.N + n0;
      // rows of the scale tensors are 512-byte tiles: (row tile, k tile)
      const int sfa_tile = valid ? m0 / 128 : 0;         // phantom half: any in-range tile will do
      const int sfb_tile = b_base / 128;                 // first 128-row scale tile touching the BN window
      for (int kt = kt0; kt < kt0 + nkt; kt += S::SF_GROUP) {
        // scales of the next SF_GROUP K tiles: rows [tile*ktiles + kt, +SF_GROUP) of the 512-byte-row scale
        // tensors (rows past this operand tile's K range are fetched too and never used)
        ok = __all_sync(0xffffffffu, mbar_wait(bar_sfempty + 8 * sfs, sfphase ^ 1));
        if (!ok) break;
        if (elect_one()) {
          const uint32_t sffull = sffull0 + 8 * sfs;
          const uint32_t dst = sf_base + sfs * S::SF_SLOT_BYTES;
          if (rank == 0) mbar_expect_tx(bar_sffull + 8 * sfs, S::SF_TX_BYTES);
          tma_load_2d_pair(dst, &tmap_sfa, sffull, 0, sfa_tile * p.sfa_ktiles + kt);
#pragma unroll
          for (int j = 0; j < S::SFB_TILES; ++j)
            tma_load_2d_pair(dst + S::SF_GROUP * 512 * (1 + j), &tmap_sfb, sffull, 0,
                             (sfb_tile + j) * p.sfb_ktiles + kt);
        }
        if (++sfs == S::SF_SLOTS) { sfs = 0; sfphase ^= 1; }
      }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 206); }
  } else {
    // ------------------------------------------------------------ epilogue (8 or 12 warps per CTA)
    const int q = warp & 3;                       // TMEM lane quadrant of this warp
    const int half = (warp - 2) >> 2;             // which group of the tile's columns
    const int row_in_tile = q * 32 + lane;
    constexpr int COLS_PER_WARP = BN / S::COL_GROUPS;
    const uint32_t stg = smem_u32(epi + (warp - 2) * S::EPI_BYTES_PER_WARP);
    const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int tile = pair_id; tile < n_total && ok; tile += n_pairs_grid) {
      const PairTile t = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      const size_t grow = (size_t)t.m0 + row_in_tile;
      const int c_base = t.n0 + half * COLS_PER_WARP;
      if (t.nkt == 0) {
        if (MODE == WGRAD && !p.accumulate) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) +
                                                  ((size_t)t.e * p.rows + grow) * p.N + c_base);
          for (int i = 0; i < COLS_PER_WARP / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        continue;
      }
      // DGATEDQ: the first chunk of z and the row's score are fetched before the wait for the accumulator,
      // so their latency hides behind this tile's main loop
      uint4 zb[4];
      uint32_t sc = 0;
      float s_row = 0.f;
      if (MODE == DGATEDQ && t.valid && c_base < p.N) {
        const int Nz = 2 * p.N;
        const uint8_t* zrow = p.z_fp8 + grow * Nz + 2 * c_base;
#pragma unroll
        for (int i = 0; i < 4; ++i) zb[i] = reinterpret_cast<const uint4*>(zrow)[i];
        sc = *reinterpret_cast<const uint16_t*>(p.z_sc + grow * (Nz / 32) + (2 * c_base) / 32);
        s_row = p.s[grow];
      }
      if (lane == 0) ok = mbar_wait(bar_tfull + 8 * as, aphase);
      ok = __shfl_sync(0xffffffff, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN + half * COLS_PER_WARP;

      bool released = false;
      if (p.debug_skip_store & 8) {
        // timing experiment: the accumulator is handed back untouched
      } else if (MODE == PLAIN) {
        // Drain the whole row segment into registers (bf16-packed), hand the accumulator back to the
        // MMA warp, then stage and store.  32 columns of bf16 = 64-byte rows, SWIZZLE_64B, 2 x 2 KB.
        constexpr int NC = COLS_PER_WARP / 32;
        uint32_t pk[NC][16];
#pragma unroll
        for (int c = 0; c < NC; c += 2) {      // two TMEM loads in flight per wait: the drain is what the MMA waits for
          uint32_t r0[32], r1[32];
          tmem_ld32(t_row + c * 32, r0);
          if (c + 1 < NC) tmem_ld32(t_row + (c + 1) * 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            pk[c][i] = pack_bf16x2(__uint_as_float(r0[2 * i]), __uint_as_float(r0[2 * i + 1]));
          if (c + 1 < NC) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pk[c + 1][i] = pack_bf16x2(__uint_as_float(r1[2 * i]), __uint_as_float(r1[2 * i + 1]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * as);
        released = true;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const uint32_t sb = stg;                 // one 2 KB staging buffer per warp
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
          if (t.valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              st_shared_v4(sb + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), pk[c][4 * j], pk[c][4 * j + 1],
                           pk[c][4 * j + 2], pk[c][4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, sb, c_base + c * 32, t.m0 + q * 32);
              bulk_commit_group();
            }
          }
        }
      } else if (MODE == WGRAD) {
        // Same scheme with f32 in 16-column pieces: 64-byte rows, SWIZZLE_64B, one 2 KB buffer; TMA reduce-add
        // when accumulating into an existing gradient.
        constexpr int NC = COLS_PER_WARP / 32;
        uint32_t acc[NC][32];
#pragma unroll
        for (int c = 0; c < NC; ++c) tmem_ld32(t_row + c * 32, acc[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * as);
        released = true;
#pragma unroll
        for (int c = 0; c < 2 * NC; ++c) {
          const uint32_t sb = stg;
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            st_shared_v4(sb + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), acc[c >> 1][(c & 1) * 16 + 4 * j],
                         acc[c >> 1][(c & 1) * 16 + 4 * j + 1], acc[c >> 1][(c & 1) * 16 + 4 * j + 2],
                         acc[c >> 1][(c & 1) * 16 + 4 * j + 3]);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int crow = t.e * p.rows + t.m0 + q * 32;
            if (p.accumulate) tma_reduce_add_2d(&tmap_c, sb, c_base + c * 16, crow);
            else tma_store_2d(&tmap_c, sb, c_base + c * 16, crow);
            bulk_commit_group();
          }
        }
      } else if (MODE == GATED) {
        // 64-column chunks of z (= 32 columns of y1 = one y1 scale group), dealt to the column groups in order;
        // BN = 192 with two groups: the first takes chunks 0 and 1, the second chunk 2.
        // BN = 256 has a single accumulator stage: the warp first drains its 128 columns into registers and
        // hands the accumulator back, so the next tile's MMAs run under the arithmetic below.
        constexpr int CHUNKS = BN / 64, PER = (CHUNKS + S::COL_GROUPS - 1) / S::COL_GROUPS;
        constexpr bool DRAIN = (S::ACC_STAGES == 1);
        const int Nz = p.N, Ny = p.N / 2;
        const int ch0 = half * PER;
        const int nch = min(PER, CHUNKS - ch0);
        const uint32_t t_tile = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;
        uint32_t acc[DRAIN ? PER * 2 * 32 : 32];
        if (DRAIN) {
          static_assert(!DRAIN || PER * 2 * 32 == 128, "the single-accumulator tile is 256 wide: 128 columns per warp");
          if constexpr (!CPG) {
            tmem_ld128(t_tile + ch0 * 64, reinterpret_cast<uint32_t(&)[128]>(acc));
          } else {      // sixteen warps per CTA leave 128 registers a thread: no room for one 128-register load
#pragma unroll
            for (int c = 0; c < PER * 2; ++c)
              tmem_ld32(t_tile + ch0 * 64 + c * 32, reinterpret_cast<uint32_t(&)[32]>(acc[DRAIN ? c * 32 : 0]));
          }
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * as);
          released = true;
        }
#pragma unroll
        for (int ci = 0; ci < PER; ++ci) {
          if (ci >= nch) break;
          const int zc = t.n0 + (ch0 + ci) * 64;           // first z column of the chunk
          float y[32];
          uint32_t zs = 0;
          // staging: z 32 rows x 64 B (64B swizzle) at stg, y1 32 rows x 32 B (32B swizzle) at stg + 2048
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t rl[32];
            if (!DRAIN) {
              tmem_ld32(t_tile + (ch0 + ci) * 64 + h * 32, rl);
              tmem_ld_wait();
            }
            const uint32_t* r = DRAIN ? &acc[DRAIN ? (ci * 2 + h) * 32 : 0] : rl;
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(__uint_as_float(r[i])));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
              y[h * 16 + i] = bf16_rne((g * fast_sigmoid(g)) * u);
            }
            const int e = e8m0_of(fmaxf(amax, 1e-4f));
            const float qs = qscale_of(e);
            zs |= (uint32_t)e << (8 * h);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const uint32_t v0 = pack_e4m3x4(__uint_as_float(r[16 * i + 0]) * qs, __uint_as_float(r[16 * i + 1]) * qs,
                                              __uint_as_float(r[16 * i + 2]) * qs, __uint_as_float(r[16 * i + 3]) * qs);
              const uint32_t v1 = pack_e4m3x4(__uint_as_float(r[16 * i + 4]) * qs, __uint_as_float(r[16 * i + 5]) * qs,
                                              __uint_as_float(r[16 * i + 6]) * qs, __uint_as_float(r[16 * i + 7]) * qs);
              const uint32_t v2 = pack_e4m3x4(__uint_as_float(r[16 * i + 8]) * qs, __uint_as_float(r[16 * i + 9]) * qs,
                                              __uint_as_float(r[16 * i + 10]) * qs, __uint_as_float(r[16 * i + 11]) * qs);
              const uint32_t v3 = pack_e4m3x4(__uint_as_float(r[16 * i + 12]) * qs, __uint_as_float(r[16 * i + 13]) * qs,
                                              __uint_as_float(r[16 * i + 14]) * qs, __uint_as_float(r[16 * i + 15]) * qs);
              st_shared_v4(stg + lane * 64 + (((2 * h + i) ^ ((lane >> 1) & 3)) << 4), v0, v1, v2, v3);
            }
          }
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(y[i]));
          const int e = e8m0_of(amax);
          const float qs = qscale_of(e);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const uint32_t v0 = pack_e4m3x4(y[16 * i + 0] * qs, y[16 * i + 1] * qs, y[16 * i + 2] * qs, y[16 * i + 3] * qs);
            const uint32_t v1 = pack_e4m3x4(y[16 * i + 4] * qs, y[16 * i + 5] * qs, y[16 * i + 6] * qs, y[16 * i + 7] * qs);
            const uint32_t v2 = pack_e4m3x4(y[16 * i + 8] * qs, y[16 * i + 9] * qs, y[16 * i + 10] * qs, y[16 * i + 11] * qs);
            const uint32_t v3 = pack_e4m3x4(y[16 * i + 12] * qs, y[16 * i + 13] * qs, y[16 * i + 14] * qs, y[16 * i + 15] * qs);
            st_shared_v4(stg + 2048 + lane * 32 + ((i ^ ((lane >> 2) & 1)) << 4), v0, v1, v2, v3);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (t.valid && !(p.debug_skip_store & 1)) {
            if (lane == 0) {
              tma_store_2d(&tmap_c, stg, zc, t.m0 + q * 32);                 // z e4m3 [rows, 2I]
              tma_store_2d(&tmap_c2, stg + 2048, zc / 2, t.m0 + q * 32);     // y1 e4m3 [rows, I]
              bulk_commit_group();
            }
            *reinterpret_cast<uint16_t*>(p.z_sc + grow * (Nz / 32) + zc / 32) = (uint16_t)zs;
            const int g = zc / 64;
            p.y1_sf[((grow / 128) * (size_t)(Ny / 128) + g / 4) * 512 + (grow % 32) * 16 + ((grow % 128) / 32) * 4 +
                    (g % 4)] = (uint8_t)e;
          }
        }
      } else if (MODE == DGATEDQ) {
        // D columns [c_base, c_base + BN/2) in chunks of 32.  Per chunk dz (64 columns) and y1s (32 columns)
        // are rounded to bf16 and quantised right here - dz with one scale per 32x32 block, y1s with one scale
        // per column and 32 rows - and leave as e4m3 in row-major order.  A 32x32-block scale serves dz both as
        // the activation-gradient operand (scales along 2I) and as the weight-gradient operand (scales along
        // TKp, fed MN-major), so one copy of the payload is enough.  Each warp works on its own.
        // a ragged last column tile (N not a multiple of BN): chunks at or beyond column N hold products with
        // rows of the next expert's weights (or TMA zero fill) and are skipped whole (N is a multiple of 32)
        if (t.valid && c_base < p.N && !(p.debug_skip_store & 2)) {
          const int Nz = 2 * p.N;
          const float s = s_row;
          const int row_grp = (t.m0 + q * 32) >> 5;      // 32-row group index along TKp
          const int kt_rows = p.rows >> 7;               // K tiles of the weight-gradient operands
          constexpr int NCH = COLS_PER_WARP / 32;
          float ds_acc = 0.f;
#pragma unroll 1
          for (int c = 0; c < NCH; ++c) {
            const int dcol = c_base + c * 32;            // first D / y1s column of the chunk
            if (dcol >= p.N) break;
            uint32_t r0[16], r1[16];                     // the accumulator arrives in two 16-column halves
            tmem_ld16(t_row + c * 32, r0);
            tmem_ld16(t_row + c * 32 + 16, r1);
            uint4 zn[4];
            uint32_t scn = 0;
            if (c + 1 < NCH && dcol + 32 < p.N) {        // next chunk's z travels while this one is computed
              const uint8_t* zrow = p.z_fp8 + grow * Nz + 2 * (dcol + 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) zn[i] = reinterpret_cast<const uint4*>(zrow)[i];
              scn = *reinterpret_cast<const uint16_t*>(p.z_sc + grow * (Nz / 32) + (2 * (dcol + 32)) / 32);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) zn[i] = make_uint4(0, 0, 0, 0);
            }
            const float sc0 = __int_as_float((int)(sc & 0xFF) << 23);
            const float sc1 = __int_as_float((int)(sc >> 8) << 23);
            tmem_ld_wait();
            if (lane == 0) bulk_wait_group_read<0>();    // the previous chunk's stores have read the staging
            __syncwarp();
            const uint32_t* zw = reinterpret_cast<const uint32_t*>(zb);
            uint32_t Y[16];                              // y1s of this lane's row, bf16 pairs of adjacent columns
            uint32_t e_blk = 0;
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              // 16 D columns -> 32 dz columns = one 32x32 scale block; dz stays packed in bf16 pairs until its
              // block maximum is known
              uint32_t P[16];
              float amax = 0.f;
              const float scale = b ? sc1 : sc0;
#pragma unroll
              for (int i2 = 0; i2 < 8; ++i2) {
                float yq[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int pi = b * 16 + 2 * i2 + h;
                  const uint32_t pair = (zw[pi >> 1] >> (16 * (pi & 1))) & 0xFFFF;
                  const float2 gu = e4m3x2_to_f32(pair);
                  const float g = gu.x * scale, u = gu.y * scale;
                  const float D = __uint_as_float(b ? r1[2 * i2 + h] : r0[2 * i2 + h]);
                  const float dout = s * D;
                  const float sig = fast_sigmoid(g);
                  const float silu = g * sig;
                  const float sd = silu * dout;
                  const float yv = silu * u;
                  ds_acc = fmaf(yv, D, ds_acc);
                  const uint32_t dzp = pack_bf16x2(((sig - silu * sig) * dout + sd) * u, sd);   // rounds to bf16
                  P[2 * i2 + h] = dzp;
                  yq[h] = s * yv;
                  amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(dzp << 16)), fabsf(__uint_as_float(dzp & 0xFFFF0000u))));
                }
                Y[b * 8 + i2] = pack_bf16x2(yq[0], yq[1]);
              }
              uint32_t w[8];
              const int e = e8m0_of(warp_max_abs(amax));
              const float qs = qscale_of(e);
              e_blk |= (uint32_t)e << (8 * b);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                w[i] = pack_e4m3x4(__uint_as_float(P[2 * i] << 16) * qs, __uint_as_float(P[2 * i] & 0xFFFF0000u) * qs,
                                   __uint_as_float(P[2 * i + 1] << 16) * qs,
                                   __uint_as_float(P[2 * i + 1] & 0xFFFF0000u) * qs);
              // this half's 32 dz bytes of the row go to the staging tile right away
#pragma unroll
              for (int j = 0; j < 2; ++j)
                st_shared_v4(stg + lane * 64 + (((2 * b + j) ^ ((lane >> 1) & 3)) << 4), w[4 * j], w[4 * j + 1],
                             w[4 * j + 2], w[4 * j + 3]);
            }
            // y1s: one scale per column over the warp's 32 rows.  Column maxima by a butterfly on bf16 pairs that
            // halves the column set at each step: lane L ends with the pair holding column L.
            uint32_t wy[8];
            uint32_t A[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) A[i] = Y[i] & 0x7FFF7FFFu;
#pragma unroll
            for (int sft = 16; sft >= 2; sft >>= 1) {
              const bool up = (lane & sft) != 0;
#pragma unroll
              for (int i = 0; i < sft / 2; ++i) {
                const uint32_t send = up ? A[i] : A[i + sft / 2];
                const uint32_t keep = up ? A[i + sft / 2] : A[i];
                A[i] = max_bf16x2(keep, __shfl_xor_sync(0xffffffff, send, sft));
              }
            }
            A[0] = max_bf16x2(A[0], __shfl_xor_sync(0xffffffff, A[0], 1));
            const int e_mine = e8m0_of(__uint_as_float((lane & 1) ? (A[0] & 0xFFFF0000u) : (A[0] << 16)));
            const float qs_mine = qscale_of(e_mine);
#pragma unroll
            for (int i4 = 0; i4 < 8; ++i4) {
              float qv[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int cc = 4 * i4 + j;
                const float yv = __uint_as_float((cc & 1) ? (Y[cc >> 1] & 0xFFFF0000u) : (Y[cc >> 1] << 16));
                qv[j] = yv * __shfl_sync(0xffffffff, qs_mine, cc);
              }
              wy[i4] = pack_e4m3x4(qv[0], qv[1], qv[2], qv[3]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
              st_shared_v4(stg + 2048 + lane * 32 + ((j ^ ((lane >> 2) & 1)) << 4), wy[4 * j], wy[4 * j + 1],
                           wy[4 * j + 2], wy[4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (p.debug_skip_store & 1) continue;
            if (lane == 0) {
              tma_store_2d(&tmap_c, stg, 2 * dcol, t.m0 + q * 32);          // dz e4m3 [TKp, 2I]
              tma_store_2d(&tmap_c2, stg + 2048, dcol, t.m0 + q * 32);      // y1s e4m3 [TKp, I]
              bulk_commit_group();
            }
            // scales: dz as a (TKp, 2I) operand - this row, two adjacent 32-column groups
            const int g_row = (2 * dcol) >> 5;
            *reinterpret_cast<uint16_t*>(p.dz_row_sf + ((grow >> 7) * (size_t)(Nz >> 7) + (g_row >> 2)) * 512 +
                                         (grow & 31) * 16 + ((grow & 127) >> 5) * 4 + (g_row & 3)) = (uint16_t)e_blk;
            // dz as a (2I, TKp) operand - lane = column, this warp's 32-row group
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              const size_t zc = (size_t)(2 * dcol + 32 * b + lane);
              p.dz_col_sf[((zc >> 7) * (size_t)kt_rows + (row_grp >> 2)) * 512 + (zc & 31) * 16 +
                          ((zc & 127) >> 5) * 4 + (row_grp & 3)] = (uint8_t)(e_blk >> (8 * b));
            }
            const size_t yc = (size_t)(dcol + lane);
            p.y1s_col_sf[((yc >> 7) * (size_t)kt_rows + (row_grp >> 2)) * 512 + (yc & 31) * 16 +
                         ((yc & 127) >> 5) * 4 + (row_grp & 3)] = (uint8_t)e_mine;
#pragma unroll
            for (int i = 0; i < 4; ++i) zb[i] = zn[i];
            sc = scn;
          }
          p.ds_partial[(size_t)((t.n0 / BN) * S::COL_GROUPS + half) * p.rows + grow] = ds_acc;
        }
      } else {  // DGATED
        // this warp: D columns [c_base, c_base + BN/2) of I in chunks of 32 -> dz 64 bf16 (128-byte rows,
        // SWIZZLE_128B, 4 KB) and y1s 32 bf16 (64-byte rows, SWIZZLE_64B, 2 KB)
        const int Nz = 2 * p.N;
        const float s = t.valid ? p.s[grow] : 0.f;
        float ds_acc = 0.f;
#pragma unroll 1
        for (int c = 0; c < COLS_PER_WARP / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          uint4 zb[4];
          float sc0 = 0.f, sc1 = 0.f;
          if (t.valid) {
            const uint8_t* zrow = p.z_fp8 + grow * Nz + 2 * (c_base + c * 32);
            const uint8_t* zsc = p.z_sc + grow * (Nz / 32) + (2 * (c_base + c * 32)) / 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) zb[i] = reinterpret_cast<const uint4*>(zrow)[i];
            const uint32_t sc = *reinterpret_cast<const uint16_t*>(zsc);
            sc0 = __int_as_float((int)(sc & 0xFF) << 23);
            sc1 = __int_as_float((int)(sc >> 8) << 23);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) zb[i] = make_uint4(0, 0, 0, 0);
          }
          tmem_ld_wait();
          const uint32_t* zw = reinterpret_cast<const uint32_t*>(zb);
          uint32_t dzp[32];
          uint32_t ysp[16];
          float yprev = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t pair = (zw[i >> 1] >> (16 * (i & 1))) & 0xFFFF;
            const float scale = (i < 16) ? sc0 : sc1;
            const float2 gu = e4m3x2_to_f32(pair);
            const float g = gu.x * scale, u = gu.y * scale;
            const float D = __uint_as_float(r[i]);
            const float dout = s * D;
            const float sig = fast_sigmoid(g);
            const float silu = g * sig;
            const float sd = silu * dout;
            const float dg = ((sig - silu * sig) * dout + sd) * u;
            const float yv = silu * u;
            ds_acc = fmaf(yv, D, ds_acc);
            dzp[i] = pack_bf16x2(dg, sd);
            const float ys = s * yv;
            if (i & 1) ysp[i >> 1] = pack_bf16x2(yprev, ys); else yprev = ys;
          }
          if (lane == 0) bulk_wait_group_read<0>();
          __syncwarp();
          if (t.valid) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_shared_v4(stg + lane * 128 + ((j ^ (lane & 7)) << 4), dzp[4 * j], dzp[4 * j + 1], dzp[4 * j + 2],
                           dzp[4 * j + 3]);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              st_shared_v4(stg + 4096 + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), ysp[4 * j], ysp[4 * j + 1],
                           ysp[4 * j + 2], ysp[4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_2d(&tmap_c, stg, 2 * (c_base + c * 32), t.m0 + q * 32);
              tma_store_2d(&tmap_c2, stg + 4096, c_base + c * 32, t.m0 + q * 32);
              bulk_commit_group();
            }
          }
        }
        if (t.valid) p.ds_partial[(size_t)((t.n0 / BN) * 2 + half) * p.rows + grow] = ds_acc;
      }

      if (!released) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * as);
      }
      if (++as == S::ACC_STAGES) { as = 0; aphase ^= 1; }
    }
    if (lane == 0) bulk_wait_group<0>();      // all staged stores have left shared memory and are visible
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 203); }
  }

  // common exit: everyone arrives here, also after a failed wait
  __syncthreads();
  if (*s_abort) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();                         // the peer may still be signalling this CTA's barriers
  tc_fence_after();
  if (warp == 1) tmem_dealloc2(tmem_base, 512);
}

}  // namespace smoe
