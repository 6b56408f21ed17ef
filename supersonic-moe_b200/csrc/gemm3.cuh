// Two-CTA MXFP8 grouped GEMM with a 256 x 384 tile held as TWO accumulators of 256 x 192 (TMEM columns 0..191 and
// 192..383) that share every A tile.
//
// Why: per 128-wide K tile a CTA of this kernel loads A (16 KB) once for two B halves (2 x 12 KB): 40 KB for 768
// tensor clocks instead of 32 KB for 512 - 17 % fewer operand bytes per MMA than the 256 x 256 tile - with no
// multicast load anywhere (each CTA fetches its own rows of A and of both B halves with plain tiled TMA copies).
// When it was written that bought 7-9 % on the plain and weight-gradient GEMMs; since the accumulator hand-back no
// longer stalls (relaxed arrival, see the epilogue) the 256 x 256 kernel runs the activation-gradient GEMM in the
// same time; this kernel stays the default where N % 384 == 0 and is the one that runs the two weight gradients
// of a layer in a single launch.
//
// The two accumulators also hide the accumulator hand-over between tiles: the last J K tiles of a tile are issued
// half 0 first, so the epilogue drains accumulator 0 under the half-1 MMAs of those K tiles, and the next tile
// starts with J K tiles of half 0 while accumulator 1 is still being drained.
//
// Modes: PLAIN (bf16 C through TMA stores) and WGRAD (f32 C through TMA store / reduce-add; A may be MN-major, B is
// K-major).  N must be a multiple of 384.
#pragma once
#include "gemm2.cuh"

namespace smoe {

constexpr int kBN3 = 384;          // tile width
constexpr int kHN3 = 192;          // width of one accumulator
constexpr int kHeadTail3 = 2;      // K tiles issued half-by-half at both ends of a tile

template <int MODE>
struct Gemm3Smem {
  static constexpr int A_BYTES = BM * BK;                       // this CTA's 128 rows of A
  static constexpr int BH_BYTES = (kHN3 / 2) * BK;              // this CTA's 96 rows of one B half
  static constexpr int STAGE_BYTES = A_BYTES + 2 * BH_BYTES;    // 40 KB
  static constexpr int SFB_TILES = 3;                           // 128-row scale tiles covering the 384 B rows
  static constexpr int SF_GROUP = kSfGroup2;
  static constexpr int SF_SLOT_BYTES = SF_GROUP * 512 * (1 + SFB_TILES);
  static constexpr int SF_SLOTS = 2;
  static constexpr int SF_BYTES = SF_SLOTS * SF_SLOT_BYTES;
  static constexpr int EPI_WARPS = 8;                           // four TMEM lane quadrants x two column groups
  static constexpr int LEAD_WARPS = 3;                          // operand producer, MMA issuer, scale producer
  static constexpr int THREADS = 32 * (LEAD_WARPS + EPI_WARPS);
  static constexpr int EPI_BUFS = 2;                            // staging buffers per warp, used in turn
  static constexpr int EPI_BYTES_PER_WARP = EPI_BUFS * 2048;    // bf16 32x32 or f32 32x16 per buffer
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BYTES_PER_WARP;
  static constexpr int AUX_BYTES = 512 + 2 * (kMaxExperts2 + 1) * 4 + 8;
  static constexpr int STAGES = 4;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + SF_BYTES + EPI_BYTES + AUX_BYTES + 1024;
  static_assert(TOTAL <= 227 * 1024, "shared memory budget");
  static constexpr int SF_COLS = 4 + 4 * SFB_TILES;             // TMEM columns of one stage's scales
  static constexpr int SF_COL0 = kBN3;
  static_assert(SF_COL0 + STAGES * SF_COLS <= 512, "TMEM budget");
  static constexpr uint32_t TX_BYTES = 2u * STAGE_BYTES;        // both CTAs' A and B per stage
  static constexpr uint32_t SF_TX_BYTES = 2u * SF_SLOT_BYTES;
};

// Tensor maps of a second weight-gradient product that shares the launch (GemmParams::rows2 > 0): two products
// whose tile counts are no multiples of the number of CTA pairs leave one partly filled last wave together instead
// of one each.
struct SecondMaps {
  CUtensorMap a, b, sfa, sfb, c;
};

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((Gemm3Smem<MODE>::THREADS), 1)
gemm3_mxf8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                  const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ SecondMaps second,
                  const GemmParams p) {
  static_assert(MODE == PLAIN || MODE == WGRAD, "the 384-wide tile exists for the plain and weight-gradient GEMMs");
  using S = Gemm3Smem<MODE>;
  constexpr int BN = kBN3, HN = kHN3;
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
  const uint32_t bar_tfull = bar_empty + 8 * S::STAGES;    // one per accumulator half
  const uint32_t bar_tempty = bar_tfull + 8 * 2;
  const uint32_t bar_sffull = bar_tempty + 8 * 2;
  const uint32_t bar_sfempty = bar_sffull + 8 * S::SF_SLOTS;

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
      mbar_init(bar_full + 8 * s, 1);        // leader's: its own producer arms it; both CTAs' copies credit it
      mbar_init(bar_empty + 8 * s, 1);       // one commit arrival per use, in each CTA
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);                   // commit arrival, in each CTA
      mbar_init(bar_tempty + 8 * s, 2 * S::EPI_WARPS);     // leader's: the epilogue warps of both CTAs
    }
    for (int s = 0; s < S::SF_SLOTS; ++s) {
      mbar_init(bar_sffull + 8 * s, 1);
      mbar_init(bar_sfempty + 8 * s, 1);
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
  const int n_col_tiles = p.N / BN;
  const int n_total = (MODE == WGRAD) ? p.E * ((p.rows + p.rows2) / (2 * BM)) * n_col_tiles
                                      : s_pairs[p.E] * n_col_tiles;
  const bool a_mn = MODE == WGRAD && p.a_mn;
  const int nst = S::STAGES - p.dbg_stage_cut;      // timing experiment: a shallower ring (0 in product use)

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs): warp-uniform loops, one
    // elected lane issues
    if (lane == 0) {
      prefetch_tmap(&tmap_a); prefetch_tmap(&tmap_b);
      if (MODE == WGRAD && p.rows2 > 0) { prefetch_tmap(&second.a); prefetch_tmap(&second.b); }
    }
    const uint32_t full0 = map_to_cta(bar_full, 0);
    const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
    const bool dbg_noload = (p.debug_skip_store & 4) != 0;   // timing experiment: operands fetched for one ring pass only
    int dbg_filled = 0;
    int stage = 0;
    uint32_t phase = 0;
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
      const int b_row = b_base + rank * (HN / 2);        // this CTA's 96 rows of half 0; half 1 lies HN rows further
      const int a_row = valid ? m0 : 0;
      const bool second_prob = MODE == WGRAD && __shfl_sync(0xffffffffu, tl.prob, 0) != 0;
      const CUtensorMap* ta = second_prob ? &second.a : &tmap_a;
      const CUtensorMap* tb = second_prob ? &second.b : &tmap_b;
      for (int kt = kt0; kt < kt0 + nkt; ++kt) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1));
        if (!ok) break;
        const uint32_t full = full0 + 8 * stage;
        const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
        const uint32_t b_dst = a_dst + S::A_BYTES;
        if (dbg_noload && dbg_filled >= nst) {
          if (rank == 0 && elect_one()) mbar_arrive(bar_full + 8 * stage);
        } else {
          ++dbg_filled;
          if (elect_one()) {
            if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, S::TX_BYTES);
            if (a_mn) tma_load_2d_pair(a_dst, ta, full, m0, kt * BK);
            else tma_load_2d_pair(a_dst, ta, full, kt * BK, a_row);
            tma_load_2d_pair(b_dst, tb, full, kt * BK, b_row);
            tma_load_2d_pair(b_dst + S::BH_BYTES, tb, full, kt * BK, b_row + HN);
          }
        }
        if (++stage == nst) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 201); }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only): warp-uniform loops,
    // one elected lane issues
    if (rank == 0) {
      const uint32_t idesc = make_idesc_mxf8(2 * BM, HN) | (a_mn ? 1u << 15 : 0u);
      const uint32_t idesc_kb[4] = {idesc_with_sf_ids(idesc, 0, 0), idesc_with_sf_ids(idesc, 1, 1),
                                    idesc_with_sf_ids(idesc, 2, 2), idesc_with_sf_ids(idesc, 3, 3)};
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t sf_hi = (128u >> 4) | (1u << 14);
      const uint32_t a_step = a_mn ? 256u : 2u;
      const uint32_t a_lo0 = ((smem_base & 0x3FFFF) >> 4) | ((a_mn ? (uint32_t)(S::A_BYTES >> 4) : 1u) << 16);
      const uint32_t b_lo0 = (((smem_base + S::A_BYTES) & 0x3FFFF) >> 4) | (1u << 16);
      const uint32_t sf_lo0 = (sf_base & 0x3FFFF) >> 4;
      const int n_total_u = __shfl_sync(0xffffffffu, n_total, 0);
      int stage = 0, sfs = 0;
      uint32_t phase = 0, aphase = 0, sfphase = 0;
      bool ok = true;
      // K tiles issued half-by-half at both ends of a tile (a timing experiment may shorten it)
      const int JJ = (p.l2_prefetch >= 0 && p.l2_prefetch < kHeadTail3) ? p.l2_prefetch : kHeadTail3;

      // MMAs of K tile number k (of its tile) held in ring stage st, into accumulator half h
      auto issue_half = [&](int st, int k, int h) {
        const uint32_t a_lo = a_lo0 + st * (S::STAGE_BYTES >> 4);
        const uint32_t b_lo = b_lo0 + st * (S::STAGE_BYTES >> 4) + h * (S::BH_BYTES >> 4);
        const uint32_t sfa_t = tmem_base + S::SF_COL0 + st * S::SF_COLS;
        const uint32_t sfb_t = sfa_t + 4 + 6 * h;              // 192 B rows = six 32-row scale columns per half
#pragma unroll
        for (int kb = 0; kb < BK / 32; ++kb)
          mma_mxf8_pair_lo(tmem_base + h * HN, a_lo + a_step * kb, b_lo + 2u * kb, desc_hi, idesc_kb[kb], sfa_t, sfb_t,
                           (k | kb) != 0);
      };

      long long* trace = (pair_id == 0) ? p.trace : nullptr;      // timing experiment, null in product use
      int trace_n = 0;
      for (int tile = pair_id; tile < n_total_u && ok; tile += n_pairs_grid) {
        const PairTile t = pair_tile<BN, MODE>(tile, 0, p, s_efo, s_pairs);
        const int nkt = __shfl_sync(0xffffffffu, t.nkt, 0);
        if (nkt == 0) continue;
        const long long tr0 = trace ? clock64() : 0;
        long long tr_full = 0, tr_sf = 0, tr_acc1 = 0, tr_first = 0;
        const int J = nkt >= 2 * JJ ? JJ : 0;
        int held0 = 0, held1 = 0;             // ring stages of the K tiles whose half-1 MMAs are still to come
        static_assert(kHeadTail3 == 2, "held0 / held1");
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty, aphase ^ 1));
        if (!ok) break;
        if (J == 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8, aphase ^ 1));
          if (!ok) break;
        }
        tc_fence_after();
        const long long tr1 = trace ? clock64() : 0;
        for (int k = 0; k < nkt; ++k) {
          // first touch of K tile k: its operands and scales have landed; scales go to TMEM; half 0 always,
          // half 1 too unless the K tile belongs to the head or the tail of the tile
          const int kg = k & (S::SF_GROUP - 1);
          if (kg == 0) {
            const long long c0 = trace ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_sffull + 8 * sfs, sfphase));
            if (!ok) break;
            if (trace) tr_sf += clock64() - c0;
          }
          const long long c1 = trace ? clock64() : 0;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase));
          if (!ok) break;
          if (trace) {
            const long long d = clock64() - c1;
            tr_full += d;
            if (k == 0) tr_first = d;
          }
          const bool both = (k >= J && k < nkt - J);
          const bool sf_done = (kg == S::SF_GROUP - 1 || k == nkt - 1);
          const uint32_t sf_lo = sf_lo0 + ((sfs * S::SF_SLOT_BYTES + kg * 512) >> 4);
          const uint32_t sfa_t = tmem_base + S::SF_COL0 + stage * S::SF_COLS;
          if (elect_one()) {
            if (!(p.debug_skip_store & 16)) {
              tc_cp_sf_pair_lo(sfa_t, sf_lo, sf_hi);
#pragma unroll
              for (int j = 0; j < S::SFB_TILES; ++j)
                tc_cp_sf_pair_lo(sfa_t + 4 + 4 * j, sf_lo + ((S::SF_GROUP * 512 * (1 + j)) >> 4), sf_hi);
            }
            if (sf_done) tc_commit_pair(bar_sfempty + 8 * sfs, 3);   // the copies above were the slot's last readers
            issue_half(stage, k, 0);
            if (both) {
              issue_half(stage, k, 1);
              tc_commit_pair(bar_empty + 8 * stage, 3);
            }
          }
          if (!both) {
            if ((k < J ? k : k - (nkt - J)) == 0) held0 = stage; else held1 = stage;
          }
          if (++stage == nst) { stage = 0; phase ^= 1; }
          if (sf_done) {
            if (++sfs == S::SF_SLOTS) { sfs = 0; sfphase ^= 1; }
          }
          // end of the head / of the tail: the half-1 MMAs of the K tiles held back
          const bool head_end = (J > 0 && k == J - 1), tail_end = (J > 0 && k == nkt - 1);
          if (head_end) {
            const long long c2 = trace ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8, aphase ^ 1));
            if (!ok) break;
            tc_fence_after();
            if (trace) tr_acc1 = clock64() - c2;
          }
          if (head_end || tail_end) {
            if (elect_one()) {
              if (tail_end) tc_commit_pair(bar_tfull, 3);          // accumulator 0 is complete
              const int kfirst = head_end ? 0 : nkt - J;
              issue_half(held0, kfirst, 1);
              tc_commit_pair(bar_empty + 8 * held0, 3);
              if (J == 2) {
                issue_half(held1, kfirst + 1, 1);
                tc_commit_pair(bar_empty + 8 * held1, 3);
              }
            }
          }
        }
        if (!ok) break;
        if (elect_one()) {
          if (J == 0) tc_commit_pair(bar_tfull, 3);
          tc_commit_pair(bar_tfull + 8, 3);
        }
        if (trace) {
          // how long the tensor pipe still works on what has been issued: wait for this tile's last commit here
          const long long c3 = clock64();
          long long drain0 = 0;
          if (J > 0) { mbar_wait(bar_tfull, aphase); drain0 = clock64() - c3; }
          mbar_wait(bar_tfull + 8, aphase);
          const long long drain = clock64() - c3;
          if (trace_n < 256 && lane == 0) {
            long long* r = trace + 8 * trace_n;
            r[0] = tr0; r[1] = tr1; r[2] = tr_full; r[3] = tr_sf; r[4] = tr_acc1; r[5] = c3; r[6] = drain0;
            r[7] = nkt | (drain << 16);
          }
        }
        ++trace_n;
        aphase ^= 1;
      }
      if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 202); }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------ scale producer (both CTAs).  A warp of its own:
    // the scales of the next group of K tiles are requested as soon as a slot of their ring is free - up to two
    // groups (eight K tiles) ahead of the MMAs - instead of when the operand ring gets there (two to four K tiles
    // ahead, about the latency of the small copies while L2 is busy with the operands).
    if (lane == 0) {
      prefetch_tmap(&tmap_sfa); prefetch_tmap(&tmap_sfb);
      if (MODE == WGRAD && p.rows2 > 0) { prefetch_tmap(&second.sfa); prefetch_tmap(&second.sfb); }
    }
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
      const int sfa_tile = valid ? m0 / 128 : 0;         // phantom half: any in-range tile will do
      const int sfb_tile = b_base / 128;                 // n0 is a multiple of 384, hence of 128
      const bool second_prob = MODE == WGRAD && __shfl_sync(0xffffffffu, tl.prob, 0) != 0;
      const CUtensorMap* tsa = second_prob ? &second.sfa : &tmap_sfa;
      const CUtensorMap* tsb = second_prob ? &second.sfb : &tmap_sfb;
      for (int kt = kt0; kt < kt0 + nkt; kt += S::SF_GROUP) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_sfempty + 8 * sfs, sfphase ^ 1));
        if (!ok) break;
        if (elect_one()) {
          const uint32_t sffull = sffull0 + 8 * sfs;
          const uint32_t dst = sf_base + sfs * S::SF_SLOT_BYTES;
          if (rank == 0) mbar_expect_tx(bar_sffull + 8 * sfs, S::SF_TX_BYTES);
          tma_load_2d_pair(dst, tsa, sffull, 0, sfa_tile * p.sfa_ktiles + kt);
#pragma unroll
          for (int j = 0; j < S::SFB_TILES; ++j)
            tma_load_2d_pair(dst + S::SF_GROUP * 512 * (1 + j), tsb, sffull, 0,
                             (sfb_tile + j) * p.sfb_ktiles + kt);
        }
        if (++sfs == S::SF_SLOTS) { sfs = 0; sfphase ^= 1; }
      }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 206); }
  } else {
    // ------------------------------------------------------------ epilogue: 8 warps per CTA, each owns 32 rows
    // (its TMEM lane quadrant) x 96 columns of each accumulator half
    const int q = warp & 3;                      // the TMEM lane quadrant a warp may read is its index modulo 4
    const int grp = (warp - S::LEAD_WARPS) >> 2;
    const int row_in_tile = q * 32 + lane;
    constexpr int CPW = HN / 2;                 // columns per warp and half
    constexpr int NC = CPW / 32;                // 32-column chunks
    const uint32_t stg = smem_u32(epi + (warp - S::LEAD_WARPS) * S::EPI_BYTES_PER_WARP);
    const uint32_t tempty0 = map_to_cta(bar_tempty, 0);
    uint32_t aphase = 0;
    int buf = 0;
    bool ok = true;
    // timing experiment: the first epilogue warp of the leader CTA of pair 0 stamps its side of the hand-over
    long long* etrace = (p.trace != nullptr && pair_id == 0 && rank == 0 && warp == S::LEAD_WARPS && lane == 0)
                            ? p.trace + 8 * 256 : nullptr;
    int etrace_n = 0;
    for (int tile = pair_id; tile < n_total && ok; tile += n_pairs_grid) {
      const PairTile t = pair_tile<BN, MODE>(tile, rank, p, s_efo, s_pairs);
      const size_t grow = (size_t)t.m0 + row_in_tile;
      long long es[6] = {0, 0, 0, 0, 0, 0};
      if (t.nkt == 0) {
        if (MODE == WGRAD && !p.accumulate) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(t.prob ? p.c2 : p.c) +
                                                    ((size_t)t.e * (t.prob ? p.rows2 : p.rows) + grow) * p.N + t.n0 +
                                                    h * HN + grp * CPW);
            for (int i = 0; i < CPW / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        continue;
      }
      if (MODE == PLAIN) {
        // both halves are drained (bf16-packed) before anything is stored, so that neither accumulator waits
        // for the other one's stores
        uint32_t pk[2][NC][16];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (etrace && h == 0) es[0] = clock64();
          if (lane == 0) ok = mbar_wait(bar_tfull + 8 * h, aphase);
          ok = __shfl_sync(0xffffffff, ok, 0);
          if (!ok) break;
          if (etrace && h == 0) es[1] = clock64();
          tc_fence_after();
          if (!(p.debug_skip_store & 8)) {
            // all of this warp's columns of the half in one go (one wait), the accumulator is handed back before
            // the conversion: the drain is what the next tile's MMAs wait for
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + h * HN + grp * CPW;
            uint32_t r[NC][32];
#pragma unroll
            for (int c = 0; c < NC; ++c) tmem_ld32(t_row + c * 32, r[c]);
            if (etrace && h == 0) es[3] = clock64();            // (experiment: loads issued)
            tmem_ld_wait();
            if (etrace && h == 0) es[4] = clock64();            // (experiment: loads complete)
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * h);
            if (etrace && h == 0) es[2] = clock64();
#pragma unroll
            for (int c = 0; c < NC; ++c)
#pragma unroll
              for (int i = 0; i < 16; ++i)
                pk[h][c][i] = pack_bf16x2(__uint_as_float(r[c][2 * i]), __uint_as_float(r[c][2 * i + 1]));
          } else {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * h);
          }
        }
        if (!ok) break;
        if (etrace && etrace_n < 256) {
#pragma unroll
          for (int i = 0; i < 6; ++i) etrace[8 * etrace_n + i] = es[i];
        }
        ++etrace_n;
        if (t.valid && !(p.debug_skip_store & 8)) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              const uint32_t sb = stg + buf * 2048;
              if (lane == 0) bulk_wait_group_read<S::EPI_BUFS - 1>();   // the store that last read this buffer is done
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 4; ++j)
                st_shared_v4(sb + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), pk[h][c][4 * j], pk[h][c][4 * j + 1],
                             pk[h][c][4 * j + 2], pk[h][c][4 * j + 3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tmap_c, sb, t.n0 + h * HN + grp * CPW + c * 32, t.m0 + q * 32);
                bulk_commit_group();
              }
              buf ^= 1;
            }
          }
        }
      } else {  // WGRAD: f32, one half at a time (96 accumulator registers per half)
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          if (lane == 0) ok = mbar_wait(bar_tfull + 8 * h, aphase);
          ok = __shfl_sync(0xffffffff, ok, 0);
          if (!ok) break;
          tc_fence_after();
          uint32_t acc[NC][32];
          const bool drain = !(p.debug_skip_store & 8);
          if (drain) {
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + h * HN + grp * CPW;
#pragma unroll
            for (int c = 0; c < NC; ++c) tmem_ld32(t_row + c * 32, acc[c]);
            tmem_ld_wait();
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster_relaxed(tempty0 + 8 * h);
          if (!drain) continue;
#pragma unroll
          for (int c = 0; c < 2 * NC; ++c) {
            const uint32_t sb = stg + buf * 2048;
            if (lane == 0) bulk_wait_group_read<S::EPI_BUFS - 1>();
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j)
              st_shared_v4(sb + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), acc[c >> 1][(c & 1) * 16 + 4 * j],
                           acc[c >> 1][(c & 1) * 16 + 4 * j + 1], acc[c >> 1][(c & 1) * 16 + 4 * j + 2],
                           acc[c >> 1][(c & 1) * 16 + 4 * j + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int crow = t.e * (t.prob ? p.rows2 : p.rows) + t.m0 + q * 32;
              const int ccol = t.n0 + h * HN + grp * CPW + c * 16;
              const CUtensorMap* tc = t.prob ? &second.c : &tmap_c;
              if (p.accumulate) tma_reduce_add_2d(tc, sb, ccol, crow);
              else tma_store_2d(tc, sb, ccol, crow);
              bulk_commit_group();
            }
            buf ^= 1;
          }
        }
        if (!ok) break;
      }
      aphase ^= 1;
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
