// Persistent, warp-specialised MXFP8 (e4m3 x e4m3, 1x32 ue8m0 scales) grouped
// GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma kind::mxf8f6f4.block_scale
// with the accumulator in TMEM and the scales staged shared memory -> TMEM.
//
// One kernel template covers the six GEMMs of the MoE layer:
//   PLAIN   C[p, :]  = A[p, :] . B[e(p)]^T            rows grouped by expert (varlen-M), bf16 out
//   GATED   z = A[idx[p], :] . W1[e]^T, y1 = swiglu(z); z and y1 re-quantised to e4m3 in the epilogue
//   DGATED  D = A[idx[p], :] . W2T[e]^T, dSwiGLU against the saved e4m3 z, dz / y1s / ds out
//   WGRAD   C[e] (+)= A[:, seg_e] . B[:, seg_e]^T      reduction over an expert's rows (varlen-K), f32 out
// Both operands are K-major in shared memory (128-byte swizzle).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx.cuh"

namespace smoe {

// DGATEDQ = DGATED with the wgrad/dgrad operand quantizers fused into the epilogue (two-CTA kernel only)
enum GemmMode : int { PLAIN = 0, GATED = 1, DGATED = 2, WGRAD = 3, DGATEDQ = 4 };

constexpr int BM = 128;          // rows of the accumulator tile (TMEM lanes)
constexpr int BK = 128;          // bytes (= e4m3 elements) along K per stage: one scale tile
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kMaxExpertsSmem = 1024;

struct GemmParams {
  int rows;         // varlen-M: allocated rows of A'/C (TKp);  WGRAD: output rows per expert (M)
  int N;            // output columns (per expert)
  int K;            // varlen-M: reduction length;              WGRAD: allocated reduction width (TKp)
  int E;
  const int* efo;   // [E+1] padded expert row offsets (device)
  const int* a_idx; // [TKp] row gather indices for A (GATED / DGATED), else null
  const void* a_src; // the un-gathered A ([T, K] e4m3) the cp.async load warps read through a_idx
  const uint8_t* sfa;   // ISA-packed scales of A'
  const uint8_t* sfb;   // ISA-packed scales of B
  int sfa_ktiles;   // number of 128-wide K tiles in the SFA layout
  int sfb_ktiles;
  // outputs / epilogue operands
  void* c;              // PLAIN: bf16 [rows,N]; WGRAD: f32 [E,rows,N]
  long long* trace;     // timing experiment (256x384 kernel): per-tile stamps of the MMA issuer, else null
  int rows2;            // WGRAD, 256x384 kernel: output rows per expert of a SECOND product run by the same launch
  void* c2;             //   (same N, K range and operand layouts; own A, B, scales and f32 [E,rows2,N] output); 0: none
  int accumulate;       // WGRAD: add into c instead of overwriting
  int a_mn, b_mn;       // WGRAD (two-CTA kernel): operand stored [TKp, M] / [TKp, N] (MN-major) instead of transposed
  uint8_t* z_fp8;       // GATED out / DGATED in: [TKp, N_z] e4m3
  uint8_t* z_sc;        // raw ue8m0 [TKp, N_z/32]
  uint8_t* y1_fp8;      // GATED out: [TKp, N/2] e4m3
  uint8_t* y1_sf;       // GATED out: ISA-packed scales for (TKp, N/2)
  const float* s;       // DGATED: per-row score [TKp]
  void* dz;             // DGATED out: bf16 [TKp, 2N]
  void* y1s;            // DGATED out: bf16 [TKp, N]
  float* ds_partial;    // DGATED out: [N/BN, TKp]
  uint8_t* dz_row_sf;   // DGATEDQ out: ISA scales of dz as a (TKp, 2N) operand (32x32 blocks share a scale)
  uint8_t* dz_col_sf;   // DGATEDQ out: ISA scales of dz^T as a (2N, TKp) operand
  uint8_t* y1s_col_sf;  // DGATEDQ out: ISA scales of y1s^T as a (N, TKp) operand (1x32 along TKp)
  int* status;          // device status word: 0 ok, else first failure code
  int debug_skip_store; // timing experiments only: drain TMEM but skip the global stores
  int dbg_stage_cut;    // timing experiments only: use this many fewer ring stages
  int l2_prefetch;      // K tiles ahead of the shared-memory ring at which operand tiles are prefetched into L2 (0 = off)
};

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK;
  static constexpr int B_BYTES = BN * BK;
  static constexpr int SF_BYTES = 2048;                       // SFA 512 + SFB up to 1024, padded
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES;
  static constexpr int AUX_BYTES = 1024 + (kMaxExpertsSmem + 1) * 4;
  static constexpr int STAGES = (227 * 1024 - 1024 - AUX_BYTES) / STAGE_BYTES > 6
                                    ? 6 : (227 * 1024 - 1024 - AUX_BYTES) / STAGE_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + AUX_BYTES + 1024;  // + alignment slack
  static constexpr int ACC_STAGES = (BN <= 128) ? 2 : 1;
  static constexpr int SF_COLS = 4 + BN / 32;                  // SFA 4 cols + SFB 4 per 128 rows
  static constexpr int SF_COL0 = ACC_STAGES * BN;
  static_assert(SF_COL0 + STAGES * SF_COLS <= 512, "TMEM budget");
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ue8m0 byte of a group amax (bits of a non-negative float).
__device__ __forceinline__ int e8m0_of(float amax) {
  const int bits = __float_as_int(amax);
  const int bexp = (bits >> 23) & 0xFF;
  const int e = bexp - 8 + ((bits & 0x7FFFFF) > 0x600000 ? 1 : 0);
  return bexp > 0 ? max(e, 0) : 0;
}
__device__ __forceinline__ float qscale_of(int e8m0) {
  return __int_as_float(min(max(254 - e8m0, 1), 254) << 23);
}
// four floats -> four e4m3 bytes (round to nearest even, saturate to +-448)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ float bf16_rne(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// two packed e4m3 bytes (low, high) -> two floats
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t pair) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)pair));
  return make_float2(__half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF))),
                     __half2float(__ushort_as_half((unsigned short)(h2 >> 16))));
}

struct TileInfo {
  int m0, n0, e, kt0, nkt;   // row/col origin, expert, first K tile and K-tile count
};

// Tile -> coordinates.  varlen-M: row tiles of 128 over [0, efo[E]); columns fastest.
// WGRAD: (expert, row tile, col tile), K range = the expert's row segment.
template <int BN, int MODE>
__device__ __forceinline__ TileInfo tile_info(int tile, const GemmParams& p, const int* s_efo) {
  TileInfo t;
  const int n_tiles = p.N / BN;
  if (MODE == WGRAD) {
    const int m_tiles = p.rows / BM;
    const int per_e = m_tiles * n_tiles;
    t.e = tile / per_e;
    const int r = tile - t.e * per_e;
    t.m0 = (r / n_tiles) * BM;
    t.n0 = (r % n_tiles) * BN;
    t.kt0 = s_efo[t.e] / BK;
    t.nkt = (s_efo[t.e + 1] - s_efo[t.e]) / BK;
  } else {
    const int mt = tile / n_tiles;
    t.m0 = mt * BM;
    t.n0 = (tile - mt * n_tiles) * BN;
    int lo = 0, hi = p.E;          // largest e with efo[e] <= m0 and efo[e+1] > m0
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_efo[mid + 1] <= t.m0) lo = mid + 1; else hi = mid;
    }
    t.e = lo;
    t.kt0 = 0;
    t.nkt = p.K / BK;
  }
  return t;
}

template <int BN, int MODE>
__device__ __forceinline__ int total_tiles(const GemmParams& p, const int* s_efo) {
  if (MODE == WGRAD) return p.E * (p.rows / BM) * (p.N / BN);
  return (s_efo[p.E] / BM) * (p.N / BN);
}

template <int BN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxf8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using S = GemmSmem<BN>;
  const bool GATHER = p.a_idx != nullptr;   // rows of A fetched by index (TMA gather4) vs. a plain tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* aux = smem + S::STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(aux);            // full[S], empty[S], tfull[2], tempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(aux + 512);
  volatile int* s_abort = reinterpret_cast<volatile int*>(aux + 516);
  int* s_efo = reinterpret_cast<int*>(aux + 1024);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * S::STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * S::STAGES;
  const uint32_t bar_tempty = bar_tfull + 8 * 2;

  for (int i = threadIdx.x; i <= p.E; i += blockDim.x) s_efo[i] = p.efo[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, kEpiWarps);
    }
    *s_abort = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_total = total_tiles<BN, MODE>(p, s_efo);
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x) {
      const TileInfo t = tile_info<BN, MODE>(tile, p, s_efo);
      if (t.nkt == 0) continue;
      int4 rows4 = make_int4(0, 0, 0, 0);
      if (GATHER) rows4 = *reinterpret_cast<const int4*>(p.a_idx + t.m0 + 4 * lane);
      const int b_row = (MODE == WGRAD) ? t.n0 : t.e * p.N + t.n0;
      const int sfa_row_tile = t.m0 / 128;
      const int sfb_row_tile = b_row / 128;
      for (int kt = t.kt0; kt < t.kt0 + t.nkt; ++kt) {
        const uint32_t full = bar_full + 8 * stage;
        if (lane == 0) ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1);
        ok = __shfl_sync(0xffffffff, ok, 0);
        if (!ok) break;
        const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
        const uint32_t b_dst = a_dst + S::A_BYTES;
        const uint32_t sf_dst = b_dst + S::B_BYTES;
        if (lane == 0) {
          mbar_expect_tx(full, S::A_BYTES + S::B_BYTES + 512 + (BN / 128) * 512);
          if (!GATHER) tma_load_2d(a_dst, &tmap_a, full, kt * BK, t.m0);
          tma_load_2d(b_dst, &tmap_b, full, kt * BK, b_row);   // box = {BK, BN}
          bulk_load(sf_dst, p.sfa + ((size_t)sfa_row_tile * p.sfa_ktiles + kt) * 512, 512, full);
#pragma unroll
          for (int j = 0; j < BN / 128; ++j)
            bulk_load(sf_dst + 512 + j * 512, p.sfb + ((size_t)(sfb_row_tile + j) * p.sfb_ktiles + kt) * 512, 512,
                      full);
        }
        if (GATHER) {
          __syncwarp();
          tma_gather4(a_dst + lane * 4 * BK, &tmap_a, full, kt * BK, rows4.x, rows4.y, rows4.z, rows4.w);
        }
        if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
      }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 101); }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_mxf8(BM, BN);
      int stage = 0, as = 0;
      uint32_t phase = 0, aphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x) {
        const TileInfo t = tile_info<BN, MODE>(tile, p, s_efo);
        if (t.nkt == 0) continue;
        ok = mbar_wait(bar_tempty + 8 * as, aphase ^ 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        for (int k = 0; k < t.nkt; ++k) {
          ok = mbar_wait(bar_full + 8 * stage, phase);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_src = a_src + S::A_BYTES;
          const uint32_t sf_src = b_src + S::B_BYTES;
          const uint32_t sfa_t = tmem_base + S::SF_COL0 + stage * S::SF_COLS;
          const uint32_t sfb_t = sfa_t + 4;
          tc_cp_sf(sfa_t, make_desc_sf(sf_src));
#pragma unroll
          for (int j = 0; j < BN / 128; ++j) tc_cp_sf(sfb_t + 4 * j, make_desc_sf(sf_src + 512 + 512 * j));
          const uint64_t a_desc = make_desc_kmajor_sw128(a_src);
          const uint64_t b_desc = make_desc_kmajor_sw128(b_src);
#pragma unroll
          for (int kb = 0; kb < BK / 32; ++kb) {
            mma_mxf8(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, idesc_with_sf_ids(idesc, kb, kb), sfa_t, sfb_t,
                     (k | kb) != 0);
          }
          tc_commit(bar_empty + 8 * stage);
          if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(bar_tfull + 8 * as);
        if (++as == S::ACC_STAGES) { as = 0; aphase ^= 1; }
      }
      if (!ok) { *s_abort = 1; atomicCAS(p.status, 0, 102); }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int row_in_tile = q * 32 + lane;
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_total && ok; tile += gridDim.x) {
      const TileInfo t = tile_info<BN, MODE>(tile, p, s_efo);
      const size_t grow = (size_t)t.m0 + row_in_tile;
      if (t.nkt == 0) {
        if (MODE == WGRAD && !p.accumulate) {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) +
                                                  ((size_t)t.e * p.rows + grow) * p.N + t.n0);
          for (int i = 0; i < BN / 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        continue;
      }
      if (lane == 0) ok = mbar_wait(bar_tfull + 8 * as, aphase);
      ok = __shfl_sync(0xffffffff, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * BN;

      if (MODE == PLAIN) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.c) + grow * p.N + t.n0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
            if (!p.debug_skip_store || v.x == 0x12345678u) dst[c * 4 + i] = v;
          }
        }
      } else if (MODE == WGRAD) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) +
                                                ((size_t)t.e * p.rows + grow) * p.N + t.n0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                   __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            if (p.accumulate) {
              const float4 o = dst[c * 8 + i];
              v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            dst[c * 8 + i] = v;
          }
        }
      } else if (MODE == GATED) {
        // z tile columns [n0, n0+BN) of 2I; y1 columns [n0/2, n0/2 + BN/2) of I.
        const int Nz = p.N, Ny = p.N / 2;
        uint8_t* zrow = p.z_fp8 + grow * Nz + t.n0;
        uint8_t* zsc = p.z_sc + grow * (Nz / 32) + t.n0 / 32;
        uint8_t* yrow = p.y1_fp8 + grow * Ny + t.n0 / 2;
        uint32_t y_sc_word = 0;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          float y[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld32(t_row + c * 64 + h * 32, r);
            tmem_ld_wait();
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(__uint_as_float(r[i])));
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = __uint_as_float(r[2 * i]), u = __uint_as_float(r[2 * i + 1]);
              const float sig = 1.0f / (1.0f + expf(-g));
              y[h * 16 + i] = bf16_rne((g * sig) * u);
            }
            const int e = e8m0_of(fmaxf(amax, 1e-4f));
            const float qs = qscale_of(e);
            uint4* zd = reinterpret_cast<uint4*>(zrow + c * 64 + h * 32);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              uint4 v;
              v.x = pack_e4m3x4(__uint_as_float(r[16 * i + 0]) * qs, __uint_as_float(r[16 * i + 1]) * qs,
                                __uint_as_float(r[16 * i + 2]) * qs, __uint_as_float(r[16 * i + 3]) * qs);
              v.y = pack_e4m3x4(__uint_as_float(r[16 * i + 4]) * qs, __uint_as_float(r[16 * i + 5]) * qs,
                                __uint_as_float(r[16 * i + 6]) * qs, __uint_as_float(r[16 * i + 7]) * qs);
              v.z = pack_e4m3x4(__uint_as_float(r[16 * i + 8]) * qs, __uint_as_float(r[16 * i + 9]) * qs,
                                __uint_as_float(r[16 * i + 10]) * qs, __uint_as_float(r[16 * i + 11]) * qs);
              v.w = pack_e4m3x4(__uint_as_float(r[16 * i + 12]) * qs, __uint_as_float(r[16 * i + 13]) * qs,
                                __uint_as_float(r[16 * i + 14]) * qs, __uint_as_float(r[16 * i + 15]) * qs);
              zd[i] = v;
            }
            zsc[c * 2 + h] = (uint8_t)e;
          }
          float amax = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(y[i]));
          const int e = e8m0_of(amax);
          const float qs = qscale_of(e);
          uint4* yd = reinterpret_cast<uint4*>(yrow + c * 32);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint4 v;
            v.x = pack_e4m3x4(y[16 * i + 0] * qs, y[16 * i + 1] * qs, y[16 * i + 2] * qs, y[16 * i + 3] * qs);
            v.y = pack_e4m3x4(y[16 * i + 4] * qs, y[16 * i + 5] * qs, y[16 * i + 6] * qs, y[16 * i + 7] * qs);
            v.z = pack_e4m3x4(y[16 * i + 8] * qs, y[16 * i + 9] * qs, y[16 * i + 10] * qs, y[16 * i + 11] * qs);
            v.w = pack_e4m3x4(y[16 * i + 12] * qs, y[16 * i + 13] * qs, y[16 * i + 14] * qs, y[16 * i + 15] * qs);
            yd[i] = v;
          }
          // ISA layout for logical (TKp, I): y1 group index g = (n0/2)/32 + c
          const int g = (t.n0 / 2) / 32 + c;
          if (BN == 256) {
            y_sc_word |= (uint32_t)e << (8 * c);
            if (c == 3) {
              const size_t off = ((grow / 128) * (size_t)(Ny / 128) + g / 4) * 512 + (grow % 32) * 16 +
                                 ((grow % 128) / 32) * 4;
              *reinterpret_cast<uint32_t*>(p.y1_sf + off) = y_sc_word;
            }
          } else {
            const size_t off = ((grow / 128) * (size_t)(Ny / 128) + g / 4) * 512 + (grow % 32) * 16 +
                               ((grow % 128) / 32) * 4 + (g % 4);
            p.y1_sf[off] = (uint8_t)e;
          }
        }
      } else {  // DGATED
        // D tile columns [n0, n0+BN) of I; z columns [2 n0, 2 n0 + 2 BN) of 2I.
        const int Ni = p.N, Nz = 2 * p.N;
        const float s = p.s[grow];
        const uint8_t* zrow = p.z_fp8 + grow * Nz + 2 * t.n0;
        const uint8_t* zsc = p.z_sc + grow * (Nz / 32) + (2 * t.n0) / 32;
        uint4* dzrow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.dz) + grow * Nz + 2 * t.n0);
        uint4* ysrow = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.y1s) + grow * Ni + t.n0);
        float ds_acc = 0.f;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_row + c * 32, r);
          uint4 zb[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) zb[i] = reinterpret_cast<const uint4*>(zrow + c * 64)[i];
          const float sc0 = __int_as_float((int)zsc[c * 2] << 23);
          const float sc1 = __int_as_float((int)zsc[c * 2 + 1] << 23);
          tmem_ld_wait();
          const uint32_t* zw = reinterpret_cast<const uint32_t*>(zb);
          uint32_t dzp[32];
          uint32_t ysp[16];
          float yprev = 0.f;
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const uint32_t pair = (zw[i >> 1] >> (16 * (i & 1))) & 0xFFFF;
            const float sc = (i < 16) ? sc0 : sc1;
            const float2 gu = e4m3x2_to_f32(pair);
            const float g = gu.x * sc, u = gu.y * sc;
            const float D = __uint_as_float(r[i]);
            const float dout = s * D;
            const float sig = 1.0f / (1.0f + expf(-g));
            const float silu = g * sig;
            const float sd = silu * dout;
            const float dg = ((sig - silu * sig) * dout + sd) * u;
            const float y = silu * u;
            ds_acc = fmaf(y, D, ds_acc);
            dzp[i] = pack_bf16x2(dg, sd);
            const float ys = s * y;
            if (i & 1) ysp[i >> 1] = pack_bf16x2(yprev, ys); else yprev = ys;
          }
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dzrow[c * 8 + i] = make_uint4(dzp[4 * i], dzp[4 * i + 1], dzp[4 * i + 2], dzp[4 * i + 3]);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            ysrow[c * 4 + i] = make_uint4(ysp[4 * i], ysp[4 * i + 1], ysp[4 * i + 2], ysp[4 * i + 3]);
        }
        p.ds_partial[(size_t)(t.n0 / BN) * p.rows + grow] = ds_acc;
      }

      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * as);
      if (++as == S::ACC_STAGES) { as = 0; aphase ^= 1; }
    }
    if (!ok && lane == 0) { *s_abort = 1; atomicCAS(p.status, 0, 103); }
  }

  // common exit: everyone arrives here, also after a failed wait
  __syncthreads();
  if (*s_abort) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

}  // namespace smoe
