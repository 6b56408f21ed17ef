// Host side of the MXFP8 grouped GEMMs: tensor-map construction and launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "gemm.cuh"
#include "gemm2.cuh"
#include "gemm3.cuh"
#include "smoe_b200.h"
#include "smoe_internal.h"

namespace smoe {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static bool load_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  return g_encode != nullptr;
}

// 2D row-major uint8 tensor [rows, cols], box {box_cols, box_rows}, 128-byte swizzle.
static int make_tmap_u8(CUtensorMap* m, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                        uint32_t box_rows) {
  if (!load_encode()) return SMOE_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols & 15)) return SMOE_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_TMAP;
}

// General 2D row-major tensor map.
static int make_tmap(CUtensorMap* m, CUtensorMapDataType dt, int esize, const void* base, uint64_t rows,
                     uint64_t cols, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
  if (!load_encode()) return SMOE_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((cols * esize) & 15)) return SMOE_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * esize};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SMOE_OK : SMOE_ERR_TMAP;
}

static int g_force_bn = 0;
static int g_skip_store = 0;
static int g_force_v1 = 0;
static int g_force_gather4 = 0;     // A rows by index: TMA gather4 instead of the cp.async load warps
static int g_stage_cut = 0;
static int g_l2_prefetch = -1;     // -1: the kernel's default
static void* g_trace = nullptr;    // timing experiment: per-tile stamps of the MMA issuer (256 x 384 kernel)

// Per-device state: the SM count and the "large dynamic shared memory" function attribute belong to a device,
// not to the process, so both are kept per device ordinal.
constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices] = {};

static int current_device() {
  int dev = 0;
  cudaGetDevice(&dev);
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

static int sm_count() {
  const int dev = current_device();
  if (g_sm_count[dev] == 0) cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
  return g_sm_count[dev];
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel instantiation, device)
template <typename Kern>
static bool ensure_smem_attr(Kern kern, int bytes, bool (&done)[kMaxDevices]) {
  const int dev = current_device();
  if (done[dev]) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  done[dev] = true;
  return true;
}

template <int BN, int MODE>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_tiles,
                  cudaStream_t stream) {
  using S = GemmSmem<BN>;
  static bool attr_set[kMaxDevices] = {};
  auto kern = gemm_mxf8_kernel<BN, MODE>;
  if (!ensure_smem_attr(kern, S::TOTAL, attr_set)) return SMOE_ERR_LAUNCH;
  int grid = sm_count();
  if (max_tiles < grid) grid = max_tiles;
  if (grid <= 0) return SMOE_OK;
  kern<<<grid, kThreads, S::TOTAL, stream>>>(ta, tb, p);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

static int pick_bn(int64_t N) {
  if (g_force_bn == 128 || g_force_bn == 256) return (N % g_force_bn == 0) ? g_force_bn : 128;
  return (N % 256 == 0) ? 256 : 128;
}

// ---- two-CTA kernel -----------------------------------------------------------
struct OutMaps {
  CUtensorMap c, c2, c3;
};

template <int BN, int MODE, bool CPG = false>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                   const OutMaps& om, const GemmParams& p, int64_t max_pair_tiles, cudaStream_t stream) {
  using S = Gemm2Smem<BN, MODE, CPG>;
  static bool attr_set[kMaxDevices] = {};
  auto kern = gemm2_mxf8_kernel<BN, MODE, CPG>;
  if (!ensure_smem_attr(kern, S::TOTAL, attr_set)) return SMOE_ERR_LAUNCH;
  int64_t pairs = sm_count() / 2;
  if (max_pair_tiles < pairs) pairs = max_pair_tiles;
  if (pairs <= 0) return SMOE_OK;
  GemmParams q = p;
  q.dbg_stage_cut = g_stage_cut;
  q.l2_prefetch = g_l2_prefetch >= 0 ? g_l2_prefetch : kDefaultL2Prefetch;
  kern<<<(unsigned)(2 * pairs), S::THREADS, S::TOTAL, stream>>>(ta, tb, tsa, tsb, om.c, om.c2, om.c3, q);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

// ---- two-CTA kernel with the 256 x 384 double-accumulator tile (PLAIN and WGRAD) ------------------------------
template <int MODE>
static int launch3(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                   const CUtensorMap& tc, const GemmParams& p, int64_t max_pair_tiles, cudaStream_t stream,
                   const SecondMaps* second = nullptr) {
  using S = Gemm3Smem<MODE>;
  static bool attr_set[kMaxDevices] = {};
  auto kern = gemm3_mxf8_kernel<MODE>;
  if (!ensure_smem_attr(kern, S::TOTAL, attr_set)) return SMOE_ERR_LAUNCH;
  int64_t pairs = sm_count() / 2;
  if (max_pair_tiles < pairs) pairs = max_pair_tiles;
  if (pairs <= 0) return SMOE_OK;
  GemmParams q = p;
  q.dbg_stage_cut = g_stage_cut > 2 ? 2 : g_stage_cut;      // the head / tail schedule holds two stages
  q.l2_prefetch = g_l2_prefetch;                            // this kernel reads it as "length of the head / tail", -1 = default
  q.trace = reinterpret_cast<long long*>(g_trace);
  SecondMaps none{};
  kern<<<(unsigned)(2 * pairs), S::THREADS, S::TOTAL, stream>>>(ta, tb, tsa, tsb, tc, second ? *second : none, q);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

// Whether the 384-wide kernel takes this problem.  WGRAD: B must be K-major ([N, TKp]); A either way.
template <int MODE>
static bool use_gemm3(const GemmParams& p) {
  if (MODE != PLAIN && MODE != WGRAD) return false;
  if (g_force_v1 || (g_force_bn != 0 && g_force_bn != kBN3)) return false;
  if (p.N % kBN3 != 0 || p.E > kMaxExperts2) return false;
  if (MODE == WGRAD && (p.rows % 256 != 0 || p.b_mn)) return false;
  if (MODE == PLAIN && p.b_mn) return false;      // a 192-byte MN-major slice is not a swizzle atom
  return true;
}

template <int MODE>
static int run3(const void* a, int64_t a_rows, int64_t a_cols, const void* b, int64_t b_rows, int64_t b_cols,
                GemmParams& p, cudaStream_t stream) {
  CUtensorMap ta, tb, tsa, tsb, tc;
  int rc = make_tmap_u8(&ta, a, a_rows, a_cols, BK, BM);
  if (rc) return rc;
  rc = make_tmap_u8(&tb, b, b_rows, b_cols, BK, kHN3 / 2);
  if (rc) return rc;
  const int64_t sfa_tiles = (int64_t)(p.rows / 128) * p.sfa_ktiles;
  const int64_t sfb_tiles = (MODE == WGRAD) ? (int64_t)(p.N / 128) * p.sfb_ktiles : (b_rows / 128) * p.sfb_ktiles;
  rc = make_tmap(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfa, sfa_tiles, 128, 128, kSfGroup2,
                 CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfb, sfb_tiles, 128, 128, kSfGroup2,
                 CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  int64_t pair_tiles;
  if (MODE == WGRAD) {
    rc = make_tmap(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.c, (uint64_t)p.E * p.rows, p.N, 16, 32,
                   CU_TENSOR_MAP_SWIZZLE_64B);
    pair_tiles = (int64_t)p.E * (p.rows / 256) * (p.N / kBN3);
  } else {
    rc = make_tmap(&tc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.c, p.rows, p.N, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
    pair_tiles = ((int64_t)p.rows / 256 + p.E) * (p.N / kBN3);
  }
  if (rc) return rc;
  constexpr int M3 = (MODE == WGRAD) ? WGRAD : PLAIN;
  return launch3<M3>(ta, tb, tsa, tsb, tc, p, pair_tiles, stream);
}

// Two weight-gradient products in ONE launch of the 256 x 384 kernel: same N, same K range (TKp), same operand
// layouts (A [TKp, M] or [M, TKp] for both; B K-major), own operands, scales and outputs.
static int run3_wgrad_pair(const void* a1, const void* b1, GemmParams& p, const void* a2, const void* b2,
                           const uint8_t* sfa2, const uint8_t* sfb2, int64_t TKp, cudaStream_t stream) {
  CUtensorMap ta, tb, tsa, tsb, tc;
  SecondMaps sm{};
  const int64_t M1 = p.rows, M2 = p.rows2;
  int rc = make_tmap_u8(&ta, a1, p.a_mn ? TKp : M1, p.a_mn ? M1 : TKp, BK, BM);
  if (!rc) rc = make_tmap_u8(&sm.a, a2, p.a_mn ? TKp : M2, p.a_mn ? M2 : TKp, BK, BM);
  if (!rc) rc = make_tmap_u8(&tb, b1, p.N, TKp, BK, kHN3 / 2);
  if (!rc) rc = make_tmap_u8(&sm.b, b2, p.N, TKp, BK, kHN3 / 2);
  if (rc) return rc;
  const int64_t sfb_tiles = (int64_t)(p.N / 128) * p.sfb_ktiles;
  rc = make_tmap(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfa, (int64_t)(M1 / 128) * p.sfa_ktiles, 128, 128, kSfGroup2,
                 CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!rc) rc = make_tmap(&sm.sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sfa2, (int64_t)(M2 / 128) * p.sfa_ktiles, 128, 128,
                          kSfGroup2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!rc) rc = make_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfb, sfb_tiles, 128, 128, kSfGroup2,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!rc) rc = make_tmap(&sm.sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, sfb2, sfb_tiles, 128, 128, kSfGroup2,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
  if (!rc) rc = make_tmap(&tc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.c, (uint64_t)p.E * M1, p.N, 16, 32,
                          CU_TENSOR_MAP_SWIZZLE_64B);
  if (!rc) rc = make_tmap(&sm.c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.c2, (uint64_t)p.E * M2, p.N, 16, 32,
                          CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  const int64_t pair_tiles = (int64_t)p.E * ((M1 + M2) / 256) * (p.N / kBN3);
  return launch3<WGRAD>(ta, tb, tsa, tsb, tc, p, pair_tiles, stream, &sm);
}

// Column tile of the two-CTA kernel for a mode and N; 0 = not applicable.
template <int MODE>
static int pick_bn2(int64_t N) {
  if (g_force_v1) return 0;
  const bool wide = (MODE == PLAIN || MODE == WGRAD || MODE == GATED);      // single-stage 256-column tiles
  if (MODE == DGATEDQ) {
    // 192-column tiles also when N is not a multiple of 192, with a ragged last tile, as long as that wastes
    // at most a tenth of the columns (N = 4096: 22 tiles for 21.3)
    const int64_t padded = (N + 191) / 192 * 192;
    return ((N % 192 == 0 || padded * 10 <= N * 11) && g_force_bn != 128) ? 192 : 128;
  }
  if (g_force_bn == 128) return 128;
  if (g_force_bn == kBN3) return (wide && N % 256 == 0) ? 256 : ((N % 192 == 0) ? 192 : 128);   // 384 did not apply
  if (g_force_bn == 192) return (N % 192 == 0) ? 192 : 128;
  if (g_force_bn == 256) return (wide && N % 256 == 0) ? 256 : 128;
  if (wide && N % 256 == 0) return 256;
  return (N % 192 == 0) ? 192 : 128;
}

template <int MODE>
static int run2(const void* a, int64_t a_rows, int64_t a_cols, const void* b, int64_t b_rows, int64_t b_cols,
                GemmParams& p, const OutMaps& om, int bn, int64_t sfa_tiles, int64_t sfb_tiles, cudaStream_t stream) {
  CUtensorMap ta, tb, tsa, tsb;
  const bool gather = p.a_idx != nullptr;
  int rc = make_tmap_u8(&ta, a, a_rows, a_cols, BK, gather ? 1 : BM);
  if (rc) return rc;
  rc = make_tmap_u8(&tb, b, b_rows, b_cols, BK, bn / 2);
  if (rc) return rc;
  rc = make_tmap(&tsa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfa, sfa_tiles, 128, 128, kSfGroup2,
                 CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  rc = make_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, p.sfb, sfb_tiles, 128, 128, kSfGroup2,
                 CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;
  // upper bound of pair tiles: varlen-M: every expert may add one half-empty pair
  int64_t pair_tiles;
  if (MODE == WGRAD) pair_tiles = (int64_t)p.E * (p.rows / 256) * (p.N / bn);
  else pair_tiles = ((int64_t)p.rows / 256 + p.E) * ((p.N + bn - 1) / bn);
  // indexed A rows: cp.async load warps (GATED / DGATED / DGATEDQ), unless the test knob asks for TMA gather4
  constexpr bool CAN_CPG = (MODE == GATED || MODE == DGATED || MODE == DGATEDQ);
  if (CAN_CPG && gather && !g_force_gather4) {
    constexpr int MC = CAN_CPG ? MODE : GATED;
    p.a_src = a;
    if (bn == 256) {
      constexpr int M256 = (MC == GATED) ? GATED : GATED;       // of the gather modes only GATED runs 256 columns
      return launch2<256, M256, true>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
    }
    if (bn == 192) return launch2<192, MC, true>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
    return launch2<128, MC, true>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
  }
  if (bn == 256) {
    constexpr int M256 = (MODE == PLAIN || MODE == WGRAD || MODE == GATED) ? MODE : PLAIN;   // only the wide modes reach here
    return launch2<256, M256>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
  }
  if (bn == 192) return launch2<192, MODE>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
  return launch2<128, MODE>(ta, tb, tsa, tsb, om, p, pair_tiles, stream);
}

template <int MODE>
static int run(const void* a, int64_t a_rows, int64_t a_cols, const void* b, int64_t b_rows, int64_t b_cols,
               GemmParams& p, int max_tiles_128, cudaStream_t stream) {
  if (p.E > kMaxExpertsSmem) return SMOE_ERR_SHAPE;
  if (use_gemm3<MODE>(p)) return run3<MODE>(a, a_rows, a_cols, b, b_rows, b_cols, p, stream);
  {
    const int bn2 = pick_bn2<MODE>(p.N);
    const bool ok2 = bn2 != 0 && p.E <= kMaxExperts2 && (MODE != WGRAD || p.rows % 256 == 0);
    if (ok2) {
      OutMaps om{};
      int rc = SMOE_OK;
      const int64_t sfa_tiles = (MODE == WGRAD) ? (int64_t)(p.rows / 128) * p.sfa_ktiles
                                                : (int64_t)(p.rows / 128) * p.sfa_ktiles;
      const int64_t sfb_tiles = (MODE == WGRAD) ? (int64_t)(p.N / 128) * p.sfb_ktiles
                                : (MODE == PLAIN && p.b_mn) ? ((int64_t)p.E * p.N / 128) * p.sfb_ktiles
                                                            : (b_rows / 128) * p.sfb_ktiles;
      if ((MODE == WGRAD || MODE == PLAIN) && (p.a_mn || p.b_mn) && bn2 != 256) return SMOE_ERR_SHAPE;
      if (MODE == PLAIN) {
        rc = make_tmap(&om.c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.c, p.rows, p.N, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B);
        om.c2 = om.c;
      } else if (MODE == WGRAD) {
        rc = make_tmap(&om.c, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, p.c, (uint64_t)p.E * p.rows, p.N, 16, 32,
                       CU_TENSOR_MAP_SWIZZLE_64B);
        om.c2 = om.c;
      } else if (MODE == DGATEDQ) {
        rc = make_tmap(&om.c, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.dz, p.rows, 2 * (uint64_t)p.N, 64, 32,
                       CU_TENSOR_MAP_SWIZZLE_64B);
        if (!rc)
          rc = make_tmap(&om.c2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.y1s, p.rows, p.N, 32, 32, CU_TENSOR_MAP_SWIZZLE_32B);
      } else if (MODE == DGATED) {
        rc = make_tmap(&om.c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.dz, p.rows, 2 * (uint64_t)p.N, 64, 32,
                       CU_TENSOR_MAP_SWIZZLE_128B);
        if (!rc)
          rc = make_tmap(&om.c2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, p.y1s, p.rows, p.N, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_64B);
      } else {  // GATED: z e4m3 [rows, N] in 32 x 64 boxes, y1 e4m3 [rows, N/2] in 32 x 32 boxes
        rc = make_tmap(&om.c, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.z_fp8, p.rows, p.N, 64, 32, CU_TENSOR_MAP_SWIZZLE_64B);
        if (!rc)
          rc = make_tmap(&om.c2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.y1_fp8, p.rows, p.N / 2, 32, 32,
                         CU_TENSOR_MAP_SWIZZLE_32B);
      }
      if (rc) return rc;
      om.c3 = om.c;
      return run2<MODE>(a, a_rows, a_cols, b, b_rows, b_cols, p, om, bn2, sfa_tiles, sfb_tiles, stream);
    }
  }
  if (MODE == DGATEDQ) return SMOE_ERR_SHAPE;     // fused-quantizer epilogue exists in the two-CTA kernel only
  if ((MODE == WGRAD || MODE == PLAIN) && (p.a_mn || p.b_mn)) return SMOE_ERR_SHAPE;   // so do MN-major operands
  constexpr int M1 = (MODE == DGATEDQ) ? DGATED : MODE;
  const int bn = pick_bn(p.N);
  CUtensorMap ta, tb;
  const bool gather = p.a_idx != nullptr;
  int rc = make_tmap_u8(&ta, a, a_rows, a_cols, BK, gather ? 1 : BM);
  if (rc) return rc;
  rc = make_tmap_u8(&tb, b, b_rows, b_cols, BK, bn);
  if (rc) return rc;
  if (bn == 256) return launch<256, M1>(ta, tb, p, max_tiles_128 / 2, stream);
  return launch<128, M1>(ta, tb, p, max_tiles_128, stream);
}

// A weight-gradient call over zero routed rows: the product is empty, so an accumulating call leaves c as it is and
// an overwriting call stores zeros.
static int wgrad_nothing_routed(float* c, int64_t M, int64_t N, int64_t E, int accumulate, cudaStream_t stream) {
  if (accumulate) return SMOE_OK;
  if (c == nullptr) return SMOE_ERR_ARG;
  return cudaMemsetAsync(c, 0, (size_t)E * M * N * sizeof(float), stream) == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_internal_gemm_trace(void* device_buffer) {
  g_trace = device_buffer;
  return SMOE_OK;
}

int smoe_internal_gemm_knobs(int bn) {
  g_force_bn = bn & 0xFFFF;
  g_skip_store = ((bn >> 16) & 1) | (((bn >> 18) & 1) << 1);   // bit 16: no stores; bit 18: no epilogue (fused dgated)
  g_force_v1 = (bn >> 17) & 1;
  g_skip_store |= ((bn >> 19) & 0x1F) << 2;    // bits 19..23 -> timing-experiment bits 2..6 of GemmParams::debug_skip_store
  g_force_gather4 = (bn >> 31) & 1;            // bit 31: indexed A rows through TMA gather4
  g_stage_cut = (bn >> 24) & 3;                // bits 24..25: ring stages to leave unused
  g_l2_prefetch = ((bn >> 26) & 0x1F) - 1;     // bits 26..30: L2 prefetch distance + 1 (0 = kernel default)
  return SMOE_OK;
}

int smoe_gemm_varlen_m(const void* a_fp8, const void* a_sf, const void* b_fp8, const void* b_sf, const int* efo,
                       void* c_bf16, int64_t rows, int64_t N, int64_t K, int64_t E, int* status, void* stream) {
  if (rows < 0 || rows % 128 || N % 128 || K % 128 || E <= 0) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;                  // no routed rows (an expert-parallel rank may receive none)
  GemmParams p{};
  p.rows = (int)rows; p.N = (int)N; p.K = (int)K; p.E = (int)E;
  p.efo = efo; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)b_sf;
  p.sfa_ktiles = (int)(K / 128); p.sfb_ktiles = (int)(K / 128);
  p.c = c_bf16; p.status = status; p.debug_skip_store = g_skip_store;
  return run<PLAIN>(a_fp8, rows, K, b_fp8, E * N, K, p, (int)((rows / 128) * (N / 128)), (cudaStream_t)stream);
}

int smoe_gemm_varlen_m_bt(const void* a_fp8, const void* a_sf, const void* b_kn_fp8, const void* b_sf, const int* efo,
                          void* c_bf16, int64_t rows, int64_t N, int64_t K, int64_t E, int* status, void* stream) {
  if (rows < 0 || rows % 128 || N % 256 || K % 128 || E <= 0 || E > kMaxExperts2) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  GemmParams p{};
  p.rows = (int)rows; p.N = (int)N; p.K = (int)K; p.E = (int)E;
  p.efo = efo; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)b_sf;
  p.sfa_ktiles = (int)(K / 128); p.sfb_ktiles = (int)(K / 128);
  p.c = c_bf16; p.status = status; p.debug_skip_store = g_skip_store;
  p.b_mn = 1;                                      // B of expert e = rows [e*K, (e+1)*K) of an [E*K, N] matrix
  return run<PLAIN>(a_fp8, rows, K, b_kn_fp8, E * K, N, p, (int)((rows / 128) * (N / 128)), (cudaStream_t)stream);
}

int smoe_gemm_gated(const void* x_fp8, int64_t T, const int* a_idx, const void* a_sf, const void* w1_fp8,
                    const void* w1_sf, const int* efo, void* z_fp8, void* z_scales, void* y1_fp8, void* y1_sf,
                    int64_t rows, int64_t N, int64_t K, int64_t E, int* status, void* stream) {
  if (rows < 0 || rows % 128 || N % 256 || K % 128 || E <= 0 || T < 0) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  if (T == 0) return SMOE_ERR_SHAPE;              // rows to compute but nothing to read them from
  GemmParams p{};
  p.rows = (int)rows; p.N = (int)N; p.K = (int)K; p.E = (int)E;
  p.efo = efo; p.a_idx = a_idx; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)w1_sf;
  p.sfa_ktiles = (int)(K / 128); p.sfb_ktiles = (int)(K / 128);
  p.z_fp8 = (uint8_t*)z_fp8; p.z_sc = (uint8_t*)z_scales; p.y1_fp8 = (uint8_t*)y1_fp8; p.y1_sf = (uint8_t*)y1_sf;
  p.status = status; p.debug_skip_store = g_skip_store;
  return run<GATED>(x_fp8, T, K, w1_fp8, E * N, K, p, (int)((rows / 128) * (N / 128)), (cudaStream_t)stream);
}

int64_t smoe_gemm_dgated_partials(int64_t N);

int smoe_gemm_dgated(const void* dout_fp8, int64_t T, const int* a_idx, const void* a_sf, const void* w2t_fp8,
                     const void* w2t_sf, const int* efo, const void* z_fp8, const void* z_scales, const float* s,
                     void* dz_bf16, void* y1s_bf16, float* ds_partial, int64_t* ds_partial_tiles, int64_t rows,
                     int64_t N, int64_t K, int64_t E, int* status, void* stream) {
  if (rows < 0 || rows % 128 || N % 128 || K % 128 || E <= 0 || T < 0) return SMOE_ERR_SHAPE;
  if (ds_partial_tiles) *ds_partial_tiles = smoe_gemm_dgated_partials(N);
  if (rows == 0) return SMOE_OK;
  if (T == 0) return SMOE_ERR_SHAPE;
  GemmParams p{};
  p.rows = (int)rows; p.N = (int)N; p.K = (int)K; p.E = (int)E;
  p.efo = efo; p.a_idx = a_idx; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)w2t_sf;
  p.sfa_ktiles = (int)(K / 128); p.sfb_ktiles = (int)(K / 128);
  p.z_fp8 = (uint8_t*)const_cast<void*>(z_fp8); p.z_sc = (uint8_t*)const_cast<void*>(z_scales);
  p.s = s; p.dz = dz_bf16; p.y1s = y1s_bf16; p.ds_partial = ds_partial; p.status = status;
  return run<DGATED>(dout_fp8, T, K, w2t_fp8, E * N, K, p, (int)((rows / 128) * (N / 128)), (cudaStream_t)stream);
}

static int dgated_fused_impl(const void* dout_fp8, int64_t a_rows, const int* a_idx, const void* a_sf,
                             const void* w2t_fp8, const void* w2t_sf, const int* efo, const void* z_fp8,
                             const void* z_scales, const float* s, void* dz_q, void* dz_row_sf, void* dz_col_sf,
                             void* y1s_q, void* y1s_col_sf, float* ds_partial, int64_t rows, int64_t N, int64_t K,
                             int64_t E, int* status, void* stream) {
  if (rows < 0 || rows % 128 || N % 128 || K % 128 || E <= 0) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  GemmParams p{};
  p.rows = (int)rows; p.N = (int)N; p.K = (int)K; p.E = (int)E;
  p.efo = efo; p.a_idx = a_idx; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)w2t_sf;
  p.sfa_ktiles = (int)(K / 128); p.sfb_ktiles = (int)(K / 128);
  p.z_fp8 = (uint8_t*)const_cast<void*>(z_fp8); p.z_sc = (uint8_t*)const_cast<void*>(z_scales);
  p.s = s; p.dz = dz_q; p.y1s = y1s_q; p.ds_partial = ds_partial; p.status = status;
  p.dz_row_sf = (uint8_t*)dz_row_sf; p.dz_col_sf = (uint8_t*)dz_col_sf; p.y1s_col_sf = (uint8_t*)y1s_col_sf;
  p.debug_skip_store = g_skip_store;
  return run<DGATEDQ>(dout_fp8, a_rows, K, w2t_fp8, E * N, K, p, (int)((rows / 128) * (N / 128)),
                      (cudaStream_t)stream);
}

int smoe_gemm_dgated_fused(const void* dout_fp8, const void* a_sf, const void* w2t_fp8, const void* w2t_sf,
                           const int* efo, const void* z_fp8, const void* z_scales, const float* s, void* dz_q,
                           void* dz_row_sf, void* dz_col_sf, void* y1s_q, void* y1s_col_sf, float* ds_partial,
                           int64_t rows, int64_t N, int64_t K, int64_t E, int* status, void* stream) {
  return dgated_fused_impl(dout_fp8, rows, nullptr, a_sf, w2t_fp8, w2t_sf, efo, z_fp8, z_scales, s, dz_q, dz_row_sf,
                           dz_col_sf, y1s_q, y1s_col_sf, ds_partial, rows, N, K, E, status, stream);
}

int smoe_gemm_dgated_fused_gather(const void* dout_fp8, int64_t T, const int* a_idx, const void* a_sf,
                                  const void* w2t_fp8, const void* w2t_sf, const int* efo, const void* z_fp8,
                                  const void* z_scales, const float* s, void* dz_q, void* dz_row_sf, void* dz_col_sf,
                                  void* y1s_q, void* y1s_col_sf, float* ds_partial, int64_t rows, int64_t N,
                                  int64_t K, int64_t E, int* status, void* stream) {
  if (rows > 0 && (T <= 0 || a_idx == nullptr)) return SMOE_ERR_ARG;
  return dgated_fused_impl(dout_fp8, T, a_idx, a_sf, w2t_fp8, w2t_sf, efo, z_fp8, z_scales, s, dz_q, dz_row_sf,
                           dz_col_sf, y1s_q, y1s_col_sf, ds_partial, rows, N, K, E, status, stream);
}

int64_t smoe_gemm_dgated_fused_partials(int64_t N) {
  const int bn = pick_bn2<DGATEDQ>(N);
  return (bn == 192 ? Gemm2Smem<192, DGATEDQ>::COL_GROUPS : Gemm2Smem<128, DGATEDQ>::COL_GROUPS) * ((N + bn - 1) / bn);
}

int64_t smoe_gemm_dgated_partials(int64_t N) {
  const int bn2 = pick_bn2<DGATED>(N);
  return bn2 ? 2 * (N / bn2) : N / pick_bn(N);
}

int smoe_gemm_wgrad(const void* a_t_fp8, const void* a_sf, const void* b_t_fp8, const void* b_sf, const int* efo,
                    float* c, int64_t M, int64_t N, int64_t TKp, int64_t E, int accumulate, int* status,
                    void* stream) {
  if (M <= 0 || N <= 0 || M % 128 || N % 128 || TKp < 0 || TKp % 128 || E <= 0) return SMOE_ERR_SHAPE;
  if (TKp == 0) return wgrad_nothing_routed(c, M, N, E, accumulate, (cudaStream_t)stream);
  GemmParams p{};
  p.rows = (int)M; p.N = (int)N; p.K = (int)TKp; p.E = (int)E;
  p.efo = efo; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)b_sf;
  p.sfa_ktiles = (int)(TKp / 128); p.sfb_ktiles = (int)(TKp / 128);
  p.c = c; p.accumulate = accumulate; p.status = status; p.debug_skip_store = g_skip_store;
  return run<WGRAD>(a_t_fp8, M, TKp, b_t_fp8, N, TKp, p, (int)(E * (M / 128) * (N / 128)), (cudaStream_t)stream);
}

int smoe_gemm_wgrad_mn(const void* a_fp8, const void* a_sf, const void* b_fp8, const void* b_sf, const int* efo,
                       float* c, int64_t M, int64_t N, int64_t TKp, int64_t E, int accumulate, int layout,
                       int* status, void* stream) {
  if (M <= 0 || N <= 0 || M % 256 || N % 256 || TKp < 0 || TKp % 128 || E <= 0 || (layout & ~3)) return SMOE_ERR_SHAPE;
  if (TKp == 0) return wgrad_nothing_routed(c, M, N, E, accumulate, (cudaStream_t)stream);
  GemmParams p{};
  p.rows = (int)M; p.N = (int)N; p.K = (int)TKp; p.E = (int)E;
  p.efo = efo; p.sfa = (const uint8_t*)a_sf; p.sfb = (const uint8_t*)b_sf;
  p.sfa_ktiles = (int)(TKp / 128); p.sfb_ktiles = (int)(TKp / 128);
  p.c = c; p.accumulate = accumulate; p.status = status; p.debug_skip_store = g_skip_store;
  p.a_mn = layout & 1; p.b_mn = (layout >> 1) & 1;
  return run<WGRAD>(a_fp8, p.a_mn ? TKp : M, p.a_mn ? M : TKp, b_fp8, p.b_mn ? TKp : N, p.b_mn ? N : TKp, p,
                    (int)(E * (M / 128) * (N / 128)), (cudaStream_t)stream);
}

/* dw_1 (+)= A1^T B1 and dw_2 (+)= A2^T B2 in one launch; see the header. */
int smoe_gemm_wgrad_mn_pair(const void* a1_fp8, const void* a1_sf, const void* b1_fp8, const void* b1_sf, float* c1,
                            int64_t M1, const void* a2_fp8, const void* a2_sf, const void* b2_fp8, const void* b2_sf,
                            float* c2, int64_t M2, const int* efo, int64_t N, int64_t TKp, int64_t E, int accumulate,
                            int a_rows_major_tk, int* status, void* stream) {
  if (M1 <= 0 || M2 <= 0 || N <= 0 || M1 % 256 || M2 % 256 || N % kBN3 || TKp < 0 || TKp % 128 || E <= 0 ||
      E > kMaxExperts2)
    return SMOE_ERR_SHAPE;
  if (g_force_v1 || (g_force_bn != 0 && g_force_bn != kBN3)) return SMOE_ERR_SHAPE;   // the tests' tile forcing
  if (TKp == 0) {
    const int rc = wgrad_nothing_routed(c1, M1, N, E, accumulate, (cudaStream_t)stream);
    return rc ? rc : wgrad_nothing_routed(c2, M2, N, E, accumulate, (cudaStream_t)stream);
  }
  GemmParams p{};
  p.rows = (int)M1; p.rows2 = (int)M2; p.N = (int)N; p.K = (int)TKp; p.E = (int)E;
  p.efo = efo; p.sfa = (const uint8_t*)a1_sf; p.sfb = (const uint8_t*)b1_sf;
  p.sfa_ktiles = (int)(TKp / 128); p.sfb_ktiles = (int)(TKp / 128);
  p.c = c1; p.c2 = c2; p.accumulate = accumulate; p.status = status; p.debug_skip_store = g_skip_store;
  p.a_mn = a_rows_major_tk ? 1 : 0;
  return run3_wgrad_pair(a1_fp8, b1_fp8, p, a2_fp8, b2_fp8, (const uint8_t*)a2_sf, (const uint8_t*)b2_sf, TKp,
                         (cudaStream_t)stream);
}

}  // extern "C"
