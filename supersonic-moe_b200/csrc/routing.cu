// Routing metadata for the MoE layer: count/cumsum of expert ids and the fused
// top-k -> padded expert-sorted layout.  Integer work, bit-exact by construction:
// no floating-point atomics, no order-dependent atomics (bit masks are built with
// atomicOr, whose result does not depend on arrival order).
//
// Layout of the work: rows are cut into units of 32 (one warp, one row per lane).
//   1. unit_masks_kernel  mask[u][e] = lanes of unit u whose row selects expert e;
//                         valid[u]   = number of valid (row, slot) pairs of the unit
//   2. scan_kernel        per expert: exclusive scan of popc(mask[.][e]) over units
//                         (rows of an expert keep ascending token order) + count[e];
//                         one more block scans valid[.] -> token-major bases, real_TK
//   3. scatter_fill_kernel recomputes the padded offsets in shared memory, writes
//                         every output, then fills pad rows and over-allocated tails
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

constexpr int kMaxTopk = 16;
constexpr int kRtThreads = 256;
constexpr int kUnitsPerBlock = kRtThreads / 32;

__device__ __forceinline__ int warp_excl_scan(int v, int lane) {
  int x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffff, x, d);
    if (lane >= d) x += y;
  }
  return x - v;
}

// Block-wide exclusive scan of n values produced by f(i), consumed by g(i, exclusive);
// returns the total.  Blocked partition: each thread owns a contiguous run.
template <typename F, typename G>
__device__ int block_excl_scan(int n, F f, G g, int* s_warp /* >= 33 ints */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const int chunk = (n + blockDim.x - 1) / blockDim.x;
  const int lo = min(tid * chunk, n), hi = min(lo + chunk, n);
  int part = 0;
  for (int i = lo; i < hi; ++i) part += f(i);
  const int wex = warp_excl_scan(part, lane);
  if (lane == 31) s_warp[warp] = wex + part;
  __syncthreads();
  if (warp == 0) {
    const int t = lane < nw ? s_warp[lane] : 0;
    const int ex = warp_excl_scan(t, lane);
    if (lane < nw) s_warp[lane] = ex;
    if (lane == 31) s_warp[32] = ex + t;
  }
  __syncthreads();
  int run = s_warp[warp] + wex;
  for (int i = lo; i < hi; ++i) {
    const int v = f(i);
    g(i, run);
    run += v;
  }
  const int total = s_warp[32];
  __syncthreads();
  return total;
}

// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kRtThreads)
unit_masks_kernel(const int* __restrict__ idx, int N, int K, int E, uint32_t* __restrict__ mask,
                  int* __restrict__ unit_valid) {
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * kUnitsPerBlock + (threadIdx.x >> 5);
  const int units = (N + 31) / 32;
  if (unit >= units) return;
  const int row = unit * 32 + lane;
  uint32_t* m = mask + (size_t)unit * E;
  for (int e = lane; e < E; e += 32) m[e] = 0u;
  __syncwarp();
  int nvalid = 0;
  if (row < N) {
    for (int k = 0; k < K; ++k) {
      const int e = idx[(size_t)row * K + k];
      if (e >= 0 && e < E) {
        atomicOr(&m[e], 1u << lane);
        ++nvalid;
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) nvalid += __shfl_xor_sync(0xffffffff, nvalid, d);
  if (lane == 0) unit_valid[unit] = nvalid;
}

// blocks [0, E): expert e -> unit_off[u][e] = exclusive scan over u of popc(mask[u][e]); counts[e] = total
// block  E     : unit_base[u] = exclusive scan of unit_valid; naept[N] = total
__global__ void __launch_bounds__(kRtThreads)
scan_kernel(const uint32_t* __restrict__ mask, const int* __restrict__ unit_valid, int units, int E, int N,
            int* __restrict__ unit_off, int* __restrict__ counts, int* __restrict__ unit_base,
            int* __restrict__ naept) {
  __shared__ int s_warp[33];
  const int e = blockIdx.x;
  if (e < E) {
    const int total = block_excl_scan(
        units, [&](int u) { return __popc(mask[(size_t)u * E + e]); },
        [&](int u, int ex) { unit_off[(size_t)u * E + e] = ex; }, s_warp);
    if (threadIdx.x == 0) counts[e] = total;
  } else {
    const int total = block_excl_scan(
        units, [&](int u) { return unit_valid[u]; }, [&](int u, int ex) { unit_base[u] = ex; }, s_warp);
    if (threadIdx.x == 0) naept[N] = total;
  }
}

__global__ void __launch_bounds__(kRtThreads)
scatter_fill_kernel(const int* __restrict__ idx, const float* __restrict__ probs, int N, int K, int E, int alignment,
                    int TK_alloc, int TKp_alloc, int lane_order, int pad_mode, const uint32_t* __restrict__ mask,
                    const int* __restrict__ unit_off, const int* __restrict__ unit_base,
                    const int* __restrict__ counts, int* __restrict__ efo_out, int* __restrict__ x_gather,
                    int* __restrict__ s_scatter, int* __restrict__ s_rev, int* __restrict__ naept,
                    float* __restrict__ scores, int* __restrict__ src_idx, int scatter_blocks) {
  extern __shared__ int s_mem[];
  int* s_efo = s_mem;              // [E+1] padded offsets
  int* s_base = s_mem + (E + 1);   // [E+1] unpadded offsets
  int* s_warp = s_base + (E + 1);  // [33]
  const int lane = threadIdx.x & 31;

  const int tot_p = block_excl_scan(
      E,
      [&](int e) {
        const int c = counts[e];
        return c > 0 ? (c + alignment - 1) / alignment * alignment : 0;
      },
      [&](int e, int ex) { s_efo[e] = ex; }, s_warp);
  const int tot_u = block_excl_scan(
      E, [&](int e) { return counts[e]; }, [&](int e, int ex) { s_base[e] = ex; }, s_warp);
  if (threadIdx.x == 0) {
    s_efo[E] = tot_p;
    s_base[E] = tot_u;
  }
  __syncthreads();
  // published offsets never point past the allocation (they can only exceed it when the caller sized the buffers
  // from counts that do not match idx): the GEMMs that walk efo then stay inside the buffers too
  if (blockIdx.x == 0)
    for (int e = threadIdx.x; e <= E; e += blockDim.x) efo_out[e] = min(s_efo[e], TKp_alloc / alignment * alignment);
  const int real_TK = tot_u;        // == naept[N]
  const int real_TKp = tot_p;

  // ---- scatter: one unit of 32 rows per warp ----
  if ((int)blockIdx.x < scatter_blocks) {
    const int unit = blockIdx.x * kUnitsPerBlock + (threadIdx.x >> 5);
    const int row = unit * 32 + lane;
    if (unit * 32 < N) {
      int ex[kMaxTopk];
      int nvalid = 0;
#pragma unroll
      for (int k = 0; k < kMaxTopk; ++k) {
        ex[k] = -1;
        if (k < K && row < N) {
          const int e = idx[(size_t)row * K + k];
          if (e >= 0 && e < E) { ex[k] = e; ++nvalid; }
        }
      }
      const int tm_base = unit_base[unit] + warp_excl_scan(nvalid, lane);
      if (row < N) {
        naept[row] = tm_base;
        int slot_rank = 0;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
          if (k < K && ex[k] >= 0) {
            const int e = ex[k];
            const uint32_t m = mask[(size_t)unit * E + e];
            const int pos = s_efo[e] + unit_off[(size_t)unit * E + e] + __popc(m & ((1u << lane) - 1u));
            int rank;
            if (lane_order == 0) {
              rank = 0;
#pragma unroll
              for (int j = 0; j < kMaxTopk; ++j) rank += (j < K && ex[j] >= 0 && ex[j] < e) ? 1 : 0;
            } else {
              rank = slot_rank;
            }
            ++slot_rank;
            const int tm = tm_base + rank;
            // buffers sized from a caller's (possibly stale) per-expert counts may be too small for what the
            // indices really hold: the excess is dropped, never written past the allocation
            if (pos < TKp_alloc) {
              x_gather[pos] = row;
              s_scatter[pos] = tm;
            }
            if (tm < TK_alloc) {
              s_rev[tm] = pos < TKp_alloc ? pos : 0;
              src_idx[tm] = row * K + k;
            }
            if (tm < TKp_alloc) scores[tm] = probs[(size_t)row * K + k];
          }
        }
      }
    }
  }

  // ---- pad rows and over-allocated tails ----
  const int nthreads = gridDim.x * blockDim.x;
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x;
  for (int pos = gtid; pos < TKp_alloc; pos += nthreads) {
    if (pos >= real_TKp) {
      x_gather[pos] = 0;
      s_scatter[pos] = pad_mode == 0 ? real_TK : pos;   // virtual numbering continues through the tail
      continue;
    }
    int lo = 0, hi = E;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_efo[mid + 1] <= pos) lo = mid + 1; else hi = mid;
    }
    const int cnt = s_base[lo + 1] - s_base[lo];
    const int local = pos - s_efo[lo];
    if (local >= cnt) {
      x_gather[pos] = 0;
      s_scatter[pos] = pad_mode == 0 ? real_TK : real_TK + (s_efo[lo] - s_base[lo]) + (local - cnt);
    }
  }
  for (int i = real_TK + gtid; i < TKp_alloc; i += nthreads) scores[i] = 0.f;
  for (int i = real_TK + gtid; i < TK_alloc; i += nthreads) {
    s_rev[i] = 0;
    src_idx[i] = 0;
  }
}

// ---------------------------------------------------------------------------
template <typename T>
__global__ void count_kernel(const T* __restrict__ ids, int64_t n, int E, int* __restrict__ count) {
  extern __shared__ int s_cnt[];
  const bool use_smem = E <= 8192;
  if (use_smem) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
    __syncthreads();
  }
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = (int64_t)ids[i];
    if (e >= 0 && e < E) atomicAdd(use_smem ? &s_cnt[e] : &count[e], 1);
  }
  if (use_smem) {
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      if (s_cnt[e]) atomicAdd(&count[e], s_cnt[e]);
  }
}

__global__ void __launch_bounds__(kRtThreads)
cumsum_kernel(const int* __restrict__ count, int E, int* __restrict__ cumsum) {
  __shared__ int s_warp[33];
  block_excl_scan(E, [&](int e) { return count[e]; }, [&](int e, int ex) { cumsum[e] = ex + count[e]; }, s_warp);
}

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_count_cumsum(const void* ids, int ids_is_int64, int64_t n, int64_t E, int32_t* count, int32_t* cumsum,
                      void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (E <= 0 || n < 0 || !count) return SMOE_ERR_ARG;
  cudaMemsetAsync(count, 0, sizeof(int) * E, stream);
  if (n > 0) {
    const int threads = 512;
    int blocks = (int)((n + threads * 4 - 1) / (threads * 4));
    if (blocks > 592) blocks = 592;
    const size_t smem = E <= 8192 ? sizeof(int) * E : 0;
    if (ids_is_int64)
      count_kernel<int64_t><<<blocks, threads, smem, stream>>>((const int64_t*)ids, n, (int)E, count);
    else
      count_kernel<int32_t><<<blocks, threads, smem, stream>>>((const int32_t*)ids, n, (int)E, count);
  }
  if (cumsum) cumsum_kernel<<<1, kRtThreads, 0, stream>>>(count, (int)E, cumsum);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int64_t smoe_topk_metadata_workspace(int64_t N, int64_t E) {
  const int64_t units = (N + 31) / 32 + 1;
  return (units * E * 2 + units * 2 + 64) * 4;
}

int smoe_topk_metadata(const int32_t* idx, const float* probs, int64_t N, int64_t K, int64_t E, int64_t alignment,
                       int64_t TK_alloc, int64_t TKp_alloc, int lane_order, int pad_mode, int32_t* efo,
                       int32_t* x_gather_idx, int32_t* s_scatter_idx, int32_t* s_reverse_scatter_idx, int32_t* naept,
                       float* topk_scores, int32_t* score_src_idx, int32_t* counts, void* workspace, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (K <= 0 || K > kMaxTopk || E <= 0 || E > 4096 || N < 0 || alignment <= 0) return SMOE_ERR_SHAPE;
  if (N * K >= (int64_t)1 << 31 || TKp_alloc >= (int64_t)1 << 31) return SMOE_ERR_SHAPE;
  if (!workspace || !efo || !counts) return SMOE_ERR_ARG;
  const int units = (int)((N + 31) / 32);
  uint32_t* mask = (uint32_t*)workspace;
  int* unit_off = (int*)(mask + (size_t)(units + 1) * E);
  int* unit_valid = unit_off + (size_t)(units + 1) * E;
  int* unit_base = unit_valid + units + 1;
  const int ublocks = (units + kUnitsPerBlock - 1) / kUnitsPerBlock;
  if (ublocks > 0)
    unit_masks_kernel<<<ublocks, kRtThreads, 0, stream>>>(idx, (int)N, (int)K, (int)E, mask, unit_valid);
  scan_kernel<<<(int)E + 1, kRtThreads, 0, stream>>>(mask, unit_valid, units, (int)E, (int)N, unit_off, counts,
                                                     unit_base, naept);
  int fill_blocks = (int)((TKp_alloc + kRtThreads - 1) / kRtThreads);
  if (fill_blocks > 1184) fill_blocks = 1184;
  int grid = ublocks > fill_blocks ? ublocks : fill_blocks;
  if (grid < 1) grid = 1;
  const size_t smem = sizeof(int) * (2 * (E + 1) + 33);
  scatter_fill_kernel<<<grid, kRtThreads, smem, stream>>>(
      idx, probs, (int)N, (int)K, (int)E, (int)alignment, (int)TK_alloc, (int)TKp_alloc, lane_order, pad_mode, mask,
      unit_off, unit_base, counts, efo, x_gather_idx, s_scatter_idx, s_reverse_scatter_idx, naept, topk_scores,
      score_src_idx, ublocks);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// smoe_topk_metadata_static: the same routing-metadata computation for callers
// that must not allocate - code running inside a CUDA-graph capture or a stream
// callback, a serving loop that forbids cudaMalloc after start-up, a host
// framework whose allocator this library cannot reach.  The scratch that
// smoe_topk_metadata takes from its caller lives here in a fixed device array
// that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------
namespace smoe {

constexpr size_t kStaticScratchBytes = 1u << 20;   // 1 MiB: e.g. 16384 rows x 128 experts, or 65536 rows x 32
static __device__ __align__(256) unsigned char g_topk_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices] = {nullptr};   // device address of g_topk_scratch, per device

// In host code the array's name is only a handle; the address a kernel can use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SMOE_ERR_ARG;
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_topk_scratch) != cudaSuccess || p == nullptr) return SMOE_ERR_DRIVER;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SMOE_OK;
}

}  // namespace smoe

extern "C" {

int64_t smoe_topk_metadata_static_capacity(void) { return (int64_t)smoe::kStaticScratchBytes; }

int smoe_topk_metadata_static(const int32_t* idx, const float* probs, int64_t N, int64_t K, int64_t E,
                              int64_t alignment, int64_t TK_alloc, int64_t TKp_alloc, int lane_order, int pad_mode,
                              int32_t* efo, int32_t* x_gather_idx, int32_t* s_scatter_idx,
                              int32_t* s_reverse_scatter_idx, int32_t* naept, float* topk_scores,
                              int32_t* score_src_idx, int32_t* counts, void* stream) {
  if (N < 0 || E <= 0) return SMOE_ERR_SHAPE;
  // the scratch need grows with rows x experts; anything beyond the fixed array is refused, never truncated
  if (smoe_topk_metadata_workspace(N, E) > (int64_t)smoe::kStaticScratchBytes) return SMOE_ERR_SHAPE;
  void* scratch = nullptr;
  const int rc = smoe::static_scratch(&scratch);
  if (rc != SMOE_OK) return rc;
  // nothing in the scratch has to start at zero: the first kernel clears the bit masks it builds on, and every
  // other word is written before it is read, so the previous call's contents are harmless
  return smoe_topk_metadata(idx, probs, N, K, E, alignment, TK_alloc, TKp_alloc, lane_order, pad_mode, efo,
                            x_gather_idx, s_scatter_idx, s_reverse_scatter_idx, naept, topk_scores, score_src_idx,
                            counts, scratch, stream);
}

}  // extern "C"
