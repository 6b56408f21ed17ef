// Token-side kernels: the top-k weighted gather-reduce ("combine"), the score
// gather to expert-sorted rows, the ds partial-sum/permute, and the router's
// top-k softmax forward/backward.  All reductions run in a fixed order, so two
// runs on the same inputs give the same bits.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

__device__ __forceinline__ void acc_bf16x8(const uint4& v, float w, float (&a)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a[2 * i] = fmaf(w, __uint_as_float(u[i] << 16), a[2 * i]);
    a[2 * i + 1] = fmaf(w, __uint_as_float(u[i] & 0xFFFF0000u), a[2 * i + 1]);
  }
}
__device__ __forceinline__ uint32_t cvt_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One block per token; a thread owns 8 consecutive columns (16-byte accesses).
// Lanes of the token are added in ascending order.
__global__ void __launch_bounds__(512)
combine_kernel(const uint4* __restrict__ y, const int* __restrict__ s_rev, const int* __restrict__ naept,
               const float* __restrict__ scores, uint4* __restrict__ out, int H8) {
  const int64_t t = blockIdx.x;
  const int beg = naept[t], end = naept[t + 1];
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int j = beg;
    for (; j + 4 <= end; j += 4) {
      uint4 v[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        v[u] = y[(int64_t)s_rev[j + u] * H8 + c];
        w[u] = scores ? scores[j + u] : 1.0f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc_bf16x8(v[u], w[u], a);
    }
    for (; j < end; ++j) acc_bf16x8(y[(int64_t)s_rev[j] * H8 + c], scores ? scores[j] : 1.0f, a);
    out[t * H8 + c] = make_uint4(cvt_bf16x2(a[0], a[1]), cvt_bf16x2(a[2], a[3]), cvt_bf16x2(a[4], a[5]),
                                 cvt_bf16x2(a[6], a[7]));
  }
}

__global__ void gather_scores_kernel(const float* __restrict__ scores, const int* __restrict__ s_scatter, int64_t rows,
                                     float* __restrict__ s) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < rows) s[i] = scores[s_scatter[i]];
}

// Entries at or beyond *real_tk (over-allocated tail) are written as 0 and never scattered.
__global__ void ds_finalize_kernel(const float* __restrict__ part, int partials, int64_t rows,
                                   const int* __restrict__ s_rev, int64_t TK, const int* __restrict__ real_tk,
                                   float* __restrict__ ds, const int* __restrict__ src_idx,
                                   float* __restrict__ scatter_out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= TK) return;
  float a = 0.f;
  const bool real = real_tk == nullptr || i < *real_tk;
  if (real) {
    const int64_t p = s_rev[i];
    for (int t = 0; t < partials; ++t) a += part[(int64_t)t * rows + p];
    if (scatter_out) scatter_out[src_idx[i]] = a;
  }
  if (ds) ds[i] = a;
}

// One warp per row: K rounds of arg-max (lowest index wins ties), then softmax
// over the K selected logits in fp32.  A NaN logit counts as -inf.  A row with
// fewer than K finite logits still gets K distinct, in-range indices: once the
// finite ones are used up, the lowest not-yet-selected index is taken with a
// score of exactly zero (all K scores are zero when nothing in the row is finite).
__global__ void __launch_bounds__(256)
topk_softmax_kernel(const float* __restrict__ logits, int64_t T, int E, int K, float* __restrict__ scores,
                    int* __restrict__ idx) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  constexpr int PER = 32;  // up to 1024 experts
  float v[PER];
  const int per = (E + 31) / 32;
  uint32_t open = 0;       // bit i: this lane's i-th expert exists and has not been selected yet
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    const bool in = (i < per && e < E);
    const float x = in ? logits[row * E + e] : -INFINITY;
    v[i] = (x != x) ? -INFINITY : x;
    if (in) open |= 1u << i;
  }
  float sel_v = 0.f;
  int sel_i = 0;
  float vmax = 0.f;
  for (int k = 0; k < K; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      if (i < per && ((open >> i) & 1u)) {
        const int e = i * 32 + lane;
        if (bi == 0x7fffffff || v[i] > bv) { bv = v[i]; bi = e; }
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffff, bv, d);
      const int oi = __shfl_xor_sync(0xffffffff, bi, d);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (k == 0) vmax = bv;
    if (lane == k) { sel_v = bv; sel_i = bi; }
    if ((bi & 31) == lane) open &= ~(1u << (bi >> 5));     // K <= E: an open slot always exists
  }
  float ex = (lane < K && sel_v != -INFINITY) ? expf(sel_v - vmax) : 0.f;
  float sum = ex;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffff, sum, d);
  if (lane < K) {
    scores[row * K + lane] = sum > 0.f ? ex / sum : 0.f;
    idx[row * K + lane] = sel_i;
  }
}

__global__ void __launch_bounds__(256)
topk_softmax_bwd_kernel(const float* __restrict__ scores, const int* __restrict__ idx, const float* __restrict__ ds,
                        int64_t T, int E, int K, float* __restrict__ dlogits) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  for (int e = lane; e < E; e += 32) dlogits[row * E + e] = 0.f;
  __syncwarp();
  const float s = lane < K ? scores[row * K + lane] : 0.f;
  const float g = lane < K ? ds[row * K + lane] : 0.f;
  float dot = s * g;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffff, dot, d);
  if (lane < K) {
    const int e = idx[row * K + lane];
    if (e >= 0 && e < E) dlogits[row * E + e] = s * (g - dot);     // an out-of-range index is ignored, never written
  }
}

// One thread copies the device status word into pinned, device-visible host memory: a kernel store instead of a
// device-to-host memcpy, so that it never queues behind large copies on a copy engine.
__global__ void status_post_kernel(const int* __restrict__ status, volatile int* host_word) { *host_word = *status; }

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_combine(const void* y_bf16, const int32_t* s_rev, const int32_t* naept, const float* scores, void* out_bf16,
                 int64_t T, int64_t H, void* stream) {
  if (T < 0 || H <= 0 || H % 8) return SMOE_ERR_SHAPE;
  if (((uintptr_t)y_bf16 & 15) || ((uintptr_t)out_bf16 & 15)) return SMOE_ERR_ALIGN;
  if (T == 0) return SMOE_OK;
  const int H8 = (int)(H / 8);
  int threads = H8 >= 512 ? 512 : ((H8 + 31) / 32) * 32;
  if (H8 > 256 && H8 < 512) threads = ((H8 + 31) / 32) * 32;
  combine_kernel<<<(unsigned)T, threads, 0, (cudaStream_t)stream>>>((const uint4*)y_bf16, s_rev, naept, scores,
                                                                    (uint4*)out_bf16, H8);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_gather_scores(const float* scores, const int32_t* s_scatter_idx, int64_t rows, float* s, void* stream) {
  if (rows <= 0) return rows == 0 ? SMOE_OK : SMOE_ERR_SHAPE;
  gather_scores_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, (cudaStream_t)stream>>>(scores, s_scatter_idx, rows,
                                                                                         s);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ds_finalize(const float* ds_partial, int64_t partials, int64_t rows, const int32_t* s_rev, int64_t TK,
                     const int32_t* real_tk, float* ds_tm, const int32_t* src_idx, float* scatter_out, void* stream) {
  if (TK <= 0) return TK == 0 ? SMOE_OK : SMOE_ERR_SHAPE;
  if (scatter_out && !src_idx) return SMOE_ERR_ARG;
  ds_finalize_kernel<<<(unsigned)((TK + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      ds_partial, (int)partials, rows, s_rev, TK, real_tk, ds_tm, src_idx, scatter_out);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_status_post(const int32_t* status, int32_t* pinned_host_word, void* stream) {
  if (!status || !pinned_host_word) return SMOE_ERR_ARG;
  status_post_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(status, pinned_host_word);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_topk_softmax(const float* logits, int64_t T, int64_t E, int64_t K, float* scores, int32_t* idx,
                      void* stream) {
  if (T < 0 || E <= 0 || E > 1024 || K <= 0 || K > 32 || K > E) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  topk_softmax_kernel<<<(unsigned)((T + 7) / 8), 256, 0, (cudaStream_t)stream>>>(logits, T, (int)E, (int)K, scores,
                                                                                 idx);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_topk_softmax_bwd(const float* scores, const int32_t* idx, const float* dscores, int64_t T, int64_t E,
                          int64_t K, float* dlogits, void* stream) {
  if (T < 0 || E <= 0 || K <= 0 || K > 32) return SMOE_ERR_SHAPE;
  if (T == 0) return SMOE_OK;
  topk_softmax_bwd_kernel<<<(unsigned)((T + 7) / 8), 256, 0, (cudaStream_t)stream>>>(scores, idx, dscores, T, (int)E,
                                                                                     (int)K, dlogits);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"
