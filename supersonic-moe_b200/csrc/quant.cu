// MXFP8 1x32 ue8m0 block-scaled quantizers (HBM-bound; 128-bit global accesses,
// warp-shuffle amax, 32-bit packed scale stores).
//
// Rule for one group of 32 values (amax = max |v|):
//   e8m0 = max(bexp(amax) - 8 + (mantissa(amax) > 0x600000), 0), 0 for zero/denormal amax
//   q    = cvt.rn.satfinite.e4m3( v * 2^(127 - e8m0) )
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

__device__ __forceinline__ int q_e8m0_of(float amax) {
  const int bits = __float_as_int(amax);
  const int bexp = (bits >> 23) & 0xFF;
  const int e = bexp - 8 + ((bits & 0x7FFFFF) > 0x600000 ? 1 : 0);
  return bexp > 0 ? max(e, 0) : 0;
}
__device__ __forceinline__ float q_scale_of(int e8m0) {
  return __int_as_float(min(max(254 - e8m0, 1), 254) << 23);
}
__device__ __forceinline__ uint32_t q_pack4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ size_t isa_offset(size_t row, size_t g, size_t k_tiles) {
  return ((row >> 7) * k_tiles + (g >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (g & 3);
}

// --------------------------------------------------------------------- rows
// One warp per row; a lane owns 8 consecutive values, 4 lanes form a group.
__global__ void __launch_bounds__(256)
quant_rows_kernel(const uint4* __restrict__ x, int64_t M, int K, uint2* __restrict__ q, uint8_t* __restrict__ raw,
                  uint8_t* __restrict__ isa, const int* __restrict__ idx, const int* __restrict__ valid_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
  const int groups = K / 32, k_tiles = (K + 127) / 128;
  // with idx: output row `row` is the quantised source row idx[row] (gather fused into the quantizer);
  // rows at or beyond *valid_rows (over-allocated tail) are skipped
  const int64_t m_end = valid_rows ? min((int64_t)*valid_rows, M) : M;
  for (int64_t row = warp0; row < m_end; row += nwarps) {
    const int64_t srow = idx ? idx[row] : row;
    for (int c0 = 0; c0 < K; c0 += 256) {
      const int col = c0 + lane * 8;
      const bool in = col < K;
      float f[8];
      if (in) {
        bf16x8_to_f32(x[(srow * K + col) >> 3], f);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.f;
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, 2));
      const int e = q_e8m0_of(amax);
      const float qs = q_scale_of(e);
      if (in) {
        uint2 o;
        o.x = q_pack4(f[0] * qs, f[1] * qs, f[2] * qs, f[3] * qs);
        o.y = q_pack4(f[4] * qs, f[5] * qs, f[6] * qs, f[7] * qs);
        q[(row * K + col) >> 3] = o;
      }
      // gather the 4 group bytes of a 128-column tile into one word (lanes 0 and 16)
      const uint32_t b1 = __shfl_down_sync(0xffffffff, (uint32_t)e, 4);
      const uint32_t b2 = __shfl_down_sync(0xffffffff, (uint32_t)e, 8);
      const uint32_t b3 = __shfl_down_sync(0xffffffff, (uint32_t)e, 12);
      const int g = col >> 5;
      if (in && (lane & 15) == 0) {
        const uint32_t word = (uint32_t)e | (b1 << 8) | (b2 << 16) | (b3 << 24);
        if (g + 3 < groups) {
          if (raw) *reinterpret_cast<uint32_t*>(raw + row * groups + g) = word;
          if (isa) *reinterpret_cast<uint32_t*>(isa + isa_offset(row, g, k_tiles)) = word;
        } else {
          for (int j = 0; g + j < groups; ++j) {
            const uint8_t b = (uint8_t)(word >> (8 * j));
            if (raw) raw[row * groups + g + j] = b;
            if (isa) isa[isa_offset(row, g + j, k_tiles)] = b;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------- rows, scatter form
// Each token row is read and quantised ONCE and written to every expert-sorted position it occupies
// (positions s_rev[naept[t] .. naept[t+1])): HBM traffic = one read of x + the gathered output, instead of
// re-reading a token once per selected expert.  Pad rows (s_scatter[row] >= real_TK) are zero-filled so that
// the GEMM consuming the buffer only ever sees finite values.
// Blocks [0, token_blocks): one warp per token, row staged in shared memory; the remaining blocks clear pad rows.
__global__ void __launch_bounds__(256)
quant_rows_scatter_kernel(const uint4* __restrict__ x, int64_t T, int K, const int* __restrict__ naept,
                          const int* __restrict__ s_rev, const int* __restrict__ s_scatter,
                          const int* __restrict__ valid_rows, int64_t rows, uint4* __restrict__ q,
                          uint8_t* __restrict__ isa, int token_blocks) {
  extern __shared__ __align__(16) uint8_t s_rowbuf[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int k_tiles = K >> 7, k16 = K >> 4;
  if ((int)blockIdx.x < token_blocks) {
    const int64_t t = (int64_t)blockIdx.x * nw + warp;
    if (t >= T) return;
    const int beg = naept[t], end = naept[t + 1];
    if (beg == end) return;
    uint8_t* sq = s_rowbuf + (size_t)warp * ((K + 4 * k_tiles + 15) & ~15);   // 16-byte aligned per warp
    uint32_t* ssc = reinterpret_cast<uint32_t*>(sq + K);
    constexpr int NB = 4;                       // 16-byte loads in flight per lane
    for (int cb = 0; cb < K; cb += 256 * NB) {
      uint4 v[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int col = cb + b * 256 + lane * 8;
        v[b] = col < K ? x[(t * K + col) >> 3] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int col = cb + b * 256 + lane * 8;
        const bool in = col < K;
        float f[8];
        bf16x8_to_f32(v[b], f);
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, 2));
        const int e = q_e8m0_of(amax);
        const float qs = q_scale_of(e);
        const uint32_t b1 = __shfl_down_sync(0xffffffff, (uint32_t)e, 4);
        const uint32_t b2 = __shfl_down_sync(0xffffffff, (uint32_t)e, 8);
        const uint32_t b3 = __shfl_down_sync(0xffffffff, (uint32_t)e, 12);
        if (in) {
          uint2 o;
          o.x = q_pack4(f[0] * qs, f[1] * qs, f[2] * qs, f[3] * qs);
          o.y = q_pack4(f[4] * qs, f[5] * qs, f[6] * qs, f[7] * qs);
          *reinterpret_cast<uint2*>(sq + col) = o;
          if ((lane & 15) == 0) ssc[col >> 7] = (uint32_t)e | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
      }
    }
    __syncwarp();
    for (int j = beg; j < end; ++j) {
      const int64_t pos = s_rev[j];
      for (int c = lane; c < k16; c += 32) q[pos * k16 + c] = reinterpret_cast<const uint4*>(sq)[c];
      for (int kt = lane; kt < k_tiles; kt += 32)
        *reinterpret_cast<uint32_t*>(isa + isa_offset(pos, (size_t)kt * 4, k_tiles)) = ssc[kt];
    }
  } else {
    const int real_tk = naept[T];
    const int64_t m_end = valid_rows ? min((int64_t)*valid_rows, rows) : rows;
    const int64_t w0 = (int64_t)(blockIdx.x - token_blocks) * nw + warp;
    const int64_t nwarps = (int64_t)(gridDim.x - token_blocks) * nw;
    for (int64_t row = w0; row < m_end; row += nwarps) {
      if (s_scatter[row] < real_tk) continue;
      for (int c = lane; c < k16; c += 32) q[row * k16 + c] = make_uint4(0, 0, 0, 0);
      for (int kt = lane; kt < k_tiles; kt += 32)
        *reinterpret_cast<uint32_t*>(isa + isa_offset(row, (size_t)kt * 4, k_tiles)) = 0u;
    }
  }
}

// ------------------------------------------------------------- scale gather
__global__ void __launch_bounds__(256)
gather_scales_isa_kernel(const uint8_t* __restrict__ raw, const int* __restrict__ idx, int64_t rows, int groups,
                         int k_tiles, uint8_t* __restrict__ isa) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= rows * k_tiles) return;
  const int64_t row = i / k_tiles;
  const int kt = (int)(i - row * k_tiles);
  const int64_t src = idx ? idx[row] : row;
  uint32_t word;
  if (kt * 4 + 3 < groups && (groups & 3) == 0) {
    word = *reinterpret_cast<const uint32_t*>(raw + src * groups + kt * 4);
  } else {
    word = 0x7F7F7F7Fu;
    for (int j = 0; kt * 4 + j < groups && j < 4; ++j)
      word = (word & ~(0xFFu << (8 * j))) | ((uint32_t)raw[src * groups + kt * 4 + j] << (8 * j));
  }
  *reinterpret_cast<uint32_t*>(isa + isa_offset(row, (size_t)kt * 4, k_tiles)) = word;
}

// ------------------------------------------------------------- row gather
// out[r, :] = q[idx[r], :] (e4m3 bytes) and the row's scales into the ISA layout of (rows, K).
// One block per output row; rows at or beyond *valid_rows (over-allocated tail) are skipped.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ q, const uint8_t* __restrict__ raw, const int* __restrict__ idx,
                   const int* __restrict__ valid_rows, int K, uint4* __restrict__ out, uint8_t* __restrict__ isa) {
  const int64_t row = blockIdx.x;
  if (valid_rows && row >= *valid_rows) return;
  const int64_t src = idx[row];
  const int k16 = K >> 4, groups = K >> 5, k_tiles = K >> 7;
  for (int c = threadIdx.x; c < k16; c += blockDim.x) out[row * k16 + c] = q[src * k16 + c];
  for (int kt = threadIdx.x; kt < k_tiles; kt += blockDim.x)
    *reinterpret_cast<uint32_t*>(isa + isa_offset(row, (size_t)kt * 4, k_tiles)) =
        *reinterpret_cast<const uint32_t*>(raw + src * groups + kt * 4);
}

// ------------------------------------------------------------- row scatter (already quantised rows)
// The scatter form of gather_rows_kernel: every source row (e4m3 bytes + raw 1x32 scales) is read once and written
// to each expert-sorted position it occupies, s_rev[naept[t] .. naept[t+1]); pad rows are zero-filled by the
// trailing blocks, as in quant_rows_scatter_kernel.  One warp per source row.
__global__ void __launch_bounds__(256)
scatter_rows_fp8_kernel(const uint4* __restrict__ q, const uint8_t* __restrict__ raw, int64_t T, int K,
                        const int* __restrict__ naept, const int* __restrict__ s_rev,
                        const int* __restrict__ s_scatter, const int* __restrict__ valid_rows, int64_t rows,
                        uint4* __restrict__ out, uint8_t* __restrict__ isa, int token_blocks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int k_tiles = K >> 7, k16 = K >> 4, groups = K >> 5;
  if ((int)blockIdx.x < token_blocks) {
    const int64_t t = (int64_t)blockIdx.x * nw + warp;
    if (t >= T) return;
    const int beg = naept[t], end = naept[t + 1];
    if (beg == end) return;
    for (int c0 = 0; c0 < k16; c0 += 32 * 4) {          // four 16-byte loads in flight per lane
      uint4 v[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int c = c0 + b * 32 + lane;
        v[b] = c < k16 ? q[t * k16 + c] : make_uint4(0, 0, 0, 0);
      }
      for (int j = beg; j < end; ++j) {
        const int64_t pos = s_rev[j];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int c = c0 + b * 32 + lane;
          if (c < k16) out[pos * k16 + c] = v[b];
        }
      }
    }
    if (isa == nullptr) return;                          // payload only: the caller already holds the packed scales
    for (int kt = lane; kt < k_tiles; kt += 32) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(raw + t * groups + kt * 4);
      for (int j = beg; j < end; ++j)
        *reinterpret_cast<uint32_t*>(isa + isa_offset((size_t)s_rev[j], (size_t)kt * 4, k_tiles)) = word;
    }
  } else {
    const int real_tk = naept[T];
    const int64_t m_end = valid_rows ? min((int64_t)*valid_rows, rows) : rows;
    const int64_t w0 = (int64_t)(blockIdx.x - token_blocks) * nw + warp;
    const int64_t nwarps = (int64_t)(gridDim.x - token_blocks) * nw;
    for (int64_t row = w0; row < m_end; row += nwarps) {
      if (s_scatter[row] < real_tk) continue;
      for (int c = lane; c < k16; c += 32) out[row * k16 + c] = make_uint4(0, 0, 0, 0);
      if (isa == nullptr) continue;
      for (int kt = lane; kt < k_tiles; kt += 32)
        *reinterpret_cast<uint32_t*>(isa + isa_offset(row, (size_t)kt * 4, k_tiles)) = 0u;
    }
  }
}

// ------------------------------------------------------------------ byte transpose
// dst[b][c][r] = src[b][r][c] for a batch of [rows, cols] byte matrices, 64 x 64 tiles through shared memory.  With
// one scale per 32x32 block the transposed bytes of an e4m3 matrix ARE its transposed quantisation.
__global__ void __launch_bounds__(256)
transpose_u8_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int rows, int cols) {
  __shared__ __align__(16) uint8_t s[64][64 + 16];
  const size_t base = (size_t)blockIdx.z * rows * cols;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tr = threadIdx.x >> 2, seg = (threadIdx.x & 3) * 16;
  *reinterpret_cast<uint4*>(&s[tr][seg]) =
      *reinterpret_cast<const uint4*>(src + base + (size_t)(r0 + tr) * cols + c0 + seg);
  __syncthreads();
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = (uint32_t)s[seg + 4 * i][tr] | ((uint32_t)s[seg + 4 * i + 1][tr] << 8) |
           ((uint32_t)s[seg + 4 * i + 2][tr] << 16) | ((uint32_t)s[seg + 4 * i + 3][tr] << 24);
  *reinterpret_cast<uint4*>(dst + base + (size_t)(c0 + tr) * rows + r0 + seg) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ------------------------------------------------------------------ columns
// Tile = 128 rows x 64 columns of src[idx].  Groups run down the rows; the
// e4m3 bytes are written transposed ([dim, rows]) so that the reduction
// dimension of the weight-gradient GEMM is contiguous.
constexpr int CT_ROWS = 128, CT_COLS = 64, CT_PITCH = CT_COLS + 2;

// ISO: one scale per 32x32 block (also emits the non-transposed bytes and the
// row-direction scales); otherwise one scale per (column, 32 rows).
// SRC_FP8: the source is e4m3 bytes with raw row-wise 1x32 scales (`src_scales`, [T, dim/32]); it is
// dequantised exactly (an e4m3 value times a power of two fits bf16) and re-quantised column-wise.
template <bool ISO, bool SRC_FP8>
__global__ void __launch_bounds__(256)
quant_cols_kernel(const void* __restrict__ src_, const uint8_t* __restrict__ src_scales,
                  const int* __restrict__ idx, int64_t rows, int dim, uint8_t* __restrict__ q_t,
                  uint8_t* __restrict__ col_isa, uint8_t* __restrict__ q, uint8_t* __restrict__ row_isa,
                  const int* __restrict__ valid_rows) {
  __shared__ __nv_bfloat16 s_in[CT_ROWS][CT_PITCH];
  __shared__ __align__(16) uint8_t s_out[CT_COLS][CT_ROWS + 16];
  __shared__ uint32_t s_sc[CT_COLS];
  const int tid = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * CT_ROWS;
  // buffers sized at an upper bound: row tiles beyond the last expert's segment are never read by any GEMM
  if (valid_rows != nullptr && r0 >= *valid_rows) return;
  const int c0 = blockIdx.y * CT_COLS;
  const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(src_);

  if (SRC_FP8) {
    // 4 threads x 16 bytes cover one 64-column row; 64 rows per pass
    const uint8_t* src8 = reinterpret_cast<const uint8_t*>(src_);
    const int rr = tid >> 2, cc = (tid & 3) * 16;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int r = pass * 64 + rr;
      const int64_t srow = idx ? idx[r0 + r] : (r0 + r);
      const uint4 v = *reinterpret_cast<const uint4*>(src8 + srow * dim + c0 + cc);
      const float sc = __int_as_float((int)src_scales[srow * (dim >> 5) + ((c0 + cc) >> 5)] << 23);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t h2;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)(w[i >> 1] >> (16 * (i & 1)))));
        s_in[r][cc + 2 * i] = __float2bfloat16_rn(__half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF))) * sc);
        s_in[r][cc + 2 * i + 1] = __float2bfloat16_rn(__half2float(__ushort_as_half((unsigned short)(h2 >> 16))) * sc);
      }
    }
  } else {
    // load: 8 threads x 16 bytes cover one 64-column row; 32 rows per pass
    const int rr = tid >> 3, cc = (tid & 7) * 8;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int r = pass * 32 + rr;
      const int64_t srow = idx ? idx[r0 + r] : (r0 + r);
      const uint4 v = *reinterpret_cast<const uint4*>(src + srow * dim + c0 + cc);
      uint32_t* d = reinterpret_cast<uint32_t*>(&s_in[r][cc]);
      d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    }
  }
  __syncthreads();

  const int c = tid & 63, g = tid >> 6;        // column, 32-row group
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __bfloat162float(s_in[g * 32 + i][c]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  if (ISO) {  // block amax over the 32 columns of this warp
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffff, amax, d));
  }
  const int e = q_e8m0_of(amax);
  const float qs = q_scale_of(e);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = q_pack4(v[4 * i] * qs, v[4 * i + 1] * qs, v[4 * i + 2] * qs, v[4 * i + 3] * qs);
  uint4* so = reinterpret_cast<uint4*>(&s_out[c][g * 32]);
  so[0] = make_uint4(w[0], w[1], w[2], w[3]);
  so[1] = make_uint4(w[4], w[5], w[6], w[7]);
  if (g == 0) s_sc[c] = 0;
  __syncthreads();
  atomicOr(&s_sc[c], (uint32_t)e << (8 * g));   // distinct bits per thread: order-free
  __syncthreads();

  // transposed bytes: 8 threads x 16 bytes cover one 128-byte row of s_out (skipped when the caller of the 32x32
  // form wants the row-major payload only)
  if (!ISO || q_t != nullptr) {
    const int cc = tid >> 3, seg = (tid & 7) * 16;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int col = pass * 32 + cc;
      *reinterpret_cast<uint4*>(q_t + (size_t)(c0 + col) * rows + r0 + seg) =
          *reinterpret_cast<const uint4*>(&s_out[col][seg]);
    }
  }
  // column scales: logical operand (dim, rows); one word = the 4 groups of this 128-row tile
  if (tid < CT_COLS) {
    const size_t col = c0 + tid;
    *reinterpret_cast<uint32_t*>(col_isa + isa_offset(col, (size_t)(r0 >> 5), (size_t)(rows >> 7))) = s_sc[tid];
  }
  if (ISO) {
    // non-transposed bytes: thread -> (row, 32-byte half of the 64 columns)
    const int r = tid >> 1, h = tid & 1;
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int cc = h * 32 + i * 4;
      o[i] = (uint32_t)s_out[cc][r] | ((uint32_t)s_out[cc + 1][r] << 8) | ((uint32_t)s_out[cc + 2][r] << 16) |
             ((uint32_t)s_out[cc + 3][r] << 24);
    }
    uint4* dst = reinterpret_cast<uint4*>(q + (size_t)(r0 + r) * dim + c0 + h * 32);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    // row scales: logical operand (rows, dim); this tile holds groups c0/32 and c0/32+1 of 128 rows
    if (tid < CT_ROWS) {
      const size_t row = r0 + tid;
      const int gr = tid >> 5;
      const int k_tiles = dim >> 7;
      const int g0 = c0 >> 5;
      const uint8_t b0 = (uint8_t)(s_sc[0] >> (8 * gr));
      const uint8_t b1 = (uint8_t)(s_sc[32] >> (8 * gr));
      *reinterpret_cast<uint16_t*>(row_isa + isa_offset(row, g0, k_tiles)) = (uint16_t)b0 | ((uint16_t)b1 << 8);
    }
  }
}

}  // namespace smoe

using namespace smoe;

// ------------------------------------------------- gathered rows, both directions
// One warp owns 32 consecutive expert-sorted rows x 256 columns (a lane: 8 columns of every row, 32 x 16-byte
// loads in flight).  Column scales (one per column and 32 rows) need no communication at all, row scales
// (one per row and 32 columns) two shuffles per row.  Both payloads leave row-major: the column-scaled one is a
// weight-gradient operand read MN-major by the tensor core, so no transposed copy is written.
template <bool WITH_ROWS>
__global__ void __launch_bounds__(128)
quant_dual_kernel(const uint4* __restrict__ x, const int* __restrict__ idx, const int* __restrict__ valid_rows,
                  int64_t rows, int K, uint2* __restrict__ q_row, uint8_t* __restrict__ row_isa,
                  uint2* __restrict__ q_col, uint8_t* __restrict__ col_isa) {
  const int lane = threadIdx.x & 31;
  const int64_t task = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int cbs = K >> 8;
  const int64_t rg = task / cbs;
  const int cb = (int)(task - rg * cbs);
  const int64_t r0 = rg * 32;
  int64_t limit = rows;
  if (valid_rows) limit = min(limit, (int64_t)*valid_rows);
  if (r0 >= limit) return;
  const int col0 = cb * 256 + lane * 8;
  const int64_t my_row = idx ? (int64_t)idx[r0 + lane] : r0 + lane;
  uint4 v[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int64_t srow = __shfl_sync(0xffffffff, my_row, r);
    v[r] = x[(srow * K + col0) >> 3];
  }
  float cam[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) cam[j] = 0.f;
  const size_t row_kt = (size_t)((K + 127) >> 7);
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    float f[8];
    bf16x8_to_f32(v[r], f);
    float ram = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      cam[j] = fmaxf(cam[j], fabsf(f[j]));
      ram = fmaxf(ram, fabsf(f[j]));
    }
    if (WITH_ROWS) {
      ram = fmaxf(ram, __shfl_xor_sync(0xffffffff, ram, 1));
      ram = fmaxf(ram, __shfl_xor_sync(0xffffffff, ram, 2));
      const int e = q_e8m0_of(ram);
      const float qs = q_scale_of(e);
      uint2 o;
      o.x = q_pack4(f[0] * qs, f[1] * qs, f[2] * qs, f[3] * qs);
      o.y = q_pack4(f[4] * qs, f[5] * qs, f[6] * qs, f[7] * qs);
      q_row[((r0 + r) * K + col0) >> 3] = o;
      if ((lane & 3) == 0) row_isa[isa_offset((size_t)(r0 + r), (size_t)(col0 >> 5), row_kt)] = (uint8_t)e;
    }
  }
  float qs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int e = q_e8m0_of(cam[j]);
    qs[j] = q_scale_of(e);
    col_isa[isa_offset((size_t)(col0 + j), (size_t)rg, (size_t)(rows >> 7))] = (uint8_t)e;
  }
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    float f[8];
    bf16x8_to_f32(v[r], f);
    uint2 o;
    o.x = q_pack4(f[0] * qs[0], f[1] * qs[1], f[2] * qs[2], f[3] * qs[3]);
    o.y = q_pack4(f[4] * qs[4], f[5] * qs[5], f[6] * qs[6], f[7] * qs[7]);
    q_col[((r0 + r) * K + col0) >> 3] = o;
  }
}


extern "C" {

int smoe_quant_rows(const void* x_bf16, int64_t M, int64_t K, void* q, void* raw_scales, void* isa_scales,
                    void* stream) {
  if (M < 0 || K <= 0 || K % 32) return SMOE_ERR_SHAPE;
  if (isa_scales && K % 128) return SMOE_ERR_SHAPE;
  if (K % 8 || ((uintptr_t)x_bf16 & 15) || ((uintptr_t)q & 7)) return SMOE_ERR_ALIGN;
  if (M == 0) return SMOE_OK;
  int64_t blocks = (M + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quant_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x_bf16, M, (int)K, (uint2*)q,
                                                                   (uint8_t*)raw_scales, (uint8_t*)isa_scales, nullptr,
                                                                   nullptr);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_quant_rows_scatter(const void* x_bf16, int64_t T, int64_t K, const int32_t* naept, const int32_t* s_rev,
                            const int32_t* s_scatter_idx, const int32_t* valid_rows, int64_t rows, void* q,
                            void* isa_scales, void* stream) {
  if (T < 0 || rows < 0 || K <= 0 || K % 128 || K > 16384) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (!naept || !s_rev || !s_scatter_idx || !isa_scales) return SMOE_ERR_ARG;
  if (((uintptr_t)x_bf16 & 15) || ((uintptr_t)q & 15)) return SMOE_ERR_ALIGN;
  const int row_bytes = (int)((K + 4 * (K / 128) + 15) & ~(int64_t)15);
  const int warps = row_bytes * 8 <= 48 * 1024 ? 8 : (row_bytes * 4 <= 48 * 1024 ? 4 : 2);
  const int token_blocks = (int)((T + warps - 1) / warps);
  int pad_blocks = (int)((rows + 63) / 64);
  if (pad_blocks > 296) pad_blocks = 296;
  quant_rows_scatter_kernel<<<token_blocks + pad_blocks, warps * 32, (size_t)warps * row_bytes,
                              (cudaStream_t)stream>>>((const uint4*)x_bf16, T, (int)K, naept, s_rev, s_scatter_idx,
                                                      valid_rows, rows, (uint4*)q, (uint8_t*)isa_scales, token_blocks);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_quant_rows_gather(const void* x_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t K,
                           void* q, void* isa_scales, void* stream) {
  if (rows < 0 || K <= 0 || K % 128) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (!idx || !isa_scales) return SMOE_ERR_ARG;
  if (((uintptr_t)x_bf16 & 15) || ((uintptr_t)q & 7)) return SMOE_ERR_ALIGN;
  int64_t blocks = (rows + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quant_rows_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const uint4*)x_bf16, rows, (int)K, (uint2*)q,
                                                                   nullptr, (uint8_t*)isa_scales, idx, valid_rows);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_gather_scales_isa(const void* raw_scales, const int32_t* idx, int64_t rows, int64_t cols, void* isa_scales,
                           void* stream) {
  if (rows < 0 || cols <= 0 || cols % 32) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  const int groups = (int)(cols / 32), k_tiles = (int)((cols + 127) / 128);
  const int64_t n = rows * k_tiles;
  gather_scales_isa_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)raw_scales, idx, rows, groups, k_tiles, (uint8_t*)isa_scales);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_gather_rows_fp8(const void* q, const void* raw_scales, const int32_t* idx, const int32_t* valid_rows,
                         int64_t rows, int64_t K, void* q_out, void* isa_out, void* stream) {
  if (rows < 0 || K <= 0 || K % 128) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (((uintptr_t)q & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)raw_scales & 3)) return SMOE_ERR_ALIGN;
  const int threads = K / 16 >= 256 ? 256 : (int)((K / 16 + 31) / 32 * 32);
  gather_rows_kernel<<<(unsigned)rows, threads, 0, (cudaStream_t)stream>>>(
      (const uint4*)q, (const uint8_t*)raw_scales, idx, valid_rows, (int)K, (uint4*)q_out, (uint8_t*)isa_out);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_quant_cols_t(const void* src_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t dim,
                      void* q_t, void* isa, void* stream) {
  if (rows < 0 || rows % 128 || dim <= 0 || dim % 64) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  dim3 grid((unsigned)(rows / CT_ROWS), (unsigned)(dim / CT_COLS));
  quant_cols_kernel<false, false><<<grid, 256, 0, (cudaStream_t)stream>>>(
      src_bf16, nullptr, idx, rows, (int)dim, (uint8_t*)q_t, (uint8_t*)isa, nullptr, nullptr, valid_rows);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_requant_cols_t(const void* src_fp8, const void* src_scales, const int32_t* idx, const int32_t* valid_rows,
                        int64_t rows, int64_t dim, void* q_t, void* isa, void* stream) {
  if (rows < 0 || rows % 128 || dim <= 0 || dim % 64) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (!src_scales) return SMOE_ERR_ARG;
  dim3 grid((unsigned)(rows / CT_ROWS), (unsigned)(dim / CT_COLS));
  quant_cols_kernel<false, true><<<grid, 256, 0, (cudaStream_t)stream>>>(
      src_fp8, (const uint8_t*)src_scales, idx, rows, (int)dim, (uint8_t*)q_t, (uint8_t*)isa, nullptr, nullptr,
      valid_rows);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_quant_iso32(const void* x_bf16, int64_t rows, int64_t cols, void* q, void* row_isa, void* q_t, void* col_isa,
                     void* stream) {
  if (rows < 0 || rows % 128 || cols <= 0 || cols % 128) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  dim3 grid((unsigned)(rows / CT_ROWS), (unsigned)(cols / CT_COLS));
  quant_cols_kernel<true, false><<<grid, 256, 0, (cudaStream_t)stream>>>(x_bf16, nullptr, nullptr, rows, (int)cols,
                                                                         (uint8_t*)q_t, (uint8_t*)col_isa, (uint8_t*)q,
                                                                         (uint8_t*)row_isa, nullptr);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_transpose_u8(const void* src, int64_t batch, int64_t rows, int64_t cols, void* dst, void* stream) {
  if (batch < 0 || rows < 0 || cols < 0 || rows % 64 || cols % 64 || batch > 65535) return SMOE_ERR_SHAPE;
  if (batch == 0 || rows == 0 || cols == 0) return SMOE_OK;
  if (!src || !dst) return SMOE_ERR_ARG;
  if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) return SMOE_ERR_ALIGN;
  dim3 grid((unsigned)(cols / 64), (unsigned)(rows / 64), (unsigned)batch);
  if (grid.y > 65535) return SMOE_ERR_SHAPE;
  transpose_u8_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)src, (uint8_t*)dst, (int)rows, (int)cols);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_quant_dual_gather(const void* x_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t K,
                           void* q_row, void* row_isa, void* q_col, void* col_isa, void* stream) {
  if (rows < 0 || rows % 128 || K <= 0 || K % 256) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (!q_col || !col_isa || ((q_row == nullptr) != (row_isa == nullptr))) return SMOE_ERR_ARG;
  const int64_t tasks = (rows / 32) * (K / 256);
  const unsigned blocks = (unsigned)((tasks + 3) / 4);
  if (q_row)
    quant_dual_kernel<true><<<blocks, 128, 0, (cudaStream_t)stream>>>(
        (const uint4*)x_bf16, idx, valid_rows, rows, (int)K, (uint2*)q_row, (uint8_t*)row_isa, (uint2*)q_col,
        (uint8_t*)col_isa);
  else
    quant_dual_kernel<false><<<blocks, 128, 0, (cudaStream_t)stream>>>(
        (const uint4*)x_bf16, idx, valid_rows, rows, (int)K, nullptr, nullptr, (uint2*)q_col, (uint8_t*)col_isa);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_scatter_rows_fp8(const void* q, const void* raw_scales, int64_t T, int64_t K, const int32_t* naept,
                          const int32_t* s_rev, const int32_t* s_scatter_idx, const int32_t* valid_rows, int64_t rows,
                          void* q_out, void* isa_out, void* stream) {
  if (T < 0 || rows < 0 || K <= 0 || K % 128) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;      // nothing routed: not an error, and the (empty) buffers may be null
  if (((uintptr_t)q & 15) || ((uintptr_t)q_out & 15) || ((uintptr_t)raw_scales & 3)) return SMOE_ERR_ALIGN;
  if (isa_out != nullptr && raw_scales == nullptr) return SMOE_ERR_ARG;
  const int token_blocks = (int)((T + 7) / 8);
  const int pad_blocks = 148;
  scatter_rows_fp8_kernel<<<(unsigned)(token_blocks + pad_blocks), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)q, (const uint8_t*)raw_scales, T, (int)K, naept, s_rev, s_scatter_idx, valid_rows, rows,
      (uint4*)q_out, (uint8_t*)isa_out, token_blocks);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"
