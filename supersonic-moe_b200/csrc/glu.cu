// Gated-linear-unit activations outside the GEMM epilogues, for the activations the fused epilogues do not carry
// (GEGLU, ReGLU): the up-projection then runs as a plain GEMM to bf16 z and these HBM-bound kernels do what the
// fused SwiGLU epilogues do - activation, z / y1 re-quantisation to MXFP8 in the forward; dequantised z, the
// activation's derivative, dz / y1s / ds in the backward.  Interleaved columns: z[:, 2j] = gate, z[:, 2j+1] = up.
// One warp per row; a lane owns 8 consecutive z columns (four gate/up pairs) of every 256-column pass.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

__device__ __forceinline__ int g_e8m0_of(float amax) {
  const int bits = __float_as_int(amax);
  const int bexp = (bits >> 23) & 0xFF;
  const int e = bexp - 8 + ((bits & 0x7FFFFF) > 0x600000 ? 1 : 0);
  return bexp > 0 ? max(e, 0) : 0;
}
__device__ __forceinline__ float g_scale_of(int e8m0) { return __int_as_float(min(max(254 - e8m0, 1), 254) << 23); }
__device__ __forceinline__ uint32_t g_pack4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ float g_bf16_rne(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ size_t g_isa_offset(size_t row, size_t g, size_t k_tiles) {
  return ((row >> 7) * k_tiles + (g >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (g & 3);
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t byte) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)byte));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF)));
}

constexpr float kGeluC0 = 0.7978845608028654f, kGeluC1 = 0.044715f;

// act: 0 = swiglu (g * sigmoid(g)), 1 = reglu (relu), 2 = geglu (tanh approximation of GELU)
__device__ __forceinline__ void act_and_slope(int act, float g, float& a, float& da) {
  if (act == 1) {
    a = fmaxf(g, 0.f);
    da = g > 0.f ? 1.f : 0.f;
  } else if (act == 2) {
    const float t = tanhf(kGeluC0 * (g + kGeluC1 * g * g * g));
    a = 0.5f * g * (1.f + t);
    da = 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * kGeluC0 * (1.f + 3.f * kGeluC1 * g * g);
  } else {
    const float sig = 1.f / (1.f + expf(-g));
    a = g * sig;
    da = sig * (1.f + g * (1.f - sig));
  }
}

// z bf16 [rows, 2I] -> z e4m3 + raw 1x32 scales (amax floor 1e-4, as the fused epilogue), y1 = bf16(act(g) * u)
// -> e4m3 + ISA scales for (rows, I).
__global__ void __launch_bounds__(256)
glu_fwd_kernel(const uint4* __restrict__ z, int64_t rows, int I, int act, uint2* __restrict__ z_q,
               uint8_t* __restrict__ z_sc, uint32_t* __restrict__ y1_q, uint8_t* __restrict__ y1_sf) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int N = 2 * I;
  const size_t y_kt = (size_t)((I + 127) >> 7);
  for (int c0 = 0; c0 < N; c0 += 256) {
    const int col = c0 + lane * 8;
    const bool in = col < N;
    float f[8];
    if (in) {
      const uint4 v = z[(row * N + col) >> 3];
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = 0.f;
    }
    // z: one scale per 32 columns = 4 lanes
    float zam = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) zam = fmaxf(zam, fabsf(f[i]));
    zam = fmaxf(zam, __shfl_xor_sync(0xffffffff, zam, 1));
    zam = fmaxf(zam, __shfl_xor_sync(0xffffffff, zam, 2));
    const int ze = g_e8m0_of(fmaxf(zam, 1e-4f));
    const float zs = g_scale_of(ze);
    // y1: four values per lane; one scale per 32 y1 columns = 64 z columns = 8 lanes
    float y[4], yam = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a, da;
      act_and_slope(act, f[2 * i], a, da);
      y[i] = g_bf16_rne(a * f[2 * i + 1]);
      yam = fmaxf(yam, fabsf(y[i]));
    }
    yam = fmaxf(yam, __shfl_xor_sync(0xffffffff, yam, 1));
    yam = fmaxf(yam, __shfl_xor_sync(0xffffffff, yam, 2));
    yam = fmaxf(yam, __shfl_xor_sync(0xffffffff, yam, 4));
    const int ye = g_e8m0_of(yam);
    const float ys = g_scale_of(ye);
    if (in) {
      uint2 o;
      o.x = g_pack4(f[0] * zs, f[1] * zs, f[2] * zs, f[3] * zs);
      o.y = g_pack4(f[4] * zs, f[5] * zs, f[6] * zs, f[7] * zs);
      z_q[(row * N + col) >> 3] = o;
      if ((lane & 3) == 0) z_sc[row * (N >> 5) + (col >> 5)] = (uint8_t)ze;
      y1_q[(row * I + (col >> 1)) >> 2] = g_pack4(y[0] * ys, y[1] * ys, y[2] * ys, y[3] * ys);
      if ((lane & 7) == 0) y1_sf[g_isa_offset((size_t)row, (size_t)(col >> 6), y_kt)] = (uint8_t)ye;
    }
  }
}

// D bf16 [rows, I] (= dout . W2 per expert), the saved e4m3 z with raw scales, the row's score s ->
// dz bf16 [rows, 2I] (interleaved dgate, dup), y1s = s * y bf16 [rows, I], ds[row] = sum_j y_j * D_j.
__global__ void __launch_bounds__(256)
glu_bwd_kernel(const uint2* __restrict__ D, const uint2* __restrict__ z_q, const uint8_t* __restrict__ z_sc,
               const float* __restrict__ s, int64_t rows, int I, int act, uint4* __restrict__ dz,
               uint2* __restrict__ y1s, float* __restrict__ ds) {
  const int lane = threadIdx.x & 31;
  const int64_t row = blockIdx.x * (int64_t)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int N = 2 * I;
  const float sr = s[row];
  float ds_acc = 0.f;
  for (int c0 = 0; c0 < N; c0 += 256) {
    const int col = c0 + lane * 8;       // first of this lane's 8 z columns; D / y1s columns col/2 .. col/2+3
    if (col < N) {
      const uint2 zq = z_q[(row * N + col) >> 3];
      const float zsc = __int_as_float((int)z_sc[row * (N >> 5) + (col >> 5)] << 23);
      const uint2 dv = D[(row * I + (col >> 1)) >> 2];
      const uint32_t zw[2] = {zq.x, zq.y}, dw[2] = {dv.x, dv.y};
      uint32_t o[4], yo[2];
      float ysv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float g = e4m3_to_f32((zw[i >> 1] >> (16 * (i & 1))) & 0xFF) * zsc;
        const float u = e4m3_to_f32((zw[i >> 1] >> (16 * (i & 1) + 8)) & 0xFF) * zsc;
        const float Dv = __uint_as_float((i & 1) ? (dw[i >> 1] & 0xFFFF0000u) : (dw[i >> 1] << 16));
        const float dout = sr * Dv;
        float a, da;
        act_and_slope(act, g, a, da);
        const float yv = a * u;
        ds_acc = fmaf(yv, Dv, ds_acc);
        const __nv_bfloat162 pr = __floats2bfloat162_rn(da * u * dout, a * dout);
        o[i] = *reinterpret_cast<const uint32_t*>(&pr);
        ysv[i] = sr * yv;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const __nv_bfloat162 pr = __floats2bfloat162_rn(ysv[2 * i], ysv[2 * i + 1]);
        yo[i] = *reinterpret_cast<const uint32_t*>(&pr);
      }
      dz[(row * N + col) >> 3] = make_uint4(o[0], o[1], o[2], o[3]);
      y1s[(row * I + (col >> 1)) >> 2] = make_uint2(yo[0], yo[1]);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) ds_acc += __shfl_xor_sync(0xffffffff, ds_acc, d);
  if (lane == 0) ds[row] = ds_acc;
}

}  // namespace smoe

using namespace smoe;

extern "C" {

int smoe_glu_fwd(const void* z_bf16, int64_t rows, int64_t I, int act, void* z_fp8, void* z_scales, void* y1_fp8,
                 void* y1_sf, void* stream) {
  if (rows < 0 || I <= 0 || I % 32 || act < 0 || act > 2) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  if (!z_bf16 || !z_fp8 || !z_scales || !y1_fp8 || !y1_sf) return SMOE_ERR_ARG;
  if (((uintptr_t)z_bf16 & 15) || ((uintptr_t)z_fp8 & 7) || ((uintptr_t)y1_fp8 & 3)) return SMOE_ERR_ALIGN;
  glu_fwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)z_bf16, rows, (int)I, act, (uint2*)z_fp8, (uint8_t*)z_scales, (uint32_t*)y1_fp8, (uint8_t*)y1_sf);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_glu_bwd(const void* d_bf16, const void* z_fp8, const void* z_scales, const float* s, int64_t rows, int64_t I,
                 int act, void* dz_bf16, void* y1s_bf16, float* ds_rows, void* stream) {
  if (rows < 0 || I <= 0 || I % 32 || act < 0 || act > 2) return SMOE_ERR_SHAPE;
  if (rows == 0) return SMOE_OK;
  if (!d_bf16 || !z_fp8 || !z_scales || !s || !dz_bf16 || !y1s_bf16 || !ds_rows) return SMOE_ERR_ARG;
  if (((uintptr_t)d_bf16 & 7) || ((uintptr_t)z_fp8 & 7) || ((uintptr_t)dz_bf16 & 15) || ((uintptr_t)y1s_bf16 & 7))
    return SMOE_ERR_ALIGN;
  glu_bwd_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
      (const uint2*)d_bf16, (const uint2*)z_fp8, (const uint8_t*)z_scales, s, rows, (int)I, act, (uint4*)dz_bf16,
      (uint2*)y1s_bf16, ds_rows);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"
