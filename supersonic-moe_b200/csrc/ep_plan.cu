// Expert-parallel dispatch planning: the two small kernels around the routing-metadata kernels that turn the
// top-k expert ids of this rank's tokens into the send order of an all-to-all dispatch.
//   1. ep_dest_kernel      idx [T,K] -> destination rank of every slot, duplicates within a token removed (a token
//                          travels once to a rank), plus the histogram of routed pairs per global expert
//   2. (routing metadata kernels with destination ranks in the role of experts: send order, per-rank offsets,
//      every token's copies)
//   3. ep_send_idx_kernel  per outgoing row: its destination rank and the K expert ids local to that rank (-1 for
//                          slots that live on another rank)
// Integer atomics only (a histogram): the results do not depend on scheduling.
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

__global__ void __launch_bounds__(256)
ep_dest_kernel(const int* __restrict__ idx, int64_t T, int K, int E, int El, int* __restrict__ dest_u,
               int* __restrict__ pairs) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int* row = idx + t * K;
  for (int k = 0; k < K; ++k) {
    const int e = row[k];
    int d = -1;
    if (e >= 0 && e < E) {
      atomicAdd(pairs + e, 1);
      d = e / El;
      for (int j = 0; j < k; ++j) {
        const int ej = row[j];
        if (ej >= 0 && ej < E && ej / El == d) { d = -1; break; }
      }
    }
    dest_u[t * K + k] = d;
  }
}

__global__ void __launch_bounds__(256)
ep_send_idx_kernel(const int* __restrict__ idx, const int* __restrict__ send_tok, const int* __restrict__ efo,
                   int64_t n_send, int K, int E, int El, int world, int* __restrict__ send_idx,
                   int* __restrict__ send_rank) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n_send || i >= efo[world]) return;            // n_send may be an upper bound: the real count is efo[world]
  int r = 0;
  while (r + 1 < world && efo[r + 1] <= i) ++r;          // rows of rank r: [efo[r], efo[r+1])
  send_rank[i] = r;
  const int* row = idx + (int64_t)send_tok[i] * K;
  for (int k = 0; k < K; ++k) {
    const int e = row[k];
    send_idx[i * K + k] = (e >= 0 && e < E && e / El == r) ? e - r * El : -1;
  }
}

}  // namespace smoe

extern "C" {

int smoe_ep_plan_dest(const int32_t* idx, int64_t T, int64_t K, int64_t E, int64_t world, int32_t* dest_u,
                      int32_t* pairs, void* stream) {
  if (T < 0 || K <= 0 || E <= 0 || world <= 0 || E % world) return SMOE_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(pairs, 0, sizeof(int32_t) * E, st) != cudaSuccess) return SMOE_ERR_LAUNCH;
  if (T == 0) return SMOE_OK;
  smoe::ep_dest_kernel<<<(unsigned)((T + 255) / 256), 256, 0, st>>>(idx, T, (int)K, (int)E, (int)(E / world), dest_u,
                                                                    pairs);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ep_plan_send_idx(const int32_t* idx, const int32_t* send_tok, const int32_t* efo, int64_t n_send, int64_t K,
                          int64_t E, int64_t world, int32_t* send_idx, int32_t* send_rank, void* stream) {
  if (n_send < 0 || K <= 0 || E <= 0 || world <= 0 || E % world) return SMOE_ERR_SHAPE;
  if (n_send == 0) return SMOE_OK;
  smoe::ep_send_idx_kernel<<<(unsigned)((n_send + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      idx, send_tok, efo, n_send, (int)K, (int)E, (int)(E / world), (int)world, send_idx, send_rank);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"
