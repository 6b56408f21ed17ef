// Expert-parallel combine over NVLink peer memory: the return exchange and the reduction of a token's copies in ONE
// kernel.  Every rank leaves its partial outputs (one bf16 row per received token) in a buffer that all ranks of the
// node have mapped (symmetric memory); the source rank then reads the copies of each of its tokens straight from
// the owners' buffers with plain 16-byte loads and adds them in ascending rank order.  No receive buffer, no second
// pass.  The kernel waits on nothing: the host orders "all ranks have written" before it with a stream-ordered
// collective, so a rank that never arrives can at worst stall that collective, not this kernel.
#include <cuda_runtime.h>
#include <stdint.h>

#include "smoe_b200.h"

namespace smoe {

constexpr int kMaxPeers = 16;

struct PeerTable {
  const uint4* base[kMaxPeers];   // rank r's partial-output buffer, mapped into this process
  int first_row[kMaxPeers];       // row, in rank r's buffer, of this rank's first row sent to r
  int send_off[kMaxPeers];        // offset of rank r's segment in this rank's send order
};

__device__ __forceinline__ void acc8(const uint4& v, float (&a)[8]) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    a[2 * i] += __uint_as_float(u[i] << 16);
    a[2 * i + 1] += __uint_as_float(u[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint32_t bf16x2_of(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One block per token; a thread owns 8 consecutive columns.  copy_pos[copy_off[t] .. copy_off[t+1]) are the token's
// outgoing rows in ascending destination rank; row i of the send order went to send_rank[i] and sits there at
// first_row[rank] + (i - send_off[rank]).
__global__ void __launch_bounds__(512)
ep_combine_pull_kernel(PeerTable tab, const int* __restrict__ copy_pos, const int* __restrict__ copy_off,
                       const int* __restrict__ send_rank, uint4* __restrict__ out, int H8) {
  const int64_t t = blockIdx.x;
  const int beg = copy_off[t], end = copy_off[t + 1];
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int j = beg;
    for (; j + 4 <= end; j += 4) {       // four remote loads in flight
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = copy_pos[j + u];
        const int r = send_rank[i];
        v[u] = tab.base[r][(int64_t)(tab.first_row[r] + i - tab.send_off[r]) * H8 + c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc8(v[u], a);
    }
    for (; j < end; ++j) {
      const int i = copy_pos[j];
      const int r = send_rank[i];
      acc8(tab.base[r][(int64_t)(tab.first_row[r] + i - tab.send_off[r]) * H8 + c], a);
    }
    out[t * H8 + c] = make_uint4(bf16x2_of(a[0], a[1]), bf16x2_of(a[2], a[3]), bf16x2_of(a[4], a[5]),
                                 bf16x2_of(a[6], a[7]));
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Dispatch over peer memory: every rank leaves its quantised tokens (e4m3 [T,H] + raw 1x32 scales [T,H/32]), their
// probabilities [T,K] and its send lists (token and local expert ids of every outgoing row, grouped by destination
// rank) in a buffer all ranks have mapped; the destination then fetches the rows addressed to it straight from the
// sources, in the order an all-to-all would deliver them (sources ascending, each in its send order).  One warp per
// received row, plain 16-byte loads over NVLink, no staging copy of the outgoing rows, no wait inside the kernel.
struct PullTable {
  const uint8_t* base[kMaxPeers];   // rank s's buffer as mapped into this process
  int recv_off[kMaxPeers + 1];      // first received row that comes from rank s (prefix of the receive counts)
  int src_off[kMaxPeers];           // where the segment addressed to this rank starts in rank s's send order
};

struct PullLayout {                 // byte offsets inside every rank's buffer (the same on all ranks)
  int64_t q, raw, tok, idx, probs;
};

__global__ void __launch_bounds__(256)
ep_dispatch_pull_kernel(PullTable tab, PullLayout lay, int world, int H, int K, int n_recv, int rot,
                        uint4* __restrict__ q_out, uint32_t* __restrict__ raw_out, int* __restrict__ idx_out,
                        float* __restrict__ p_out) {
  const int lane = threadIdx.x & 31;
  // The grid walks the received rows starting at `rot` (the first row that comes from the NEXT rank) and wraps
  // around: rank r begins with source r+1, so at any moment the ranks read from different sources instead of all
  // draining rank 0's links first.
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_recv) return;
  row += rot;
  if (row >= n_recv) row -= n_recv;
  int s = 0;
  while (s + 1 < world && tab.recv_off[s + 1] <= row) ++s;
  const int64_t j = tab.src_off[s] + (row - tab.recv_off[s]);      // row of rank s's send order
  const uint8_t* base = tab.base[s];
  const int64_t tok = reinterpret_cast<const int*>(base + lay.tok)[j];
  const int h16 = H >> 4, words = H >> 7;                          // 16-byte pieces of a row; 4-byte scale words
  const uint4* src = reinterpret_cast<const uint4*>(base + lay.q) + tok * h16;
  uint4* dst = q_out + row * h16;
  for (int c0 = 0; c0 < h16; c0 += 32 * 8) {                       // eight remote loads in flight per lane
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u * 32 + lane;
      if (c < h16) v[u] = src[c];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u * 32 + lane;
      if (c < h16) dst[c] = v[u];
    }
  }
  const uint32_t* rsrc = reinterpret_cast<const uint32_t*>(base + lay.raw) + tok * words;
  for (int c = lane; c < words; c += 32) raw_out[row * words + c] = rsrc[c];
  if (idx_out != nullptr && lane < K) {
    idx_out[row * K + lane] = reinterpret_cast<const int*>(base + lay.idx)[j * K + lane];
    p_out[row * K + lane] = reinterpret_cast<const float*>(base + lay.probs)[tok * K + lane];
  }
}

// ---------------------------------------------------------------------------------------------------------------
// The same two kernels without any host-side count: every rank also leaves, in its mapped buffer, how many rows it
// sends to each rank (counts[world]) and where each destination's segment starts in its send order (seg[world+1]);
// a one-warp kernel turns all ranks' copies of those into this rank's tables, in device memory, and the pull
// kernels read the tables from there.  Buffers are then sized at a bound and rows beyond the real count are masked.
struct DevTables {
  int recv_off[kMaxPeers + 1];   // prefix over sources of the rows this rank receives
  int src_off[kMaxPeers];        // start of this rank's segment in source s's send order
  int first_row[kMaxPeers];      // row, in rank r's receive order, of this rank's first row sent to r
  int send_off[kMaxPeers];       // start of rank r's segment in this rank's send order
  int n_recv;
};

struct PeerBases {
  const uint8_t* base[kMaxPeers];
};

__global__ void ep_tables_kernel(PeerBases pb, int world, int me, int64_t off_counts, int64_t off_seg,
                                 DevTables* __restrict__ out) {
  if (threadIdx.x != 0) return;
  int acc = 0;
  for (int s = 0; s < world; ++s) {
    out->recv_off[s] = acc;
    acc += reinterpret_cast<const int*>(pb.base[s] + off_counts)[me];
    out->src_off[s] = reinterpret_cast<const int*>(pb.base[s] + off_seg)[me];
  }
  out->recv_off[world] = acc;
  out->n_recv = acc;
  for (int r = 0; r < world; ++r) {
    int before = 0;
    for (int s = 0; s < me; ++s) before += reinterpret_cast<const int*>(pb.base[s] + off_counts)[r];
    out->first_row[r] = before;
    out->send_off[r] = reinterpret_cast<const int*>(pb.base[me] + off_seg)[r];
  }
}

__global__ void __launch_bounds__(256)
ep_dispatch_pull_dev_kernel(PeerBases pb, const DevTables* __restrict__ tab, PullLayout lay, int world, int me, int H,
                            int K, int n_bound, uint4* __restrict__ q_out, uint32_t* __restrict__ raw_out,
                            int* __restrict__ idx_out, float* __restrict__ p_out) {
  const int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_bound) return;
  const int n_recv = tab->n_recv;
  if (row >= n_recv) {                                   // beyond what arrived: a row that routes nowhere
    if (idx_out != nullptr && lane < K) {
      idx_out[row * K + lane] = -1;
      p_out[row * K + lane] = 0.f;
    }
    return;
  }
  int rot = tab->recv_off[(me + 1) % world];             // start with the next rank's rows (see the kernel above)
  if (rot >= n_recv) rot = 0;
  row += rot;
  if (row >= n_recv) row -= n_recv;
  int s = 0;
  while (s + 1 < world && tab->recv_off[s + 1] <= row) ++s;
  const int64_t j = tab->src_off[s] + (row - tab->recv_off[s]);
  const uint8_t* base = pb.base[s];
  const int64_t tok = reinterpret_cast<const int*>(base + lay.tok)[j];
  const int h16 = H >> 4, words = H >> 7;
  const uint4* src = reinterpret_cast<const uint4*>(base + lay.q) + tok * h16;
  uint4* dst = q_out + row * h16;
  for (int c0 = 0; c0 < h16; c0 += 32 * 8) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u * 32 + lane;
      if (c < h16) v[u] = src[c];
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u * 32 + lane;
      if (c < h16) dst[c] = v[u];
    }
  }
  const uint32_t* rsrc = reinterpret_cast<const uint32_t*>(base + lay.raw) + tok * words;
  for (int c = lane; c < words; c += 32) raw_out[row * words + c] = rsrc[c];
  if (idx_out != nullptr && lane < K) {
    idx_out[row * K + lane] = reinterpret_cast<const int*>(base + lay.idx)[j * K + lane];
    p_out[row * K + lane] = reinterpret_cast<const float*>(base + lay.probs)[tok * K + lane];
  }
}

__global__ void __launch_bounds__(512)
ep_combine_pull_dev_kernel(PeerBases pb, const DevTables* __restrict__ tab, const int* __restrict__ copy_pos,
                           const int* __restrict__ copy_off, const int* __restrict__ send_rank,
                           uint4* __restrict__ out, int H8) {
  const int64_t t = blockIdx.x;
  const int beg = copy_off[t], end = copy_off[t + 1];
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int j = beg;
    for (; j + 4 <= end; j += 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = copy_pos[j + u];
        const int r = send_rank[i];
        v[u] = reinterpret_cast<const uint4*>(pb.base[r])[(int64_t)(tab->first_row[r] + i - tab->send_off[r]) * H8 + c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) acc8(v[u], a);
    }
    for (; j < end; ++j) {
      const int i = copy_pos[j];
      const int r = send_rank[i];
      acc8(reinterpret_cast<const uint4*>(pb.base[r])[(int64_t)(tab->first_row[r] + i - tab->send_off[r]) * H8 + c], a);
    }
    out[t * H8 + c] = make_uint4(bf16x2_of(a[0], a[1]), bf16x2_of(a[2], a[3]), bf16x2_of(a[4], a[5]),
                                 bf16x2_of(a[6], a[7]));
  }
}

}  // namespace smoe

extern "C" {

int64_t smoe_ep_tables_bytes(void) { return (int64_t)sizeof(smoe::DevTables); }

int smoe_ep_tables(const void* const* peer_bases, int64_t world, int64_t rank, int64_t off_counts, int64_t off_seg,
                   void* tables_out, void* stream) {
  if (world <= 0 || world > smoe::kMaxPeers || rank < 0 || rank >= world) return SMOE_ERR_SHAPE;
  if (!tables_out || ((off_counts | off_seg) & 3) || ((uintptr_t)tables_out & 3)) return SMOE_ERR_ARG;
  smoe::PeerBases pb{};
  for (int r = 0; r < world; ++r) pb.base[r] = (const uint8_t*)peer_bases[r];
  smoe::ep_tables_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pb, (int)world, (int)rank, off_counts, off_seg,
                                                             (smoe::DevTables*)tables_out);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ep_dispatch_pull_dev(const void* const* peer_bases, const void* tables, int64_t world, int64_t rank,
                              int64_t off_q, int64_t off_raw, int64_t off_tok, int64_t off_idx, int64_t off_probs,
                              int64_t H, int64_t K, int64_t n_bound, void* q_out, void* raw_out, int32_t* idx_out,
                              float* p_out, void* stream) {
  if (world <= 0 || world > smoe::kMaxPeers || H <= 0 || H % 128 || K <= 0 || K > 32) return SMOE_ERR_SHAPE;
  if (rank < 0 || rank >= world || n_bound < 0 || n_bound > INT32_MAX) return SMOE_ERR_ARG;
  if ((idx_out == nullptr) != (p_out == nullptr) || !tables) return SMOE_ERR_ARG;
  if ((off_q | off_raw | off_tok | off_idx | off_probs) & 15) return SMOE_ERR_ALIGN;
  if (n_bound == 0) return SMOE_OK;
  if (!q_out || !raw_out) return SMOE_ERR_ARG;
  if (((uintptr_t)q_out & 15) || ((uintptr_t)raw_out & 3)) return SMOE_ERR_ALIGN;
  smoe::PeerBases pb{};
  for (int r = 0; r < world; ++r) {
    if ((uintptr_t)peer_bases[r] & 15) return SMOE_ERR_ALIGN;
    pb.base[r] = (const uint8_t*)peer_bases[r];
  }
  smoe::PullLayout lay{off_q, off_raw, off_tok, off_idx, off_probs};
  const int64_t blocks = (n_bound + 7) / 8;
  smoe::ep_dispatch_pull_dev_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      pb, (const smoe::DevTables*)tables, lay, (int)world, (int)rank, (int)H, (int)K, (int)n_bound, (uint4*)q_out,
      (uint32_t*)raw_out, idx_out, p_out);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ep_combine_pull_dev(const void* const* peer_bases, const void* tables, int64_t world,
                             const int32_t* copy_pos, const int32_t* copy_off, const int32_t* send_rank,
                             void* out_bf16, int64_t T, int64_t H, void* stream) {
  if (world <= 0 || world > smoe::kMaxPeers || T < 0 || H <= 0 || H % 8) return SMOE_ERR_SHAPE;
  if (!tables) return SMOE_ERR_ARG;
  if ((uintptr_t)out_bf16 & 15) return SMOE_ERR_ALIGN;
  if (T == 0) return SMOE_OK;
  smoe::PeerBases pb{};
  for (int r = 0; r < world; ++r) {
    if ((uintptr_t)peer_bases[r] & 15) return SMOE_ERR_ALIGN;
    pb.base[r] = (const uint8_t*)peer_bases[r];
  }
  const int H8 = (int)(H / 8);
  int threads = H8 >= 512 ? 512 : ((H8 + 31) / 32) * 32;
  smoe::ep_combine_pull_dev_kernel<<<(unsigned)T, threads, 0, (cudaStream_t)stream>>>(
      pb, (const smoe::DevTables*)tables, copy_pos, copy_off, send_rank, (uint4*)out_bf16, H8);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ep_dispatch_pull(const void* const* peer_bases, const int32_t* recv_counts, const int32_t* src_off,
                          int64_t world, int64_t rank, int64_t off_q, int64_t off_raw, int64_t off_tok, int64_t off_idx,
                          int64_t off_probs, int64_t H, int64_t K, void* q_out, void* raw_out, int32_t* idx_out,
                          float* p_out, void* stream) {
  if (world <= 0 || world > smoe::kMaxPeers || H <= 0 || H % 128 || K <= 0 || K > 32) return SMOE_ERR_SHAPE;
  if (rank < 0 || rank >= world) return SMOE_ERR_ARG;
  if ((idx_out == nullptr) != (p_out == nullptr)) return SMOE_ERR_ARG;
  if ((off_q | off_raw | off_tok | off_idx | off_probs) & 15) return SMOE_ERR_ALIGN;
  smoe::PullTable tab{};
  int64_t n = 0;
  for (int r = 0; r < world; ++r) {
    if (recv_counts[r] < 0 || src_off[r] < 0) return SMOE_ERR_ARG;
    if ((uintptr_t)peer_bases[r] & 15) return SMOE_ERR_ALIGN;
    tab.base[r] = (const uint8_t*)peer_bases[r];
    tab.recv_off[r] = (int)n;
    tab.src_off[r] = src_off[r];
    n += recv_counts[r];
  }
  tab.recv_off[world] = (int)n;
  if (n == 0) return SMOE_OK;
  if (n > INT32_MAX) return SMOE_ERR_SHAPE;
  if (!q_out || !raw_out) return SMOE_ERR_ARG;
  if (((uintptr_t)q_out & 15) || ((uintptr_t)raw_out & 3)) return SMOE_ERR_ALIGN;
  smoe::PullLayout lay{off_q, off_raw, off_tok, off_idx, off_probs};
  const int64_t blocks = (n + 7) / 8;
  const int rot = tab.recv_off[(rank + 1) % world];     // == n when the ranks after this one send nothing: wraps to 0
  smoe::ep_dispatch_pull_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      tab, lay, (int)world, (int)H, (int)K, (int)n, rot >= n ? 0 : rot, (uint4*)q_out, (uint32_t*)raw_out, idx_out,
      p_out);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

int smoe_ep_combine_pull(const void* const* peer_bases, const int32_t* first_row, const int32_t* send_off,
                         int64_t world, const int32_t* copy_pos, const int32_t* copy_off, const int32_t* send_rank,
                         void* out_bf16, int64_t T, int64_t H, void* stream) {
  if (world <= 0 || world > smoe::kMaxPeers || T < 0 || H <= 0 || H % 8) return SMOE_ERR_SHAPE;
  if ((uintptr_t)out_bf16 & 15) return SMOE_ERR_ALIGN;
  if (T == 0) return SMOE_OK;
  smoe::PeerTable tab{};
  for (int r = 0; r < world; ++r) {
    if ((uintptr_t)peer_bases[r] & 15) return SMOE_ERR_ALIGN;
    tab.base[r] = (const uint4*)peer_bases[r];
    tab.first_row[r] = first_row[r];
    tab.send_off[r] = send_off[r];
  }
  const int H8 = (int)(H / 8);
  int threads = H8 >= 512 ? 512 : ((H8 + 31) / 32) * 32;
  smoe::ep_combine_pull_kernel<<<(unsigned)T, threads, 0, (cudaStream_t)stream>>>(
      tab, copy_pos, copy_off, send_rank, (uint4*)out_bf16, H8);
  return cudaGetLastError() == cudaSuccess ? SMOE_OK : SMOE_ERR_LAUNCH;
}

}  // extern "C"
