/* C ABI of libsmoe_b200.so: the sm_100a kernels of the MoE layer forward/backward hot path.
 *
 * Conventions (all entry points):
 *   - plain pointers to DEVICE memory owned by the caller, 64-bit sizes, a
 *     cudaStream_t passed as void*; nothing is allocated, nothing synchronises:
 *     work is enqueued on `stream` and the call returns.
 *   - return value 0 (SMOE_OK) or a SMOE_ERR_* code for argument / launch errors
 *     detected on the host.  A problem with zero rows (nothing routed to this
 *     rank) is not an error: the call returns SMOE_OK without a launch.  Failures detected on the device (a bounded wait
 *     that ran out) are written to the caller's `status` word (0 = ok).
 *   - "ISA-packed" scales: for a logical (rows, cols) operand with one ue8m0
 *     byte per 1x32 group, byte(row, g) lives at
 *       ((row/128)*ceil(cols/128) + g/4)*512 + (row%32)*16 + ((row%128)/32)*4 + g%4.
 *
 * Each declaration cites the reference interface it replaces (paths inside
 * PFCCLab/supersonic-moe).
 */
#ifndef SMOE_B200_H_
#define SMOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  SMOE_OK = 0,
  SMOE_ERR_SHAPE = 1,   /* a size violates the documented divisibility / range rules */
  SMOE_ERR_ALIGN = 2,   /* a pointer or row pitch is not 16-byte aligned */
  SMOE_ERR_DRIVER = 3,  /* cuTensorMapEncodeTiled could not be resolved */
  SMOE_ERR_TMAP = 4,    /* tensor-map encoding failed */
  SMOE_ERR_LAUNCH = 5,  /* kernel launch failed */
  SMOE_ERR_ARG = 6      /* null pointer / unsupported option */
};

/* ---- routing metadata ---------------------------------------------------- */

/* count[e] = #(ids == e) and its inclusive cumsum, int32.
 * Replaces count_cumsum (sonicmoe/count_cumsum/__init__.py:20-35, kernel.cu:154-218).
 * ids_is_int64: 0 = int32 ids, 1 = int64 ids.  cumsum may be null. */
int smoe_count_cumsum(const void* ids, int ids_is_int64, int64_t n, int64_t E, int32_t* count, int32_t* cumsum,
                      void* stream);

/* Bytes of scratch smoe_topk_metadata needs for N rows and E experts. */
int64_t smoe_topk_metadata_workspace(int64_t N, int64_t E);

/* top-k indices/probs -> padded routing metadata, replaces deepep_topk_to_sonic_metadata
 * (sonicmoe/ernie_compat/deepep_metadata.py:180-358, deepep_topk_metadata_cuda/kernel.cu:829-1191).
 *   idx [N,K] int32 (valid iff 0 <= e < E, a row's valid experts distinct), probs [N,K] f32
 *   efo [E+1], x_gather_idx [TKp_alloc], s_scatter_idx [TKp_alloc], s_reverse_scatter_idx [TK_alloc],
 *   naept [N+1], topk_scores [TKp_alloc] f32, score_src_idx [TK_alloc], counts [E]
 *   lane_order: 0 = a token's lanes by ascending expert id (kernel.cu:567-578),
 *               1 = by top-k slot (dense path, functional/triton_kernels/__init__.py:66-155)
 *   pad_mode:   0 = pad rows scatter to real_TK (kernel.cu:611-650),
 *               1 = i-th pad row scatters to real_TK + i (functional/__init__.py:226-234)
 *   TK_alloc / TKp_alloc smaller than what idx really holds (buffers sized from stale per-expert counts): the rows
 *   that do not fit are dropped and efo is clamped to TKp_alloc - nothing is written outside the buffers. */
int smoe_topk_metadata(const int32_t* idx, const float* probs, int64_t N, int64_t K, int64_t E, int64_t alignment,
                       int64_t TK_alloc, int64_t TKp_alloc, int lane_order, int pad_mode, int32_t* efo,
                       int32_t* x_gather_idx, int32_t* s_scatter_idx, int32_t* s_reverse_scatter_idx, int32_t* naept,
                       float* topk_scores, int32_t* score_src_idx, int32_t* counts, void* workspace, void* stream);

/* smoe_topk_metadata for callers that cannot allocate device memory (no counterpart in the reference, whose
 * launcher allocates its scratch and outputs itself): work captured into a CUDA graph or run from a stream
 * callback, a serving process that bans cudaMalloc after start-up, a host framework whose allocator this
 * library has no handle to.  The scratch is a fixed 1 MiB array inside the library (every GPU that loads the
 * library holds it until the process exits); the caller still passes inputs and outputs.
 *   - sizes whose scratch need, smoe_topk_metadata_workspace(N, E), exceeds
 *     smoe_topk_metadata_static_capacity() are refused with SMOE_ERR_SHAPE (e.g. 16384 rows x 128 experts fit);
 *   - the first call on a device looks the array's device address up (once per device, with that device
 *     current); make that first call before any stream capture begins;
 *   - all calls share the one array, which keeps the previous call's contents: nothing in it needs clearing
 *     between calls, but two calls whose kernels can overlap on the GPU (different streams) race on it;
 *   - calls no cudaMalloc / cudaFree and no allocating library routine. */
int smoe_topk_metadata_static(const int32_t* idx, const float* probs, int64_t N, int64_t K, int64_t E,
                              int64_t alignment, int64_t TK_alloc, int64_t TKp_alloc, int lane_order, int pad_mode,
                              int32_t* efo, int32_t* x_gather_idx, int32_t* s_scatter_idx,
                              int32_t* s_reverse_scatter_idx, int32_t* naept, float* topk_scores,
                              int32_t* score_src_idx, int32_t* counts, void* stream);
int64_t smoe_topk_metadata_static_capacity(void);

/* ---- expert-parallel dispatch planning --------------------------------------
 * No counterpart in the reference, which ships no communication code (its host framework calls DeepEP around
 * run_sonic_moe); these two kernels bracket smoe_topk_metadata, run with destination ranks in the role of experts,
 * to build the send order of the all-to-all dispatch on the device. */

/* idx [T,K] global expert ids (valid iff 0 <= e < E; E % world == 0, rank r owns [r*E/world, (r+1)*E/world)) ->
 * dest_u [T,K]: owning rank of each slot, -1 for invalid slots and for every slot after the first that goes to the
 * same rank (a token travels once per rank); pairs [E]: routed (token, slot) pairs per global expert (zeroed here). */
int smoe_ep_plan_dest(const int32_t* idx, int64_t T, int64_t K, int64_t E, int64_t world, int32_t* dest_u,
                      int32_t* pairs, void* stream);

/* Per outgoing row i < n_send (send_tok[i] = its token, efo = per-rank offsets of the send order):
 * send_rank[i] and send_idx[i,K] = the token's expert ids local to that rank, -1 for slots owned elsewhere. */
int smoe_ep_plan_send_idx(const int32_t* idx, const int32_t* send_tok, const int32_t* efo, int64_t n_send, int64_t K,
                          int64_t E, int64_t world, int32_t* send_idx, int32_t* send_rank, void* stream);

/* Combine over NVLink peer memory: out[t,:] (bf16) = sum, in ascending destination rank and fp32, of the partial
 * output rows the owning ranks hold for token t, read straight from their buffers (peer_bases[r]: rank r's bf16
 * [rows,H] buffer as mapped into this process; host arrays of `world` entries).  Outgoing row i (send order) went to
 * send_rank[i] and is row first_row[rank] + (i - send_off[rank]) there; copy_pos / copy_off list every token's
 * outgoing rows.  The caller must order "every rank has written its buffer" before this call on the stream (any
 * collective on that stream does).  No counterpart in the reference (DeepEP's combine plays this role outside it). */
int smoe_ep_combine_pull(const void* const* peer_bases, const int32_t* first_row, const int32_t* send_off,
                         int64_t world, const int32_t* copy_pos, const int32_t* copy_off, const int32_t* send_rank,
                         void* out_bf16, int64_t T, int64_t H, void* stream);

/* Dispatch over NVLink peer memory: this rank fetches the rows addressed to it straight from the sources' buffers
 * (peer_bases[s]: rank s's buffer as mapped into this process; the same byte layout on every rank: e4m3 tokens [T,H]
 * at off_q, raw 1x32 scales [T,H/32] at off_raw, the token of every outgoing row [n_send] int32 at off_tok, its local
 * expert ids [n_send,K] int32 at off_idx, the tokens' probabilities [T,K] f32 at off_probs).  recv_counts[s] rows
 * come from rank s, starting at row src_off[s] of its send order; they land in q_out / raw_out / idx_out / p_out in
 * the order an all-to-all delivers them (sources ascending).  idx_out and p_out may both be null (payload only: the
 * gradient's dispatch in the backward).  The caller orders "every rank has written its buffer" before the call on
 * the stream.  `rank` (this rank's index among the sources) only sets where the grid starts: with the next rank's
 * rows, so that the ranks do not all read from the same source at the same time.  Plain loads, no multicast, no
 * wait in the kernel.  No counterpart in the reference (DeepEP's dispatch plays this role outside it).
 * H % 128 == 0, K <= 32, world <= 16. */
int smoe_ep_dispatch_pull(const void* const* peer_bases, const int32_t* recv_counts, const int32_t* src_off,
                          int64_t world, int64_t rank, int64_t off_q, int64_t off_raw, int64_t off_tok, int64_t off_idx,
                          int64_t off_probs, int64_t H, int64_t K, void* q_out, void* raw_out, int32_t* idx_out,
                          float* p_out, void* stream);

/* The two pull kernels without host-side counts.  Every rank additionally leaves, in its mapped buffer, the rows it
 * sends to each rank (int32 [world] at off_counts) and the start of each destination's segment in its send order
 * (int32 [world+1] at off_seg).  smoe_ep_tables (one warp) turns all ranks' copies into this rank's tables in device
 * memory (`tables_out`: smoe_ep_tables_bytes() bytes); smoe_ep_dispatch_pull_dev walks `n_bound` rows (the capacity the
 * outputs are allocated for), fetches the rows that exist and marks the others as routed nowhere (idx -1, probability
 * 0, payload untouched); smoe_ep_combine_pull_dev is smoe_ep_combine_pull with its two offset tables read from
 * `tables`.  With them a step needs no device-to-host read-back before its return exchange. */
int64_t smoe_ep_tables_bytes(void);
int smoe_ep_tables(const void* const* peer_bases, int64_t world, int64_t rank, int64_t off_counts, int64_t off_seg,
                   void* tables_out, void* stream);
int smoe_ep_dispatch_pull_dev(const void* const* peer_bases, const void* tables, int64_t world, int64_t rank,
                              int64_t off_q, int64_t off_raw, int64_t off_tok, int64_t off_idx, int64_t off_probs,
                              int64_t H, int64_t K, int64_t n_bound, void* q_out, void* raw_out, int32_t* idx_out,
                              float* p_out, void* stream);
int smoe_ep_combine_pull_dev(const void* const* peer_bases, const void* tables, int64_t world,
                             const int32_t* copy_pos, const int32_t* copy_off, const int32_t* send_rank,
                             void* out_bf16, int64_t T, int64_t H, void* stream);

/* ---- MXFP8 1x32 ue8m0 quantizers ------------------------------------------ */

/* Row-wise: x bf16 [M,K] -> e4m3 [M,K] + raw scales [M,K/32] and/or ISA-packed scales
 * (either scale pointer may be null).  Replaces quantize_and_pack_activation
 * (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:3214-3283) and
 * quantize_activation_blockscaled_fast (:518-596).  K % 32 == 0. */
int smoe_quant_rows(const void* x_bf16, int64_t M, int64_t K, void* q, void* raw_scales, void* isa_scales,
                    void* stream);

/* Row quantizer with the expert-sorted gather fused in: q[r,:] = quant(x[idx[r],:]) for r < min(rows, *valid_rows),
 * ISA scales for (rows, K).  One pass instead of quantise + gather (sonicmoe/quack_utils/sm100_funcs.py:248-283 does
 * quantize_and_pack_activation followed by _gather_1x32_scales_to_isa and gathers rows inside its GEMM). */
int smoe_quant_rows_gather(const void* x_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t K,
                           void* q, void* isa_scales, void* stream);

/* Gathered quantizer for both GEMM directions in one pass over 32-row groups of the expert-sorted order:
 * q_row[r,:] = row-wise 1x32 quantisation of x[idx[r],:] with ISA scales for (rows,K) (what smoe_quant_rows_gather
 * writes; both pointers may be null to skip it) and q_col[r,:] = the same rows quantised with one scale per column
 * and 32 consecutive rows, ISA scales for (K,rows) - the bytes of smoe_quant_cols_t, not transposed: the payload
 * stays [rows,K] and smoe_gemm_wgrad_mn reads it MN-major.  Rows at or beyond *valid_rows are left untouched.
 * Replaces dual_quantize_and_pack with gather_idx and dual_quantize_varlen
 * (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:1428-1500, :1964-2148), whose column-quantised payload is likewise
 * kept (TK, dim).  K % 256 == 0, rows % 128 == 0. */
int smoe_quant_dual_gather(const void* x_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t K,
                           void* q_row, void* row_isa, void* q_col, void* col_isa, void* stream);

/* Same result in scatter form: every token row of x [T,K] is read and quantised once and written to each
 * expert-sorted position it occupies, s_rev[naept[t] .. naept[t+1]); pad rows (s_scatter_idx[row] >= naept[T]) are
 * zero-filled (the gather form copies token 0 there; either way they are multiplied by a zero score downstream).
 * K % 128 == 0, K <= 16384. */
int smoe_quant_rows_scatter(const void* x_bf16, int64_t T, int64_t K, const int32_t* naept, const int32_t* s_rev,
                            const int32_t* s_scatter_idx, const int32_t* valid_rows, int64_t rows, void* q,
                            void* isa_scales, void* stream);

/* raw row scales [T, cols/32] gathered to `rows` rows by idx, ISA layout for (rows, cols).
 * Replaces _gather_1x32_scales_to_isa (sonicmoe/quack_utils/sm100_funcs.py:148-180). */
int smoe_gather_scales_isa(const void* raw_scales, const int32_t* idx, int64_t rows, int64_t cols, void* isa_scales,
                           void* stream);

/* Rows of an already quantised activation gathered into expert-sorted order: q_out[r,:] = q[idx[r],:] and the
 * rows' raw scales [T,K/32] written in the ISA layout of (rows, K).  Rows >= *valid_rows (device int, may be null)
 * are left untouched.  Materialises the A operand of the up-projection / GemmDGated for the tiled-TMA load path;
 * the reference gathers inside its GEMM (sonicmoe/quack_utils/gemm_sm100_fp8_zeromat.py:65-67) and packs the scales
 * with _gather_1x32_scales_to_isa (sm100_funcs.py:148-180).  K % 128 == 0. */
int smoe_gather_rows_fp8(const void* q, const void* raw_scales, const int32_t* idx, const int32_t* valid_rows,
                         int64_t rows, int64_t K, void* q_out, void* isa_out, void* stream);

/* Same result in scatter form (pad rows zero instead of a copy of row idx[r]): every source row is read once and
 * written to its positions s_rev[naept[t] .. naept[t+1]); used for the e4m3 payload an expert-parallel dispatch
 * delivers, where a received row feeds several local experts.  isa_out (and then raw_scales) may be null: payload
 * only, for a caller that already holds the packed scales (deepep_topk_to_sonic_metadata_with_scales). */
int smoe_scatter_rows_fp8(const void* q, const void* raw_scales, int64_t T, int64_t K, const int32_t* naept,
                          const int32_t* s_rev, const int32_t* s_scatter_idx, const int32_t* valid_rows, int64_t rows,
                          void* q_out, void* isa_out, void* stream);

/* Column-wise (groups of 32 consecutive rows) of src[idx] (idx may be null): src bf16 [T,dim] ->
 *   q_t  e4m3 [dim, rows]  (TRANSPOSED: the reduction dimension of the weight-gradient GEMM is contiguous)
 *   isa  ISA-packed scales for the logical (dim, rows) operand.
 * Replaces colwise_quantize_and_pack (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:1517-1592,1824-1847);
 * same bytes and scale bytes, transposed storage.  rows % 128 == 0, dim % 64 == 0.  Row tiles at or beyond
 * *valid_rows (device int, may be null) are left untouched: with buffers sized at an upper bound, only the rows of
 * the experts' segments are ever read. */
int smoe_quant_cols_t(const void* src_bf16, const int32_t* idx, const int32_t* valid_rows, int64_t rows, int64_t dim,
                      void* q_t, void* isa, void* stream);

/* Same, for a source that is already e4m3 with raw row-wise 1x32 scales [T,dim/32] (an FP8 dispatch payload):
 * dequantise, then column-wise re-quantise.  Replaces _dequant_colwise_quantize_and_pack_from_isa_kernel
 * (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:5206-5359). */
int smoe_requant_cols_t(const void* src_fp8, const void* src_scales, const int32_t* idx, const int32_t* valid_rows,
                        int64_t rows, int64_t dim, void* q_t, void* isa, void* stream);

/* 32x32 block ("iso32") quantizer: dz bf16 [rows, cols] -> q e4m3 [rows, cols] + row-ISA scales for (rows, cols),
 * q_t e4m3 [cols, rows] + col-ISA scales for (cols, rows).  Replaces dual_quantize_varlen iso32
 * (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:2052-2198).  rows % 128 == 0, cols % 128 == 0. */
int smoe_quant_iso32(const void* x_bf16, int64_t rows, int64_t cols, void* q, void* row_isa, void* q_t, void* col_isa,
                     void* stream);
/* q_t may be null: the row-major payload then serves both orientations (with 32x32-block scales the transposed
 * bytes are the transposed quantisation), which is the reference's single-buffer ISO32 weight cache
 * (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:3765-3856): a weight [N,K] is kept once, K-major for the forward
 * GEMM (row_isa) and read MN-major by smoe_gemm_varlen_m_bt for the activation gradient (col_isa). */

/* dst[b][c][r] = src[b][r][c] over a batch of [rows, cols] byte matrices (rows, cols multiples of 64, batch <=
 * 65535).  Makes the transient K-major copy of an ISO32 weight for a GEMM that cannot read it MN-major (the
 * reference does the same for w2 in its backward, sonicmoe/functional/__init__.py:2160). */
int smoe_transpose_u8(const void* src, int64_t batch, int64_t rows, int64_t cols, void* dst, void* stream);

/* ---- grouped GEMMs (tcgen05 block-scaled) --------------------------------- */

/* C[p,:] = A[p,:] . B[e(p)]^T for rows grouped by expert (segments 128-aligned), bf16 out.
 * A e4m3 [rows,K] + ISA scales (rows,K); B e4m3 [E,N,K] + ISA scales (E*N,K).
 * Replaces fp8_kernels.gemm -> blockscaled_fp8_gemm_varlen
 * (sonicmoe/quack_utils/sm100_funcs.py:784-807, blockscaled_fp8_gemm.py:4563-4748). */
int smoe_gemm_varlen_m(const void* a_fp8, const void* a_sf, const void* b_fp8, const void* b_sf, const int32_t* efo,
                       void* c_bf16, int64_t rows, int64_t N, int64_t K, int64_t E, int32_t* status, void* stream);

/* The same product with B stored [E,K,N] (N contiguous, "MN-major"): B[e] is read as it lies in a weight kept once
 * for both orientations; b_sf = ISA scales for (E*N, K) as above.  Replaces the zero-copy `.permute(0,2,1)` view the
 * reference hands its GEMM in ISO32 mode (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:3822-3840).  256-column
 * two-CTA tiles only: N % 256 == 0, E <= 256, else SMOE_ERR_SHAPE. */
int smoe_gemm_varlen_m_bt(const void* a_fp8, const void* a_sf, const void* b_kn_fp8, const void* b_sf,
                          const int32_t* efo, void* c_bf16, int64_t rows, int64_t N, int64_t K, int64_t E,
                          int32_t* status, void* stream);

/* Up-projection: z = x[a_idx] . W1[e]^T (N = 2I, K = H), y1 = swiglu(z) on interleaved gate/up columns;
 * z -> e4m3 [rows,N] + raw scales [rows,N/32] (amax floor 1e-4), y1 -> bf16 RNE -> e4m3 [rows,N/2] + ISA scales.
 * a_idx == NULL: x_fp8 is already in expert-sorted row order ([rows,K]) and is loaded as plain TMA tiles;
 * a_idx != NULL: x_fp8 is the un-gathered [T,K] activation and row p of the GEMM is x_fp8[a_idx[p]], fetched inside
 * the kernel by four cp.async load warps per CTA (as the reference's gather_A does,
 * sonicmoe/quack_utils/gemm_sm100_fp8_zeromat.py:60-67) - no gathered copy exists; a_sf holds the scales already in
 * expert-sorted ISA layout (smoe_gather_scales_isa).
 * Replaces gemm_gated (sonicmoe/quack_utils/sm100_funcs.py:207-455, gemm_sm100_fp8_zeromat.py:379-406,
 * _gated_epilogues.py:1331-1513).  N % 256 == 0. */
int smoe_gemm_gated(const void* x_fp8, int64_t T, const int32_t* a_idx, const void* a_sf, const void* w1_fp8,
                    const void* w1_sf, const int32_t* efo, void* z_fp8, void* z_scales, void* y1_fp8, void* y1_sf,
                    int64_t rows, int64_t N, int64_t K, int64_t E, int32_t* status, void* stream);

/* Backward of the activation: D = dout[a_idx] . W2T[e]^T (N = I, K = H) and, against the saved e4m3 z,
 * dz (bf16 [rows,2N]), y1s = s*y (bf16 [rows,N]) and per-column-tile partial sums of ds ([partials, rows] f32).
 * Replaces gemm_dgated (sonicmoe/quack_utils/sm100_funcs.py:824-885, _gated_epilogues.py:2772-3000). */
int smoe_gemm_dgated(const void* dout_fp8, int64_t T, const int32_t* a_idx, const void* a_sf, const void* w2t_fp8,
                     const void* w2t_sf, const int32_t* efo, const void* z_fp8, const void* z_scales, const float* s,
                     void* dz_bf16, void* y1s_bf16, float* ds_partial, int64_t* ds_partial_tiles, int64_t rows,
                     int64_t N, int64_t K, int64_t E, int32_t* status, void* stream);
int64_t smoe_gemm_dgated_partials(int64_t N);

/* GemmDGated with the operand quantizers of the following GEMMs fused into its epilogue: instead of dz / y1s in
 * bf16 it emits the payload and scale bytes that smoe_quant_iso32(dz) and smoe_quant_cols_t(y1s) would produce
 * from the bf16 tensors, both payloads row-major: dz_q e4m3 [rows,2N] with ISA scales for (rows,2N) and for
 * (2N,rows) - one scale per 32x32 block, so the one payload is the activation-gradient operand and, fed MN-major
 * through smoe_gemm_wgrad_mn, the weight-gradient operand - and y1s_q e4m3 [rows,N] with column ISA scales
 * (N,rows).  A operand already gathered ([rows,K]).  Replaces gemm_dgated + quantize_dz_dout +
 * quantize_wgrad_operand(y1s) (sonicmoe/quack_utils/sm100_funcs.py:824-944).  Two-CTA kernel only: E <= 256,
 * else SMOE_ERR_SHAPE. */
int smoe_gemm_dgated_fused(const void* dout_fp8, const void* a_sf, const void* w2t_fp8, const void* w2t_sf,
                           const int32_t* efo, const void* z_fp8, const void* z_scales, const float* s, void* dz_q,
                           void* dz_row_sf, void* dz_col_sf, void* y1s_q, void* y1s_col_sf, float* ds_partial,
                           int64_t rows, int64_t N, int64_t K, int64_t E, int32_t* status, void* stream);
int64_t smoe_gemm_dgated_fused_partials(int64_t N);

/* The same with the A rows fetched by index inside the kernel: dout_fp8 is the un-gathered [T,K] e4m3 gradient, row p
 * of the GEMM is dout_fp8[a_idx[p]] (cp.async load warps, see smoe_gemm_gated); a_sf as above, expert-sorted. */
int smoe_gemm_dgated_fused_gather(const void* dout_fp8, int64_t T, const int32_t* a_idx, const void* a_sf,
                                  const void* w2t_fp8, const void* w2t_sf, const int32_t* efo, const void* z_fp8,
                                  const void* z_scales, const float* s, void* dz_q, void* dz_row_sf, void* dz_col_sf,
                                  void* y1s_q, void* y1s_col_sf, float* ds_partial, int64_t rows, int64_t N,
                                  int64_t K, int64_t E, int32_t* status, void* stream);

/* Weight gradient: C[e] (M x N, f32) (+)= A_t[:, seg_e] . B_t[:, seg_e]^T with A_t e4m3 [M,TKp], B_t e4m3 [N,TKp]
 * and ISA scales for (M,TKp) / (N,TKp).  Replaces wgrad_gemm_varlen_k
 * (sonicmoe/quack_utils/sm100_funcs.py:947-976, blockscaled_fp8_gemm.py:2210-2687). */
int smoe_gemm_wgrad(const void* a_t_fp8, const void* a_sf, const void* b_t_fp8, const void* b_sf, const int32_t* efo,
                    float* c, int64_t M, int64_t N, int64_t TKp, int64_t E, int accumulate, int32_t* status,
                    void* stream);

/* Weight gradient with operands in their natural orientation.  layout bit 0: A is e4m3 [TKp, M] (row = routed
 * token position) instead of [M, TKp]; bit 1: B is e4m3 [TKp, N] instead of [N, TKp].  Such an operand is fed to
 * the tensor core MN-major, so the activation-gradient GEMM's row-major outputs serve as weight-gradient operands
 * without a transposed copy.  Scales are ISA-packed for (M,TKp) / (N,TKp) either way.  Same reference operation as
 * smoe_gemm_wgrad (the reference's quantize_wgrad_operand writes transposed copies instead,
 * sonicmoe/quack_utils/blockscaled_fp8_gemm.py:2210-2687).  Needs M % 256 == 0, N % 256 == 0, E <= 256. */
int smoe_gemm_wgrad_mn(const void* a_fp8, const void* a_sf, const void* b_fp8, const void* b_sf, const int32_t* efo,
                       float* c, int64_t M, int64_t N, int64_t TKp, int64_t E, int accumulate, int layout,
                       int32_t* status, void* stream);

/* Two such products in ONE launch: c1[e] (+)= A1_e^T B1_e (M1 x N) and c2[e] (+)= A2_e^T B2_e (M2 x N) over the same
 * expert segments - in the layer dw1 (A = dz, B = x) and dw2 (A = y1s, B = dout).  Run one after the other their
 * tile counts (768 and 384 at the reference shape, on 74 CTA pairs) leave a partly filled last wave each; together
 * they leave one.  256 x 384 kernel only: N % 384 == 0, M1, M2 % 256 == 0, E <= 256; both A operands stored
 * [TKp, M] (a_rows_major_tk = 1) or both [M, TKp] (0); both B operands [N, TKp]; every output element still has a
 * single writer.  The reference issues the two weight-gradient GEMMs separately
 * (sonicmoe/quack_utils/sm100_funcs.py:947-976). */
int smoe_gemm_wgrad_mn_pair(const void* a1_fp8, const void* a1_sf, const void* b1_fp8, const void* b1_sf, float* c1,
                            int64_t M1, const void* a2_fp8, const void* a2_sf, const void* b2_fp8, const void* b2_sf,
                            float* c2, int64_t M2, const int32_t* efo, int64_t N, int64_t TKp, int64_t E,
                            int accumulate, int a_rows_major_tk, int32_t* status, void* stream);

/* ---- gated activations outside the GEMM epilogues ----------------------------
 * The fused epilogues of smoe_gemm_gated / smoe_gemm_dgated* carry SwiGLU.  For the reference's other gated
 * activations (sonicmoe/enums.py:18-33; mapped to quack.activation.reglu / geglu in quack_utils/gemm_gated.py:171-177)
 * the projections run as plain GEMMs (smoe_gemm_varlen_m) and these two HBM-bound kernels do the epilogues' work.
 * act: 0 = swiglu, 1 = reglu (relu(g) * u), 2 = geglu (tanh-approximated gelu(g) * u); gate / up interleaved. */

/* z bf16 [rows,2I] -> z e4m3 [rows,2I] + raw 1x32 scales [rows,2I/32] (amax floor 1e-4) and y1 = bf16(act(g)*u) ->
 * e4m3 [rows,I] + ISA scales for (rows,I): what the epilogue of gemm_gated emits
 * (sonicmoe/quack_utils/_gated_epilogues.py:1331-1513).  I % 32 == 0. */
int smoe_glu_fwd(const void* z_bf16, int64_t rows, int64_t I, int act, void* z_fp8, void* z_scales, void* y1_fp8,
                 void* y1_sf, void* stream);

/* D bf16 [rows,I] (= dout . W2 per expert) against the saved e4m3 z: dz bf16 [rows,2I] (interleaved), y1s = s*y bf16
 * [rows,I], ds_rows[row] = sum_j y_j D_j: what the epilogue of gemm_dgated emits
 * (sonicmoe/quack_utils/_gated_epilogues.py:2864-3000). */
int smoe_glu_bwd(const void* d_bf16, const void* z_fp8, const void* z_scales, const float* s, int64_t rows, int64_t I,
                 int act, void* dz_bf16, void* y1s_bf16, float* ds_rows, void* stream);

/* ---- combine / router ------------------------------------------------------ */

/* o[t,:] = sum_j w * y[s_rev[naept[t]+j], :] in ascending j, f32 accumulate, bf16 store; w = scores[naept[t]+j]
 * when scores != null else 1.  Replaces token_gather_and_sum_varlen_K_triton
 * (sonicmoe/functional/reduction_over_k_gather.py:99-196,340-395). */
int smoe_combine(const void* y_bf16, const int32_t* s_rev, const int32_t* naept, const float* scores, void* out_bf16,
                 int64_t T, int64_t H, void* stream);

/* s[p] = scores[s_scatter_idx[p]] for p < rows (replaces the score gather of
 * sonicmoe/functional/__init__.py:2105). */
int smoe_gather_scores(const float* scores, const int32_t* s_scatter_idx, int64_t rows, float* s, void* stream);

/* ds_tm[i] = sum_t ds_partial[t][s_rev[i]] for i < min(TK, *real_tk), 0 beyond (real_tk may be null);
 * optionally also scatter_out[src_idx[i]] = ds_tm[i] for the real entries (scatter_out must be pre-zeroed).
 * Replaces the partial-sum + permutation of sonicmoe/quack_utils/sm100_funcs.py:885,
 * sonicmoe/functional/__init__.py:2384 and the ds scatter of :2488-2500. */
int smoe_ds_finalize(const float* ds_partial, int64_t partials, int64_t rows, const int32_t* s_rev, int64_t TK,
                     const int32_t* real_tk, float* ds_tm, const int32_t* src_idx, float* scatter_out, void* stream);

/* *pinned_host_word = *status, written by a one-thread kernel on `stream`: `status` is the device word the GEMM entry
 * points report failures in, `pinned_host_word` page-locked host memory the device can address (cudaHostAlloc /
 * torch pin_memory).  Lets a host poll for device-side failures without a synchronisation and without a memcpy that
 * would queue behind bulk transfers.  No counterpart in the reference, whose kernels report nothing. */
int smoe_status_post(const int32_t* status, int32_t* pinned_host_word, void* stream);

/* top-K of each row of logits [T,E] (f32) and softmax over the K selected values.
 * Replaces _softmax_topk_fwd (sonicmoe/functional/forward.py:217-236, topk_softmax.py). */
int smoe_topk_softmax(const float* logits, int64_t T, int64_t E, int64_t K, float* scores, int32_t* idx, void* stream);

/* dlogits[t, idx[t,k]] = s_k (g_k - sum_j g_j s_j), zero elsewhere.
 * Replaces _softmax_topk_bwd (sonicmoe/functional/backward.py:572-641). */
int smoe_topk_softmax_bwd(const float* scores, const int32_t* idx, const float* dscores, int64_t T, int64_t E, int64_t K,
                          float* dlogits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SMOE_B200_H_ */
