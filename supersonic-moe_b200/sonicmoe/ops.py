"""Tensor-level wrappers over the C ABI: allocate outputs with the caching
allocator, pass raw device pointers and the current stream.  CUDA tensors only;
there is no CPU path.
"""
from __future__ import annotations

import torch

from ._lib import check, lib

_U8 = torch.uint8
_I32 = torch.int32


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("sonicmoe kernels need CUDA tensors (no CPU fallback)")
        if t is not None and not t.is_contiguous():
            raise RuntimeError("sonicmoe kernels need contiguous tensors")


def isa_bytes(rows: int, cols: int) -> int:
    return -(-rows // 128) * -(-cols // 128) * 512


_status = {}

# Optional per-op CUDA-event recorder (bench / profiling): a list that receives
# (op name, start event, end event) for every kernel-launching wrapper below.
_recorder = None


def set_recorder(rec):
    global _recorder
    _recorder = rec


def _timed(fn):
    import functools

    @functools.wraps(fn)
    def wrapper(*a, **k):
        if _recorder is None:
            return fn(*a, **k)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **k)
        e1.record()
        _recorder.append((fn.__name__, e0, e1))
        return out
    return wrapper


def _dev_index(device) -> int:
    """Ordinal of a CUDA device given as a device, a string or an int; "cuda" without an ordinal means the current
    device (so that "cuda" and "cuda:0" name the same status word)."""
    d = torch.device(device) if not isinstance(device, int) else torch.device("cuda", device)
    if d.type != "cuda":
        raise RuntimeError("sonicmoe kernels need CUDA tensors (no CPU fallback)")
    return d.index if d.index is not None else torch.cuda.current_device()


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the GEMM kernels write a failure code into (0 = ok)."""
    key = _dev_index(device)
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=_I32, device=torch.device("cuda", key))
    return _status[key]


def _raise_status(device, code):
    status_word(device).zero_()
    raise RuntimeError(f"sonicmoe GEMM kernel reported device failure code {code} on cuda:{_dev_index(device)} "
                       "(a bounded wait inside a kernel ran out; results of that step are invalid)")


def check_status(device):
    """Synchronous read of the device status word; raises when a kernel recorded a failure."""
    s = int(status_word(device).item())
    if s != 0:
        _raise_status(device, s)


# The layer reads the status word without ever waiting for the GPU: the end of a forward / backward launches a
# one-thread kernel that stores the word into pinned host memory (a kernel store, not a memcpy: it cannot queue behind
# bulk transfers on a copy engine); the next entry into the layer looks at that host word and raises if it is
# non-zero.  The word is sticky on the device, so a failure surfaces at the latest one call after the pass whose
# post saw it, and a healthy run pays one tiny launch per pass and no synchronisation.
_posted = {}     # device index -> pinned int32[1] mirror of the device status word


def post_status(device):
    """Enqueue, on the current stream, the store of the status word into its pinned host mirror (no-op while a graph
    is captured)."""
    if torch.device(device).type != "cuda" or torch.cuda.is_current_stream_capturing():
        return
    key = _dev_index(device)
    host = _posted.get(key)
    if host is None:
        host = _posted[key] = torch.zeros(1, dtype=_I32).pin_memory()
    check(lib.smoe_status_post(_p(status_word(device)), host.data_ptr(), _stream()), "status_post")


def poll_status(device):
    """Look at the host mirror of the status word; raise on a recorded failure.  Never waits."""
    if torch.device(device).type != "cuda":
        return
    host = _posted.get(_dev_index(device))
    if host is not None:
        code = int(host[0])
        if code != 0:
            host[0] = 0
            _raise_status(device, code)


# ---------------------------------------------------------------- routing
@_timed
def count_cumsum(x: torch.Tensor, E: int, do_cumsum: bool = True):
    _cuda(x)
    if x.dtype not in (torch.int32, torch.int64):
        raise ValueError(f"count_cumsum: expected int32/int64 ids, got {x.dtype}")
    count = torch.empty(E, dtype=_I32, device=x.device)
    cum = torch.empty(E, dtype=_I32, device=x.device) if do_cumsum else None
    check(lib.smoe_count_cumsum(_p(x), int(x.dtype == torch.int64), x.numel(), E, _p(count), _p(cum), _stream()),
          "count_cumsum")
    return (count, cum) if do_cumsum else count


@_timed
def topk_metadata(idx, probs, E, alignment=128, TK_alloc=None, TKp_alloc=None, lane_order=0, pad_mode=0):
    """Returns dict(efo, x_gather_idx, s_scatter_idx, s_reverse_scatter_idx, naept, topk_scores,
    score_src_idx, counts).  Default sizing is the sync-free upper bound."""
    _cuda(idx, probs)
    if idx.dtype != _I32:
        raise ValueError(f"dispatched_indices: expected int32, got {idx.dtype}")
    if probs.dtype != torch.float32:
        raise ValueError(f"dispatched_probs: expected float32, got {probs.dtype}")
    if idx.ndim != 2 or probs.shape != idx.shape:
        raise ValueError(f"shape mismatch: indices={tuple(idx.shape)} vs probs={tuple(probs.shape)}")
    N, K = idx.shape
    if TK_alloc is None:
        TK_alloc = N * min(K, E)
    if TKp_alloc is None:
        TKp_alloc = -(-TK_alloc // alignment) * alignment + E * alignment
    dev = idx.device
    e = lambda n, dt=_I32: torch.empty(max(int(n), 0), dtype=dt, device=dev)
    out = dict(efo=e(E + 1), x_gather_idx=e(TKp_alloc), s_scatter_idx=e(TKp_alloc),
               s_reverse_scatter_idx=e(TK_alloc), naept=e(N + 1), topk_scores=e(TKp_alloc, torch.float32),
               score_src_idx=e(TK_alloc), counts=e(E))
    ws = e(lib.smoe_topk_metadata_workspace(N, E), _U8)
    check(lib.smoe_topk_metadata(_p(idx), _p(probs), N, K, E, alignment, TK_alloc, TKp_alloc, lane_order, pad_mode,
                                 _p(out["efo"]), _p(out["x_gather_idx"]), _p(out["s_scatter_idx"]),
                                 _p(out["s_reverse_scatter_idx"]), _p(out["naept"]), _p(out["topk_scores"]),
                                 _p(out["score_src_idx"]), _p(out["counts"]), _p(ws), _stream()), "topk_metadata")
    out["TK_alloc"], out["TKp_alloc"] = TK_alloc, TKp_alloc
    return out


# ---------------------------------------------------------------- expert-parallel planning
def ep_plan_dest(idx, E, world):
    """idx i32 [T,K] -> (dest_u i32 [T,K]: owning rank per slot, first slot per rank only; pairs i32 [E])."""
    _cuda(idx)
    T, K = idx.shape
    dest_u = torch.empty(T, K, dtype=_I32, device=idx.device)
    pairs = torch.empty(E, dtype=_I32, device=idx.device)
    check(lib.smoe_ep_plan_dest(_p(idx), T, K, E, world, _p(dest_u), _p(pairs), _stream()), "ep_plan_dest")
    return dest_u, pairs


def ep_plan_send_idx(idx, send_tok, efo, n_send, E, world):
    """-> (send_idx i32 [n_send,K] local expert ids per outgoing row, send_rank i32 [n_send])."""
    _cuda(idx, send_tok, efo)
    K = idx.shape[1]
    send_idx = torch.empty(n_send, K, dtype=_I32, device=idx.device)
    send_rank = torch.empty(n_send, dtype=_I32, device=idx.device)
    check(lib.smoe_ep_plan_send_idx(_p(idx), _p(send_tok), _p(efo), n_send, K, E, world, _p(send_idx),
                                    _p(send_rank), _stream()), "ep_plan_send_idx")
    return send_idx, send_rank


@_timed
def ep_combine_pull(peer_ptrs, first_row, send_off, copy_pos, copy_off, send_rank, T, H, device):
    """Sum every token's partial-output rows straight from the owning ranks' buffers (peer_ptrs: device addresses of
    their bf16 [rows,H] buffers in this process; first_row / send_off: host ints per rank) -> bf16 [T,H]."""
    import ctypes
    _cuda(copy_pos, copy_off, send_rank)
    world = len(peer_ptrs)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    bases = (ctypes.c_void_p * world)(*[int(p) for p in peer_ptrs])
    fr = (ctypes.c_int32 * world)(*[int(v) for v in first_row])
    so = (ctypes.c_int32 * world)(*[int(v) for v in send_off])
    check(lib.smoe_ep_combine_pull(bases, fr, so, world, _p(copy_pos), _p(copy_off), _p(send_rank), _p(out), T, H,
                                   _stream()), "ep_combine_pull")
    return out


@_timed
def ep_dispatch_pull(peer_ptrs, recv_counts, src_off, rank, layout, H, K, device, with_meta=True):
    """Fetch the rows addressed to this rank straight from the sources' mapped buffers (peer_ptrs: their device
    addresses in this process; recv_counts / src_off: host ints per source; layout: byte offsets (q, raw, tok, idx,
    probs) inside every buffer) -> (e4m3 rows [n,H], raw scales [n,H/32], local expert ids [n,K] | None,
    probabilities [n,K] | None), sources ascending."""
    import ctypes
    world = len(peer_ptrs)
    n = int(sum(recv_counts))
    q = torch.empty(n, H, dtype=_U8, device=device)
    raw = torch.empty(n, H // 32, dtype=_U8, device=device)
    idx = torch.empty(n, K, dtype=_I32, device=device) if with_meta else None
    p = torch.empty(n, K, dtype=torch.float32, device=device) if with_meta else None
    bases = (ctypes.c_void_p * world)(*[int(v) for v in peer_ptrs])
    rc = (ctypes.c_int32 * world)(*[int(v) for v in recv_counts])
    so = (ctypes.c_int32 * world)(*[int(v) for v in src_off])
    oq, oraw, otok, oidx, oprobs = (int(v) for v in layout)
    check(lib.smoe_ep_dispatch_pull(bases, rc, so, world, int(rank), oq, oraw, otok, oidx, oprobs, H, K, _p(q), _p(raw), _p(idx),
                                    _p(p), _stream()), "ep_dispatch_pull")
    return q, raw, idx, p


def ep_tables(peer_ptrs, rank, off_counts, off_seg, device):
    """This rank's receive / send offset tables, built on the device from the counts every rank left in its mapped
    buffer -> opaque u8 tensor for `ep_dispatch_pull_dev` / `ep_combine_pull_dev`."""
    import ctypes
    world = len(peer_ptrs)
    tab = torch.empty(int(lib.smoe_ep_tables_bytes()), dtype=_U8, device=device)
    bases = (ctypes.c_void_p * world)(*[int(v) for v in peer_ptrs])
    check(lib.smoe_ep_tables(bases, world, int(rank), int(off_counts), int(off_seg), _p(tab), _stream()), "ep_tables")
    return tab


@_timed
def ep_dispatch_pull_dev(peer_ptrs, tables, rank, layout, H, K, n_bound, device, with_meta=True):
    """`ep_dispatch_pull` with device-side counts: outputs have `n_bound` rows; rows beyond what arrived carry
    idx -1 / probability 0 and an unwritten payload."""
    import ctypes
    world = len(peer_ptrs)
    q = torch.empty(n_bound, H, dtype=_U8, device=device)
    raw = torch.empty(n_bound, H // 32, dtype=_U8, device=device)
    idx = torch.empty(n_bound, K, dtype=_I32, device=device) if with_meta else None
    p = torch.empty(n_bound, K, dtype=torch.float32, device=device) if with_meta else None
    bases = (ctypes.c_void_p * world)(*[int(v) for v in peer_ptrs])
    oq, oraw, otok, oidx, oprobs = (int(v) for v in layout)
    check(lib.smoe_ep_dispatch_pull_dev(bases, _p(tables), world, int(rank), oq, oraw, otok, oidx, oprobs, H, K,
                                        n_bound, _p(q), _p(raw), _p(idx), _p(p), _stream()), "ep_dispatch_pull_dev")
    return q, raw, idx, p


@_timed
def ep_combine_pull_dev(peer_ptrs, tables, copy_pos, copy_off, send_rank, T, H, device):
    """`ep_combine_pull` with its offset tables read from device memory."""
    import ctypes
    _cuda(copy_pos, copy_off, send_rank)
    world = len(peer_ptrs)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=device)
    bases = (ctypes.c_void_p * world)(*[int(p) for p in peer_ptrs])
    check(lib.smoe_ep_combine_pull_dev(bases, _p(tables), world, _p(copy_pos), _p(copy_off), _p(send_rank), _p(out), T,
                                       H, _stream()), "ep_combine_pull_dev")
    return out


# ---------------------------------------------------------------- quantizers
@_timed
def quant_rows(x, raw=True, isa=False, out=None):
    """bf16 [M,K] -> (e4m3 bytes [M,K] u8, raw scales [M,K/32] u8 | None, ISA scales u8 | None).  `out` = (q, raw)
    u8 buffers of those shapes to fill instead of fresh allocations."""
    _cuda(x)
    assert x.dtype == torch.bfloat16 and x.ndim == 2
    M, K = x.shape
    if out is not None:
        q, r = out
        _cuda(q, r)
        assert q.dtype == _U8 and tuple(q.shape) == (M, K) and r.dtype == _U8 and tuple(r.shape) == (M, K // 32)
        i = torch.empty(isa_bytes(M, K), dtype=_U8, device=x.device) if isa else None
        check(lib.smoe_quant_rows(_p(x), M, K, _p(q), _p(r), _p(i), _stream()), "quant_rows")
        return q, r, i
    q = torch.empty(M, K, dtype=_U8, device=x.device)
    r = torch.empty(M, K // 32, dtype=_U8, device=x.device) if raw else None
    i = torch.empty(isa_bytes(M, K), dtype=_U8, device=x.device) if isa else None
    check(lib.smoe_quant_rows(_p(x), M, K, _p(q), _p(r), _p(i), _stream()), "quant_rows")
    return q, r, i


@_timed
def quant_rows_gather(x, idx, rows, valid_rows=None):
    """bf16 [T,K] -> (e4m3 of x[idx] [rows,K], ISA scales of (rows,K)) in one pass."""
    _cuda(x, idx, valid_rows)
    assert x.dtype == torch.bfloat16 and x.ndim == 2
    K = x.shape[1]
    q = torch.empty(rows, K, dtype=_U8, device=x.device)
    isa = torch.empty(isa_bytes(rows, K), dtype=_U8, device=x.device)
    check(lib.smoe_quant_rows_gather(_p(x), _p(idx), _p(valid_rows), rows, K, _p(q), _p(isa), _stream()),
          "quant_rows_gather")
    return q, isa


@_timed
def quant_dual_gather(x, idx, rows, valid_rows=None, with_rows=True):
    """bf16 [T,K] -> gathered rows x[idx] quantised row-wise (e4m3 [rows,K] + ISA scales of (rows,K); skipped when
    with_rows is false) and column-wise (e4m3 [rows,K], not transposed, + ISA scales of (K,rows))."""
    _cuda(x, idx, valid_rows)
    assert x.dtype == torch.bfloat16 and x.ndim == 2
    K = x.shape[1]
    dev = x.device
    q_row = torch.empty(rows, K, dtype=_U8, device=dev) if with_rows else None
    row_isa = torch.empty(isa_bytes(rows, K), dtype=_U8, device=dev) if with_rows else None
    q_col = torch.empty(rows, K, dtype=_U8, device=dev)
    col_isa = torch.empty(isa_bytes(K, rows), dtype=_U8, device=dev)
    check(lib.smoe_quant_dual_gather(_p(x), _p(idx), _p(valid_rows), rows, K, _p(q_row), _p(row_isa), _p(q_col),
                                     _p(col_isa), _stream()), "quant_dual_gather")
    return q_row, row_isa, q_col, col_isa


@_timed
def quant_rows_scatter(x, naept, s_rev, s_scatter_idx, rows, valid_rows=None):
    """bf16 [T,K] -> (e4m3 rows in expert-sorted order [rows,K], ISA scales of (rows,K)); each token is
    quantised once and written to all its positions; pad rows are zero."""
    _cuda(x, naept, s_rev, s_scatter_idx, valid_rows)
    assert x.dtype == torch.bfloat16 and x.ndim == 2
    T, K = x.shape
    q = torch.empty(rows, K, dtype=_U8, device=x.device)
    isa = torch.empty(isa_bytes(rows, K), dtype=_U8, device=x.device)
    check(lib.smoe_quant_rows_scatter(_p(x), T, K, _p(naept), _p(s_rev), _p(s_scatter_idx), _p(valid_rows), rows,
                                      _p(q), _p(isa), _stream()), "quant_rows_scatter")
    return q, isa


@_timed
def gather_scales_isa(raw, idx, rows, cols):
    _cuda(raw, idx)
    out = torch.empty(isa_bytes(rows, cols), dtype=_U8, device=raw.device)
    check(lib.smoe_gather_scales_isa(_p(raw), _p(idx), rows, cols, _p(out), _stream()), "gather_scales_isa")
    return out


@_timed
def gather_rows_fp8(q, raw, idx, rows, valid_rows=None):
    """q u8 [T,K], raw scales u8 [T,K/32] -> (q[idx] [rows,K], ISA scales of (rows,K))."""
    _cuda(q, raw, idx, valid_rows)
    K = q.shape[1]
    out = torch.empty(rows, K, dtype=_U8, device=q.device)
    isa = torch.empty(isa_bytes(rows, K), dtype=_U8, device=q.device)
    check(lib.smoe_gather_rows_fp8(_p(q), _p(raw), _p(idx), _p(valid_rows), rows, K, _p(out), _p(isa), _stream()),
          "gather_rows_fp8")
    return out, isa


@_timed
def scatter_rows_fp8(q, raw, naept, s_rev, s_scatter_idx, rows, valid_rows=None, with_scales=True):
    """q u8 [T,K], raw scales u8 [T,K/32] -> (rows in expert-sorted order [rows,K], ISA scales of (rows,K)); each
    source row is read once and written to all its positions; pad rows are zero.  `with_scales=False`: payload
    only (the second result is None), for a caller that already holds the packed scales."""
    _cuda(q, raw, naept, s_rev, s_scatter_idx, valid_rows)
    T, K = q.shape
    out = torch.empty(rows, K, dtype=_U8, device=q.device)
    isa = torch.empty(isa_bytes(rows, K), dtype=_U8, device=q.device) if with_scales else None
    if not with_scales:
        raw = None
    check(lib.smoe_scatter_rows_fp8(_p(q), _p(raw), T, K, _p(naept), _p(s_rev), _p(s_scatter_idx), _p(valid_rows),
                                    rows, _p(out), _p(isa), _stream()), "scatter_rows_fp8")
    return out, isa


@_timed
def quant_cols_t(src, idx, rows, out=None, valid_rows=None):
    """bf16 [T,dim] (rows gathered by idx, or None) -> (e4m3 bytes [dim, rows], ISA scales for (dim, rows)); `out` =
    (q_t, isa) places the results in caller-owned buffers (slices of a stacked tensor); `valid_rows` (device int):
    row tiles at or beyond it are skipped."""
    _cuda(src, idx, valid_rows)
    assert src.dtype == torch.bfloat16
    dim = src.shape[1]
    if out is not None:
        q_t, isa = out
        _cuda(q_t, isa)
        assert q_t.dtype == _U8 and tuple(q_t.shape) == (dim, rows) and isa.numel() == isa_bytes(dim, rows)
    else:
        q_t = torch.empty(dim, rows, dtype=_U8, device=src.device)
        isa = torch.empty(isa_bytes(dim, rows), dtype=_U8, device=src.device)
    check(lib.smoe_quant_cols_t(_p(src), _p(idx), _p(valid_rows), rows, dim, _p(q_t), _p(isa), _stream()),
          "quant_cols_t")
    return q_t, isa


@_timed
def requant_cols_t(src_q, src_raw, idx, rows, valid_rows=None):
    """e4m3 bytes [T,dim] + raw row scales [T,dim/32] -> (e4m3 [dim, rows], ISA scales for (dim, rows)); `valid_rows`
    (device int): row tiles at or beyond it are skipped."""
    _cuda(src_q, src_raw, idx, valid_rows)
    dim = src_q.shape[1]
    q_t = torch.empty(dim, rows, dtype=_U8, device=src_q.device)
    isa = torch.empty(isa_bytes(dim, rows), dtype=_U8, device=src_q.device)
    check(lib.smoe_requant_cols_t(_p(src_q), _p(src_raw), _p(idx), _p(valid_rows), rows, dim, _p(q_t), _p(isa),
                                  _stream()),
          "requant_cols_t")
    return q_t, isa


@_timed
def quant_iso32(x, transposed_payload=True, out=None):
    """bf16 [rows, cols] -> (q [rows,cols], row ISA, q_t [cols,rows] or None, col ISA); one scale per 32x32 block.
    `out` = (q, row ISA, col ISA) buffers to fill (then no transposed payload is written)."""
    _cuda(x)
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    rows, cols = x.shape
    dev = x.device
    if out is not None:
        q, ri, ci = out
        q_t = None
        assert q.is_contiguous() and q.numel() == rows * cols and ri.numel() == isa_bytes(rows, cols) \
            and ci.numel() == isa_bytes(cols, rows)
    else:
        q = torch.empty(rows, cols, dtype=_U8, device=dev)
        q_t = torch.empty(cols, rows, dtype=_U8, device=dev) if transposed_payload else None
        ri = torch.empty(isa_bytes(rows, cols), dtype=_U8, device=dev)
        ci = torch.empty(isa_bytes(cols, rows), dtype=_U8, device=dev)
    check(lib.smoe_quant_iso32(_p(x), rows, cols, _p(q), _p(ri), _p(q_t), _p(ci), _stream()), "quant_iso32")
    return q, ri, q_t, ci


@_timed
def transpose_u8(src):
    """u8 [B, R, C] -> u8 [B, C, R] (R, C multiples of 64)."""
    _cuda(src)
    assert src.dtype == _U8 and src.is_contiguous() and src.dim() == 3
    B, R, C = src.shape
    dst = torch.empty(B, C, R, dtype=_U8, device=src.device)
    check(lib.smoe_transpose_u8(_p(src), B, R, C, _p(dst), _stream()), "transpose_u8")
    return dst


# ---------------------------------------------------------------- GEMMs
@_timed
def gemm_varlen_m(a_q, a_sf, b_q, b_sf, efo):
    """a_q u8 [rows,K], b_q u8 [E,N,K] -> bf16 [rows,N]."""
    _cuda(a_q, a_sf, b_q, b_sf, efo)
    rows, K = a_q.shape
    E, N, _ = b_q.shape
    c = torch.empty(rows, N, dtype=torch.bfloat16, device=a_q.device)
    check(lib.smoe_gemm_varlen_m(_p(a_q), _p(a_sf), _p(b_q), _p(b_sf), _p(efo), _p(c), rows, N, K, E,
                                 _p(status_word(a_q.device)), _stream()), "gemm_varlen_m")
    return c


@_timed
def gemm_varlen_m_bt(a_q, a_sf, b_kn_q, b_sf, efo):
    """a_q u8 [rows,K], b_kn_q u8 [E,K,N] (B[e] stored N-contiguous), b_sf ISA scales for (E*N, K) -> bf16 [rows,N]."""
    _cuda(a_q, a_sf, b_kn_q, b_sf, efo)
    rows, K = a_q.shape
    E, Kb, N = b_kn_q.shape
    assert Kb == K
    c = torch.empty(rows, N, dtype=torch.bfloat16, device=a_q.device)
    check(lib.smoe_gemm_varlen_m_bt(_p(a_q), _p(a_sf), _p(b_kn_q), _p(b_sf), _p(efo), _p(c), rows, N, K, E,
                                    _p(status_word(a_q.device)), _stream()), "gemm_varlen_m_bt")
    return c


@_timed
def gemm_gated(x_q, a_idx, a_sf, w1_q, w1_sf, efo, rows, out=None):
    """x_q u8 [T,H], w1_q u8 [E,2I,H] -> z_q [rows,2I], z_sc [rows,2I/32], y1_q [rows,I], y1_sf (ISA).
    `out` = those four as buffers allocated by the caller (any one-byte dtype; sizes checked)."""
    _cuda(x_q, a_idx, a_sf, w1_q, w1_sf, efo)
    if a_idx is None and x_q.shape[0] != rows:
        raise ValueError("gemm_gated without a_idx needs x_q in expert-sorted order [rows, K]")
    T, K = x_q.shape
    E, N, _ = w1_q.shape
    dev = x_q.device
    if out is not None:
        z_q, z_sc, y1_q, y1_sf = (t.view(_U8) for t in out)
        _cuda(z_q, z_sc, y1_q, y1_sf)
        want = (rows * N, rows * (N // 32), rows * (N // 2), isa_bytes(rows, N // 2))
        got = (z_q.numel(), z_sc.numel(), y1_q.numel(), y1_sf.numel())
        if got != want:
            raise ValueError(f"gemm_gated: pre-allocated outputs hold {got} bytes, the call needs {want}")
        z_q, z_sc, y1_q = z_q.view(rows, N), z_sc.view(rows, N // 32), y1_q.view(rows, N // 2)
        y1_sf = y1_sf.view(-1)
    else:
        z_q = torch.empty(rows, N, dtype=_U8, device=dev)
        z_sc = torch.empty(rows, N // 32, dtype=_U8, device=dev)
        y1_q = torch.empty(rows, N // 2, dtype=_U8, device=dev)
        y1_sf = torch.empty(isa_bytes(rows, N // 2), dtype=_U8, device=dev)
    check(lib.smoe_gemm_gated(_p(x_q), T, _p(a_idx), _p(a_sf), _p(w1_q), _p(w1_sf), _p(efo), _p(z_q), _p(z_sc),
                              _p(y1_q), _p(y1_sf), rows, N, K, E, _p(status_word(dev)), _stream()), "gemm_gated")
    return z_q, z_sc, y1_q, y1_sf


@_timed
def gemm_dgated(dout_q, a_idx, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, rows):
    """dout_q u8 [T,H], w2t_q u8 [E,I,H] -> dz bf16 [rows,2I], y1s bf16 [rows,I], ds_partial f32 [parts, rows]."""
    _cuda(dout_q, a_idx, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s)
    if a_idx is None and dout_q.shape[0] != rows:
        raise ValueError("gemm_dgated without a_idx needs dout_q in expert-sorted order [rows, K]")
    T, K = dout_q.shape
    E, N, _ = w2t_q.shape
    dev = dout_q.device
    parts = lib.smoe_gemm_dgated_partials(N)
    dz = torch.empty(rows, 2 * N, dtype=torch.bfloat16, device=dev)
    y1s = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
    dsp = torch.zeros(parts, rows, dtype=torch.float32, device=dev)
    check(lib.smoe_gemm_dgated(_p(dout_q), T, _p(a_idx), _p(a_sf), _p(w2t_q), _p(w2t_sf), _p(efo), _p(z_q), _p(z_sc),
                               _p(s), _p(dz), _p(y1s), _p(dsp), None, rows, N, K, E, _p(status_word(dev)),
                               _stream()), "gemm_dgated")
    return dz, y1s, dsp


@_timed
def gemm_dgated_fused(dg_q, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, rows, a_idx=None):
    """GemmDGated with fused operand quantizers.  dg_q u8 [rows,H] (expert-sorted) - or, with a_idx, the un-gathered
    [T,H] whose rows the kernel fetches by index - w2t_q u8 [E,I,H] ->
    (dz_q [rows,2I], dz ISA scales for (rows,2I), dz ISA scales for (2I,rows), y1s_q [rows,I], y1s ISA scales for
    (I,rows), ds_partial).  dz_q / y1s_q stay row-major; gemm_wgrad_mn takes them as they are."""
    _cuda(dg_q, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, a_idx)
    K = dg_q.shape[1]
    E, N, _ = w2t_q.shape
    dev = dg_q.device
    parts = lib.smoe_gemm_dgated_fused_partials(N)
    dz_q = torch.empty(rows, 2 * N, dtype=_U8, device=dev)
    y1s_q = torch.empty(rows, N, dtype=_U8, device=dev)
    dz_rsf = torch.empty(isa_bytes(rows, 2 * N), dtype=_U8, device=dev)
    dz_csf = torch.empty(isa_bytes(2 * N, rows), dtype=_U8, device=dev)
    y1s_sf = torch.empty(isa_bytes(N, rows), dtype=_U8, device=dev)
    dsp = torch.zeros(parts, rows, dtype=torch.float32, device=dev)
    if a_idx is not None:
        check(lib.smoe_gemm_dgated_fused_gather(_p(dg_q), dg_q.shape[0], _p(a_idx), _p(a_sf), _p(w2t_q), _p(w2t_sf),
                                                _p(efo), _p(z_q), _p(z_sc), _p(s), _p(dz_q), _p(dz_rsf), _p(dz_csf),
                                                _p(y1s_q), _p(y1s_sf), _p(dsp), rows, N, K, E,
                                                _p(status_word(dev)), _stream()), "gemm_dgated_fused_gather")
        return dz_q, dz_rsf, dz_csf, y1s_q, y1s_sf, dsp
    check(lib.smoe_gemm_dgated_fused(_p(dg_q), _p(a_sf), _p(w2t_q), _p(w2t_sf), _p(efo), _p(z_q), _p(z_sc), _p(s),
                                     _p(dz_q), _p(dz_rsf), _p(dz_csf), _p(y1s_q), _p(y1s_sf), _p(dsp),
                                     rows, N, K, E, _p(status_word(dev)), _stream()), "gemm_dgated_fused")
    return dz_q, dz_rsf, dz_csf, y1s_q, y1s_sf, dsp


@_timed
def gemm_wgrad(a_t, a_sf, b_t, b_sf, efo, out, accumulate):
    """a_t u8 [M,TKp], b_t u8 [N,TKp]; out f32 [E,M,N] (+)= per-expert products."""
    _cuda(a_t, a_sf, b_t, b_sf, efo, out)
    M, TKp = a_t.shape
    N = b_t.shape[0]
    E = out.shape[0]
    assert out.dtype == torch.float32 and out.shape == (E, M, N)
    check(lib.smoe_gemm_wgrad(_p(a_t), _p(a_sf), _p(b_t), _p(b_sf), _p(efo), _p(out), M, N, TKp, E, int(accumulate),
                              _p(status_word(a_t.device)), _stream()), "gemm_wgrad")
    return out


@_timed
def gemm_wgrad_mn(a, a_sf, b, b_sf, efo, out, accumulate, a_rowmajor_tk, b_rowmajor_tk):
    """Weight gradient with either operand kept as u8 [TKp, dim] (row = routed position) instead of [dim, TKp];
    out f32 [E,M,N] (+)= per-expert products.  Needs M, N multiples of 256."""
    _cuda(a, a_sf, b, b_sf, efo, out)
    E, M, N = out.shape
    TKp = a.shape[0] if a_rowmajor_tk else a.shape[1]
    assert tuple(a.shape) == ((TKp, M) if a_rowmajor_tk else (M, TKp))
    assert tuple(b.shape) == ((TKp, N) if b_rowmajor_tk else (N, TKp))
    assert out.dtype == torch.float32
    layout = (1 if a_rowmajor_tk else 0) | (2 if b_rowmajor_tk else 0)
    check(lib.smoe_gemm_wgrad_mn(_p(a), _p(a_sf), _p(b), _p(b_sf), _p(efo), _p(out), M, N, TKp, E, int(accumulate),
                                 layout, _p(status_word(a.device)), _stream()), "gemm_wgrad_mn")
    return out


@_timed
def gemm_wgrad_pair(a1, a1_sf, b1, b1_sf, out1, a2, a2_sf, b2, b2_sf, out2, efo, accumulate, a_rowmajor_tk):
    """Two weight gradients in one launch (256 x 384 kernel): out1 [E,M1,N] (+)= A1^T B1 and out2 [E,M2,N] (+)= A2^T B2
    over the same expert segments.  A operands u8 [TKp, M] (a_rowmajor_tk) or [M, TKp]; B operands u8 [N, TKp];
    N % 384 == 0, M1, M2 % 256 == 0."""
    _cuda(a1, a1_sf, b1, b1_sf, out1, a2, a2_sf, b2, b2_sf, out2, efo)
    E, M1, N = out1.shape
    E2, M2, N2 = out2.shape
    TKp = b1.shape[1]
    assert (E2, N2) == (E, N) and tuple(b1.shape) == (N, TKp) and tuple(b2.shape) == (N, TKp)
    assert tuple(a1.shape) == ((TKp, M1) if a_rowmajor_tk else (M1, TKp))
    assert tuple(a2.shape) == ((TKp, M2) if a_rowmajor_tk else (M2, TKp))
    assert out1.dtype == torch.float32 and out2.dtype == torch.float32
    check(lib.smoe_gemm_wgrad_mn_pair(_p(a1), _p(a1_sf), _p(b1), _p(b1_sf), _p(out1), M1, _p(a2), _p(a2_sf), _p(b2),
                                      _p(b2_sf), _p(out2), M2, _p(efo), N, TKp, E, int(accumulate),
                                      int(bool(a_rowmajor_tk)), _p(status_word(a1.device)), _stream()),
          "gemm_wgrad_pair")
    return out1, out2


# ---------------------------------------------------------------- gated activations outside the GEMMs
@_timed
def glu_fwd(z, act):
    """z bf16 [rows,2I] -> (z_q [rows,2I], z_sc raw [rows,2I/32], y1_q [rows,I], y1_sf ISA); act 0 swiglu, 1 reglu,
    2 geglu."""
    _cuda(z)
    assert z.dtype == torch.bfloat16 and z.ndim == 2
    rows, N = z.shape
    I = N // 2
    dev = z.device
    z_q = torch.empty(rows, N, dtype=_U8, device=dev)
    z_sc = torch.empty(rows, N // 32, dtype=_U8, device=dev)
    y1_q = torch.empty(rows, I, dtype=_U8, device=dev)
    y1_sf = torch.empty(isa_bytes(rows, I), dtype=_U8, device=dev)
    check(lib.smoe_glu_fwd(_p(z), rows, I, int(act), _p(z_q), _p(z_sc), _p(y1_q), _p(y1_sf), _stream()), "glu_fwd")
    return z_q, z_sc, y1_q, y1_sf


@_timed
def glu_bwd(D, z_q, z_sc, s, act):
    """D bf16 [rows,I], saved z (e4m3 + raw scales), row scores -> (dz bf16 [rows,2I], y1s bf16 [rows,I],
    ds partial f32 [1, rows])."""
    _cuda(D, z_q, z_sc, s)
    rows, I = D.shape
    dev = D.device
    dz = torch.empty(rows, 2 * I, dtype=torch.bfloat16, device=dev)
    y1s = torch.empty(rows, I, dtype=torch.bfloat16, device=dev)
    dsp = torch.empty(1, rows, dtype=torch.float32, device=dev)
    check(lib.smoe_glu_bwd(_p(D), _p(z_q), _p(z_sc), _p(s), rows, I, int(act), _p(dz), _p(y1s), _p(dsp), _stream()),
          "glu_bwd")
    return dz, y1s, dsp


# ---------------------------------------------------------------- token side
@_timed
def combine(y, s_rev, naept, scores, T, out=None):
    """out[t] = sum over the token's lanes of scores * y[row] (bf16, fp32 accumulate); `out` places the result in a
    caller-owned bf16 [T,H] buffer (e.g. memory that peer GPUs read)."""
    _cuda(y, s_rev, naept, scores)
    H = y.shape[1]
    if out is None:
        out = torch.empty(T, H, dtype=torch.bfloat16, device=y.device)
    elif out.dtype != torch.bfloat16 or tuple(out.shape) != (T, H) or not out.is_contiguous() or not out.is_cuda:
        raise ValueError(f"combine: out must be contiguous CUDA bf16 [{T},{H}]")
    check(lib.smoe_combine(_p(y), _p(s_rev), _p(naept), _p(scores), _p(out), T, H, _stream()), "combine")
    return out


@_timed
def gather_scores(scores, s_scatter_idx):
    _cuda(scores, s_scatter_idx)
    rows = s_scatter_idx.numel()
    s = torch.empty(rows, dtype=torch.float32, device=scores.device)
    check(lib.smoe_gather_scores(_p(scores), _p(s_scatter_idx), rows, _p(s), _stream()), "gather_scores")
    return s


@_timed
def ds_finalize(ds_partial, s_rev, TK, real_tk=None, src_idx=None, scatter_numel=0):
    """Token-major ds [TK]; with src_idx also the scatter into a zeroed [scatter_numel] buffer."""
    _cuda(ds_partial, s_rev, real_tk, src_idx)
    parts, rows = ds_partial.shape
    out = torch.empty(TK, dtype=torch.float32, device=ds_partial.device)
    sc = torch.zeros(scatter_numel, dtype=torch.float32, device=ds_partial.device) if src_idx is not None else None
    check(lib.smoe_ds_finalize(_p(ds_partial), parts, rows, _p(s_rev), TK, _p(real_tk), _p(out), _p(src_idx), _p(sc),
                               _stream()), "ds_finalize")
    return out, sc


@_timed
def topk_softmax(logits, K):
    _cuda(logits)
    assert logits.dtype == torch.float32 and logits.ndim == 2
    T, E = logits.shape
    scores = torch.empty(T, K, dtype=torch.float32, device=logits.device)
    idx = torch.empty(T, K, dtype=_I32, device=logits.device)
    check(lib.smoe_topk_softmax(_p(logits), T, E, K, _p(scores), _p(idx), _stream()), "topk_softmax")
    return scores, idx


@_timed
def topk_softmax_bwd(scores, idx, dscores, E):
    _cuda(scores, idx, dscores)
    T, K = scores.shape
    out = torch.empty(T, E, dtype=torch.float32, device=scores.device)
    check(lib.smoe_topk_softmax_bwd(_p(scores), _p(idx), _p(dscores), T, E, K, _p(out), _stream()), "topk_softmax_bwd")
    return out
