"""Autograd orchestration of the MoE layer on the sm_100a MXFP8 kernels.

Mirrors the reference's functional layer (sonicmoe/functional/__init__.py):
`_UpProjection` / `_DownProjection` autograd Functions with the reference's
argument lists (:828-847, :1617-1640), the FP8 hand-off between them
(:430-502), `main_grad` accumulation (:393-414), `enable_fp8` /
`enable_quack_gemm` (functional/utils.py:15-76) and the dense entry point
`moe_TC_softmax_topk_layer` (call sites sonicmoe/moe.py:604-616).

Dataflow (one code path, MXFP8 1x32 ue8m0 everywhere a GEMM runs):
  forward   x --row quant, written in expert-sorted order--> x_fp8 [TKp,H] + ISA scales
            up-proj GEMM + SwiGLU + z/y1 re-quant in the epilogue
            down-proj GEMM -> y2 bf16 ; top-k weighted combine -> o
  backward  dout row quant (expert-sorted) ; GemmDGated (e4m3 z reload, dSwiGLU, dz / y1s quantizers
            in the epilogue) -> dz, y1s as e4m3, ds
            dgrad GEMM -> dx_expanded ; unweighted combine -> dx
            column quantizers of x / dout (transposed outputs) ; dw2 + dw1 varlen-K GEMMs into fp32
"""
from __future__ import annotations

import os
import weakref
from contextlib import contextmanager

import torch
import torch.nn.functional as F

from .. import ops
from ..config import get_active_config
from ..enums import ActivationType, activation_code, require_swiglu

# ----------------------------------------------------------------------------
# flags (API kept; a single compute path sits behind them)
# ----------------------------------------------------------------------------
_IS_USING_QUACK_GEMM = os.getenv("USE_QUACK_GEMM", "1") == "1"
_IS_FP8_ACTIVE = os.getenv("SONIC_MOE_FP8_MODE", "").strip().lower() in ("perf", "mem")


@contextmanager
def enable_quack_gemm(enable: bool = True):
    global _IS_USING_QUACK_GEMM
    prev = _IS_USING_QUACK_GEMM
    _IS_USING_QUACK_GEMM = enable
    try:
        yield
    finally:
        _IS_USING_QUACK_GEMM = prev


@contextmanager
def enable_fp8(enable: bool = True):
    global _IS_FP8_ACTIVE, _IS_USING_QUACK_GEMM
    prev = (_IS_FP8_ACTIVE, _IS_USING_QUACK_GEMM)
    _IS_FP8_ACTIVE = enable
    if enable:
        _IS_USING_QUACK_GEMM = True
    try:
        yield
    finally:
        _IS_FP8_ACTIVE, _IS_USING_QUACK_GEMM = prev


def is_fp8_active() -> bool:
    cfg = get_active_config()
    if cfg is not None and cfg.use_fp8 is not None:
        return cfg.use_fp8
    return _IS_FP8_ACTIVE


def is_using_quack_gemm() -> bool:
    cfg = get_active_config()
    if cfg is not None and cfg.use_quack_gemm is not None:
        return cfg.use_quack_gemm
    return _IS_USING_QUACK_GEMM


def _require_fp8():
    if not is_fp8_active():
        raise NotImplementedError(
            "this build implements the MXFP8 path of the MoE layer only: wrap the call in enable_fp8(), pass "
            "use_fp8=True / fp8=True, or activate SonicMoEConfig(use_fp8=True) (the BF16 GEMM path is out of scope)")


# How the up-projection and GemmDGated get their A rows (row p of the GEMM = activation row x_gather_idx[p]):
#   "copy"     the row quantizer writes an expert-sorted e4m3 copy [TKp,H], loaded as plain TMA tiles
#   "cpasync"  the activation is quantised once as [T,H]; four load warps per CTA fetch the rows by index inside the
#              GEMM (no [TKp,H] copy is written or read); only the scales are gathered (1/32 of the bytes)
# ("1" in SONIC_MOE_TMA_GATHER is the older spelling of in-kernel gathering)
A_GATHER = os.getenv("SONIC_MOE_A_GATHER", "cpasync" if os.getenv("SONIC_MOE_TMA_GATHER", "0") == "1" else "copy")
if A_GATHER not in ("copy", "cpasync"):
    raise ValueError(f"SONIC_MOE_A_GATHER={A_GATHER!r}: expected 'copy' or 'cpasync'")
USE_TMA_GATHER = A_GATHER == "cpasync"          # in-kernel gathering of A rows
# GemmDGated emits the e4m3 operands of the three GEMMs that follow it (dgrad, dw1, dw2) straight from its
# epilogue instead of bf16 dz / y1s plus separate quantizer passes (same bytes either way).
FUSE_DGATED_QUANT = os.getenv("SONIC_MOE_FUSE_DGATED_QUANT", "1") == "1"
# With a main_grad accumulator the dw2 GEMM is run by _UpProjection.backward after dx (see there); "0" keeps it in
# _DownProjection.backward (needed only if a caller differentiates with respect to w2 alone, so that the first
# Function's backward never runs).
_DEFER_DW2 = os.getenv("SONIC_MOE_DEFER_DW2", "1") == "1"
# A deferred dw2 and dw1 run as ONE launch of the 256 x 384 kernel when both accumulate into main_grad and their
# shapes allow it: the two tile counts then leave one partly filled last wave instead of one each.
_PAIR_WGRADS = os.getenv("SONIC_MOE_PAIR_WGRADS", "1") == "1"


def _mn_wgrad_ok(E: int, M: int, N: int) -> bool:
    """Shapes the weight-gradient GEMM accepts with operands left [TKp, dim] (MN-major)."""
    return E <= 256 and M % 256 == 0 and N % 256 == 0


def _wide_wgrad_ok(E: int, M: int, N: int) -> bool:
    """Shapes the 256 x 384 weight-gradient kernel takes (fewest operand bytes per MMA): its A operand may stay
    [TKp, M], its B operand must be K-major, i.e. the column quantizer writes it transposed [N, TKp]."""
    return E <= 256 and M % 256 == 0 and N % 384 == 0


def _col_operand(src, idx, TKp, valid_rows, E, M, N):
    """Column-quantised (1x32 along the routed rows) B operand of a weight-gradient GEMM from bf16 `src` rows
    gathered by `idx`: (payload, ISA scales for (N, TKp), payload_is_rows_major)."""
    if _mn_wgrad_ok(E, M, N) and not _wide_wgrad_ok(E, M, N):
        _, _, q, sf = ops.quant_dual_gather(src, idx, TKp, valid_rows, with_rows=False)
        return q, sf, True
    q_t, sf = ops.quant_cols_t(src, idx, TKp, valid_rows=valid_rows)
    return q_t, sf, False


def _wgrad(a, a_sf, a_rows_tk, b, b_sf, b_rows_tk, efo, out, accumulate):
    """out[e] (+)= A_e^T B_e over expert e's rows; either operand is [dim, TKp] or, *_rows_tk, [TKp, dim]."""
    if a_rows_tk or b_rows_tk:
        ops.gemm_wgrad_mn(a, a_sf, b, b_sf, efo, out, accumulate, a_rows_tk, b_rows_tk)
    else:
        ops.gemm_wgrad(a, a_sf, b, b_sf, efo, out, accumulate=accumulate)


# ----------------------------------------------------------------------------
# FP8 weight cache (four row-wise 1x32 layouts, refreshed when a weight's
# version counter moves, i.e. once per optimizer step)
# ----------------------------------------------------------------------------
_WEIGHT_CACHE: dict = {}
_WEIGHT_CACHE_MAX = 256


def _base_of(w: torch.Tensor) -> torch.Tensor:
    return w._base if w._base is not None else w


def weight_fp8(w: torch.Tensor, transposed: bool):
    """w [E,N,K] bf16 -> (e4m3 bytes [E,N,K], ISA scales) or, transposed, the same for w^T [E,K,N].
    Replaces precompute_weight_fp8_warmup / the per-weight caches
    (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:299-345,4363-4406)."""
    base = _base_of(w)
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()), transposed, w.device.index)
    ver = base._version
    hit = _WEIGHT_CACHE.get(key)
    # address + version are not enough: a freed weight's address is handed out again by the caching allocator,
    # with a fresh version counter that can coincide - the entry also remembers WHICH tensor it was made from
    if hit is not None and hit[0] == ver and hit[3]() is base:
        return hit[1], hit[2]
    with torch.no_grad():
        src = w.detach()
        if src.dtype != torch.bfloat16:
            src = src.to(torch.bfloat16)
        src = src.contiguous()
        E, N, K = src.shape
        if transposed and N % 128 == 0 and K % 128 == 0:
            # W^T quantised row-wise (1x32 along N) is W quantised column-wise (32 consecutive rows of W) with the
            # bytes written transposed: the column quantizer reads W as it lies and no transposed bf16 copy is made
            # (the reference reads each weight once for both orientations, blockscaled_fp8_gemm.py:4243-4315)
            q = torch.empty(E, K, N, dtype=torch.uint8, device=src.device)
            per = ops.isa_bytes(K, N)
            sf = torch.empty(E * per, dtype=torch.uint8, device=src.device)
            for e in range(E):
                ops.quant_cols_t(src[e], None, N, out=(q[e], sf[e * per:(e + 1) * per]))
        else:
            if transposed:
                src = src.transpose(1, 2).contiguous()
                E, N, K = src.shape
            q, _, sf = ops.quant_rows(src.view(E * N, K), raw=False, isa=True)
            q = q.view(E, N, K)
    if len(_WEIGHT_CACHE) >= _WEIGHT_CACHE_MAX:
        _WEIGHT_CACHE.pop(next(iter(_WEIGHT_CACHE)))
    _WEIGHT_CACHE[key] = (ver, q, sf, weakref.ref(base))
    return q, sf


def _iso32_ok(w: torch.Tensor) -> bool:
    return w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0


def weight_fp8_iso32(w: torch.Tensor):
    """w [E,N,K] bf16 -> (e4m3 bytes [E,N,K], ISA scales for (E*N, K), ISA scales for (E*K, N)) with ONE scale per
    32x32 block: the one payload is W K-major for the forward GEMM and, read N-contiguous, W^T for the backward
    one, so half the FP8 weight memory of the two 1x32 copies (the reference's ISO32 weight cache,
    sonicmoe/quack_utils/blockscaled_fp8_gemm.py:3765-3856; coarser scales: one per 1024 values instead of 32)."""
    base = _base_of(w)
    key = (w.data_ptr(), tuple(w.shape), tuple(w.stride()), "iso32", w.device.index)
    ver = base._version
    hit = _WEIGHT_CACHE.get(key)
    if hit is not None and hit[0] == ver and hit[3]() is base:
        return hit[1], hit[2][0], hit[2][1]
    with torch.no_grad():
        src = w.detach()
        if src.dtype != torch.bfloat16:
            src = src.to(torch.bfloat16)
        src = src.contiguous()
        E, N, K = src.shape
        q = torch.empty(E, N, K, dtype=torch.uint8, device=src.device)
        per_r, per_c = ops.isa_bytes(N, K), ops.isa_bytes(K, N)
        row_sf = torch.empty(E * per_r, dtype=torch.uint8, device=src.device)
        col_sf = torch.empty(E * per_c, dtype=torch.uint8, device=src.device)
        for e in range(E):
            ops.quant_iso32(src[e], out=(q[e], row_sf[e * per_r:(e + 1) * per_r], col_sf[e * per_c:(e + 1) * per_c]))
    if len(_WEIGHT_CACHE) >= _WEIGHT_CACHE_MAX:
        _WEIGHT_CACHE.pop(next(iter(_WEIGHT_CACHE)))
    _WEIGHT_CACHE[key] = (ver, q, (row_sf, col_sf), weakref.ref(base))
    return q, row_sf, col_sf


def _weight_operand(w: torch.Tensor, transposed: bool, iso32: bool):
    """(payload, ISA scales, stored_kn) of W (or W^T) as the B operand of a GEMM.  `stored_kn`: the payload is the
    single ISO32 buffer, which holds the wanted operand [E, K', N'] with N' contiguous - the caller reads it through
    `_gemm_plain` (MN-major B) or makes a transient byte transpose."""
    if iso32 and _iso32_ok(w):
        q, row_sf, col_sf = weight_fp8_iso32(w)
        return (q, col_sf, True) if transposed else (q, row_sf, False)
    q, sf = weight_fp8(w, transposed)
    return q, sf, False


def _gemm_plain(a_q, a_sf, b_q, b_sf, stored_kn, efo):
    """rows grouped by expert x B[e]^T -> bf16.  `stored_kn`: B lies [E, K, N] (see `_weight_operand`)."""
    if not stored_kn:
        return ops.gemm_varlen_m(a_q, a_sf, b_q, b_sf, efo)
    E, K, N = b_q.shape
    if N % 256 == 0 and E <= 256:
        return ops.gemm_varlen_m_bt(a_q, a_sf, b_q, b_sf, efo)
    return ops.gemm_varlen_m(a_q, a_sf, ops.transpose_u8(b_q), b_sf, efo)     # transient K-major copy


def _modes(fp8_config):
    """(iso32_weight, stagewise_memory) of this call: an explicit config wins, then the active one, then the
    environment."""
    cfg = fp8_config if fp8_config is not None else get_active_config()
    if cfg is None:
        from ..config import SonicMoEConfig
        cfg = SonicMoEConfig()
    return cfg.resolve_iso32_weight(), cfg.resolve_stagewise_memory()


# Per-stage memory record of the memory-lean mode (reference: _log_stage_memory, functional/__init__.py:726-737):
# (stage, bytes allocated, peak bytes allocated since the previous record); each record synchronises the device.
STAGE_MEMORY_LOG: list = []


def _log_stage_memory(enabled: bool, stage: str):
    if not enabled or torch.cuda.is_current_stream_capturing():
        return
    torch.cuda.synchronize()
    STAGE_MEMORY_LOG.append((stage, torch.cuda.memory_allocated(), torch.cuda.max_memory_allocated()))
    if len(STAGE_MEMORY_LOG) > 4096:
        del STAGE_MEMORY_LOG[:2048]
    torch.cuda.reset_peak_memory_stats()


_GATED_OUTPUT_PAYLOAD_ATTR = "_sonic_preallocated_gated_outputs"


def attach_preallocated_gated_outputs(packed_scales: torch.Tensor, outputs):
    """Carry the four per-call up-projection outputs (pre-activation, post-activation, raw pre-activation scales,
    post-activation ISA scales: what `deepep_topk_to_sonic_metadata_with_scales` allocates) on the packed-scales
    tensor of the prequantised payload, so that they need not be explicit autograd inputs
    (sonicmoe/functional/__init__.py:505-513)."""
    if len(outputs) != 4:
        raise ValueError(f"expected four gated outputs, got {len(outputs)}")
    setattr(packed_scales, _GATED_OUTPUT_PAYLOAD_ATTR, tuple(outputs))
    return packed_scales


def precompute_weight_fp8(w1: torch.Tensor, w2: torch.Tensor, iso32_weight: bool | None = None):
    """Fill the cached layouts: W1 (E,2I,H), W1^T (E,H,2I), W2 (E,H,I), W2^T (E,I,H) - or, in ISO32 mode, the one
    buffer per weight."""
    iso = _modes(None)[0] if iso32_weight is None else iso32_weight
    for w in (w1, w2):
        if iso and _iso32_ok(w):
            weight_fp8_iso32(w)
        else:
            weight_fp8(w, False)
            weight_fp8(w, True)


def clear_weight_cache():
    """Forget every cached FP8 weight copy.  Freshness is judged by (address, tensor version counter, identity);
    an in-place update that bypasses the version counter - `param.data.copy_(master)`, the usual pattern of
    master-weight optimizers - is invisible to it, so such a training loop calls this (or `drop_weight_fp8`)
    once per optimizer step."""
    _WEIGHT_CACHE.clear()


def drop_weight_fp8(*weights: torch.Tensor):
    """Forget the cached FP8 copies (both orientations) of the given weights only."""
    for w in weights:
        for transposed in (False, True, "iso32"):
            _WEIGHT_CACHE.pop((w.data_ptr(), tuple(w.shape), tuple(w.stride()), transposed, w.device.index), None)


# ----------------------------------------------------------------------------
# main_grad accumulation (sonicmoe/functional/__init__.py:393-414)
# ----------------------------------------------------------------------------
def _grad_target(w: torch.Tensor, shape):
    """fp32 accumulator living on the parameter (`main_grad`), or None."""
    base = _base_of(w)
    mg = getattr(base, "main_grad", None)
    if mg is None:
        return None, base
    if mg.dtype != torch.float32 or tuple(mg.shape) != tuple(shape) or not mg.is_contiguous():
        raise ValueError(f"main_grad must be contiguous fp32 of shape {tuple(shape)}, got {mg.dtype} "
                         f"{tuple(mg.shape)}")
    return mg, base


def _after_accumulate(base):
    hook = getattr(base, "_apply_backward_hook", None)
    if hook is not None:
        hook()


# "This tensor is complete on the stream that produced it": an event per freshly produced dx, recorded BEFORE the
# weight-gradient GEMMs are enqueued.  A consumer on another stream (the expert-parallel return exchange on its
# communication stream) waits for that event instead of for everything the compute stream has been given.
_RESULT_READY: dict = {}


def note_result_ready(t: torch.Tensor):
    if t.is_cuda and not torch.cuda.is_current_stream_capturing():
        if len(_RESULT_READY) >= 16:
            _RESULT_READY.pop(next(iter(_RESULT_READY)))
        ev = torch.cuda.Event()
        ev.record()
        _RESULT_READY[t.data_ptr()] = ev


def take_result_ready(t: torch.Tensor):
    """The event recorded when `t` was produced, or None (then the consumer orders itself after the whole stream)."""
    return _RESULT_READY.pop(t.data_ptr(), None)


# Where the next layer call should put its two token-side results (forward output, dx).  The expert-parallel layer
# points them at memory that the peer GPUs have mapped, so that the return exchange reads them in place.
_PLACEMENT: list = []       # innermost `place_results` block last


@contextmanager
def place_results(out: torch.Tensor | None = None, dx: torch.Tensor | None = None):
    """Within the block, the next `_UpProjection` / `_DownProjection` pair writes its forward output into `out` and,
    in its backward, dx into `dx` (contiguous bf16 [N,H] CUDA tensors) instead of fresh allocations.  The request
    is consumed by the first `_UpProjection.forward` that runs inside the block."""
    frame = {"out_buf": out, "dx_buf": dx}
    _PLACEMENT.append(frame)
    try:
        yield
    finally:
        _PLACEMENT.remove(frame)


def _take_placement():
    if not _PLACEMENT:
        return None, None
    frame = _PLACEMENT[-1]
    out, dx = frame["out_buf"], frame["dx_buf"]
    frame["out_buf"] = frame["dx_buf"] = None
    return out, dx


# Hand-off of the FP8 payloads from _UpProjection.forward to _DownProjection.forward.  The y1 / z tensors the first
# Function returns are zero-stride placeholders that only carry the autograd edges; each invocation allocates a fresh
# one-element storage for its z placeholder, and the address of that storage is the invocation's token: it is unique
# while the placeholder is alive, and it survives autograd handing the second Function a new Tensor object over the
# same storage (the reference stamps a token attribute on the returned tensors instead,
# sonicmoe/functional/__init__.py:438-488).  Two layers whose forwards interleave therefore pair up correctly.
_HANDOFF: dict = {}
_HANDOFF_MAX = 64           # entries of invocations whose second half never ran are dropped oldest-first


def _placeholder(like: torch.Tensor, shape):
    return torch.empty((), dtype=torch.bfloat16, device=like.device).expand(*shape)


def _handoff_put(z_placeholder: torch.Tensor, link: dict):
    if len(_HANDOFF) >= _HANDOFF_MAX:
        _HANDOFF.pop(next(iter(_HANDOFF)))
    _HANDOFF[z_placeholder.data_ptr()] = link


def _handoff_take(z_placeholder: torch.Tensor) -> dict:
    link = _HANDOFF.pop(z_placeholder.data_ptr(), None)
    if link is None:
        raise RuntimeError("_DownProjection got a z that no _UpProjection.forward produced: the FP8 hand-off is "
                           "addressed by the z placeholder _UpProjection returned, pass that tensor on unchanged")
    return link


class Fp8CombineGradHandle:
    """Carrier for an FP8 `dout` payload: the backward of an FP8 combine all-to-all `put`s the received
    (e4m3 bytes [N,H], raw 1x32 ue8m0 scales [N,H/32]); `_DownProjection.backward` `take`s it instead of
    quantising the gradient tensor it is handed (reference: fp8_combine_grad_handle,
    sonicmoe/functional/__init__.py:2130-2157)."""

    def __init__(self):
        self._payload = None

    def put(self, q, raw):
        self._payload = (q, raw)

    def take(self):
        p, self._payload = self._payload, None
        return p


def _up_projection(xg_q, a_sf, w1_q, w1_sf, efo, TKp, act, out=None):
    """z = x_sorted . W1^T, y1 = act(gate) * up; z and y1 leave as MXFP8.  SwiGLU: one GEMM with the activation and
    both quantizers in its epilogue; ReGLU / GEGLU: a plain GEMM to bf16 z, then the stand-alone activation kernel
    (rows beyond the last expert's segment hold whatever the allocator left: they are never read downstream)."""
    if act == 0:
        return ops.gemm_gated(xg_q, None, a_sf, w1_q, w1_sf, efo, TKp, out=out)
    z = ops.gemm_varlen_m(xg_q, a_sf, w1_q, w1_sf, efo)
    return ops.glu_fwd(z, act)


class _UpProjection(torch.autograd.Function):
    @classmethod
    def apply(cls, x, w1, b1, expert_frequency_offset, total_expert_freq, K, stream_id, x_gather_idx, s_scatter_idx,
              s_reverse_scatter_idx, num_activated_expert_per_token_offset, is_varlen_K, activation_type,
              is_inference_mode_enabled, use_low_precision_postact_buffer=False, prequant_activation_payload=None,
              fp8_config=None):
        return super().apply(x, w1, b1, expert_frequency_offset, total_expert_freq, K, stream_id, x_gather_idx,
                             s_scatter_idx, s_reverse_scatter_idx, num_activated_expert_per_token_offset,
                             is_varlen_K, activation_type, is_inference_mode_enabled,
                             use_low_precision_postact_buffer, prequant_activation_payload, fp8_config)

    @staticmethod
    def forward(ctx, x, w1, b1, efo, TKp, K, stream_id, x_gather_idx, s_scatter_idx, s_rev, naept, is_varlen_K,
                activation_type, is_inference, low_precision_postact, prequant_payload, fp8_config):
        ctx.set_materialize_grads(False)   # an unused output must not be handed a zero-filled [TKp, I] gradient
        _require_fp8()
        act = activation_code(activation_type)
        if b1 is not None:
            raise NotImplementedError("expert biases are not supported on the MXFP8 path")
        E, N2, H = w1.shape
        TKp = int(TKp)
        x_q = x_raw = packed_sf = gated_out = None
        if prequant_payload is not None:
            # x arrives as e4m3 bytes + raw 1x32 ue8m0 scales (expert-parallel dispatch payload); a third element is
            # the scales already gathered to expert-sorted rows in the ISA layout, and may carry the four
            # up-projection outputs allocated with the metadata (attach_preallocated_gated_outputs)
            x_q, x_raw = prequant_payload[0], prequant_payload[1]
            x_q = x_q.view(torch.uint8)
            if len(prequant_payload) > 2 and prequant_payload[2] is not None:
                packed_sf = prequant_payload[2]
                gated_out = getattr(packed_sf, _GATED_OUTPUT_PAYLOAD_ATTR, None)
                if gated_out is not None:      # (pre-activation, post-activation, z scales, y1 scales) -> op order
                    gated_out = (gated_out[0], gated_out[2], gated_out[1], gated_out[3])
                packed_sf = packed_sf.view(torch.uint8).reshape(-1)
                if packed_sf.numel() != ops.isa_bytes(TKp, H):
                    raise ValueError(f"packed scales hold {packed_sf.numel()} bytes, ({TKp}, {H}) needs "
                                     f"{ops.isa_bytes(TKp, H)}")
        elif USE_TMA_GATHER and act == 0:
            x_q, x_raw, _ = ops.quant_rows(x.contiguous(), raw=True)
        iso32, stagewise = _modes(fp8_config)
        w1_q, w1_sf, _ = _weight_operand(w1, False, iso32)
        if USE_TMA_GATHER and act == 0:
            a_sf = packed_sf if packed_sf is not None else ops.gather_scales_isa(x_raw, x_gather_idx, TKp, H)
            z_q, z_sc, y1_q, y1_sf = ops.gemm_gated(x_q, x_gather_idx, a_sf, w1_q, w1_sf, efo, TKp, out=gated_out)
        else:
            if x_q is not None and packed_sf is not None:
                xg_q, _ = ops.scatter_rows_fp8(x_q, None, naept, s_rev, s_scatter_idx, TKp, efo[-1:],
                                               with_scales=False)
                a_sf = packed_sf
            elif x_q is not None:
                xg_q, a_sf = ops.scatter_rows_fp8(x_q, x_raw, naept, s_rev, s_scatter_idx, TKp, efo[-1:])
            else:      # quantise straight into expert-sorted order
                xg_q, a_sf = ops.quant_rows_scatter(x.contiguous(), naept, s_rev, s_scatter_idx, TKp, efo[-1:])
            z_q, z_sc, y1_q, y1_sf = _up_projection(xg_q, a_sf, w1_q, w1_sf, efo, TKp, act, out=gated_out)
            del xg_q
        _log_stage_memory(stagewise, "forward: after up-projection")
        out_buf, ctx.dx_buf = _take_placement()
        link = {"y1": (y1_q, y1_sf), "z": (z_q, z_sc), "out_buf": out_buf, "act": act, "iso32": iso32,
                "stagewise": stagewise,
                # whether a backward of this Function will run (it then also runs the weight-gradient GEMM that
                # _DownProjection.backward hands over)
                "up_runs_backward": bool(ctx.needs_input_grad[0] or ctx.needs_input_grad[1])}
        cfg = fp8_config if fp8_config is not None else get_active_config()
        if cfg is not None and cfg.resolve_recompute_z() and not is_inference:
            # keep what regenerates z instead of z itself; the backward re-runs this GEMM and gets the same bytes
            link["z"] = None
            link["z_recompute"] = (x if prequant_payload is None else None, x_q, x_raw, w1, efo, x_gather_idx,
                                   s_scatter_idx, s_rev, naept, TKp, act, iso32)
            del z_q, z_sc
        ctx.link = link
        ctx.T = x.shape[0]
        ctx.x_is_fp8 = prequant_payload is not None
        ctx.x_dtype = x.dtype
        ctx.save_for_backward(x if prequant_payload is None else x_q, x_raw if prequant_payload is not None else None,
                              w1, efo, x_gather_idx, s_rev, naept)
        y1 = _placeholder(x, (TKp, N2 // 2))
        z = _placeholder(x, (TKp, N2))
        _handoff_put(z, link)
        ctx.mark_non_differentiable(y1)
        return y1, z

    @staticmethod
    def backward(ctx, _dy1, _dz):
        x, x_raw, w1, efo, x_gather_idx, s_rev, naept = ctx.saved_tensors
        link = ctx.link
        dz_q, dz_rsf, dz_t, dz_csf = link.pop("dz")
        E, N2, H = w1.shape
        TKp = dz_q.shape[0]
        # dx first: it is what an enclosing exchange (the expert-parallel return all-to-all) waits for, and the
        # weight gradients that follow on this stream then run underneath that exchange (the reference opens the
        # same slot for dw1: sonicmoe/functional/__init__.py:278-311)
        dx = None
        if ctx.needs_input_grad[0]:
            w1t_q, w1t_sf, kn = _weight_operand(w1, True, link.get("iso32", False))
            dx_exp = _gemm_plain(dz_q, dz_rsf, w1t_q, w1t_sf, kn, efo)
            del w1t_q, w1t_sf
            buf = ctx.dx_buf if (ctx.dx_buf is not None and ctx.x_dtype == torch.bfloat16) else None
            dx = ops.combine(dx_exp, s_rev, naept, None, ctx.T, out=buf)
            del dx_exp
            if dx.dtype != ctx.x_dtype:
                dx = dx.to(ctx.x_dtype)
            note_result_ready(dx)
            _log_stage_memory(link.get("stagewise", False), "backward: after dx")
        deferred_dw2 = link.pop("dw2_job", None)
        paired = None
        if deferred_dw2 is not None:
            ops2 = getattr(deferred_dw2, "operands", None)
            mg1, _ = _grad_target(w1, (E, N2, H)) if ctx.needs_input_grad[1] else (None, None)
            # dw2 joins dw1's launch: both into main_grad, dz / y1s left [TKp, dim], column operands transposed
            if (_PAIR_WGRADS and ops2 is not None and mg1 is not None and dz_t is None and ops2["a_rows"]
                    and not ops2["b_rows"] and _wide_wgrad_ok(E, N2, H)
                    and _wide_wgrad_ok(E, ops2["a_op"].shape[1], H)):
                paired = ops2
            else:
                deferred_dw2()
        dw1 = None
        if ctx.needs_input_grad[1]:
            if ctx.x_is_fp8:     # x is e4m3 + raw scales: dequantise, then column-wise re-quantise
                xc, x_sf, xc_rows = *ops.requant_cols_t(x, x_raw, x_gather_idx, TKp, efo[-1:]), False
            else:                # column scales; payload [TKp, H] or transposed, whichever the GEMM runs fastest on
                xc, x_sf, xc_rows = _col_operand(x, x_gather_idx, TKp, efo[-1:], E, N2, H)
            mg, base = _grad_target(w1, (E, N2, H))
            out = mg if mg is not None else torch.empty(E, N2, H, dtype=torch.float32, device=dz_q.device)
            # a row-major dz payload (32x32-block scales) doubles as the MN-major weight-gradient operand
            if paired is not None and not xc_rows:
                ops.gemm_wgrad_pair(dz_q, dz_csf, xc, x_sf, mg, paired["a_op"], paired["sf_a"], paired["b_op"],
                                    paired["sf_b"], paired["mg"], efo, True, True)
                _after_accumulate(paired["base"])
                paired = None
            else:
                if paired is not None:
                    deferred_dw2()
                    paired = None
                _wgrad(dz_q if dz_t is None else dz_t, dz_csf, dz_t is None, xc, x_sf, xc_rows, efo, out,
                       mg is not None)
            if mg is not None:
                _after_accumulate(base)
            else:
                dw1 = out.to(w1.dtype)
            del xc, x_sf
        del dz_q, dz_rsf, dz_t, dz_csf
        _log_stage_memory(link.get("stagewise", False), "backward: after dw1")
        ops.post_status(x.device)      # last kernels of the layer's backward: let the next call see their status
        return (dx, dw1) + (None,) * 15


def _recompute_z(args):
    """z as e4m3 + raw scales, regenerated from the up-projection's inputs (same kernels, same bytes as the
    forward produced; the re-computed y1 is discarded)."""
    x, x_q, x_raw, w1, efo, x_gather_idx, s_scatter_idx, s_rev, naept, TKp, act, iso32 = args
    H = w1.shape[2]
    w1_q, w1_sf, _ = _weight_operand(w1, False, iso32)
    if USE_TMA_GATHER and act == 0:
        if x_q is None:
            x_q, x_raw, _ = ops.quant_rows(x.contiguous(), raw=True)
        a_sf = ops.gather_scales_isa(x_raw, x_gather_idx, TKp, H)
        z_q, z_sc, _, _ = ops.gemm_gated(x_q, x_gather_idx, a_sf, w1_q, w1_sf, efo, TKp)
    else:
        if x_q is not None:
            xg_q, a_sf = ops.scatter_rows_fp8(x_q, x_raw, naept, s_rev, s_scatter_idx, TKp, efo[-1:])
        else:
            xg_q, a_sf = ops.quant_rows_scatter(x.contiguous(), naept, s_rev, s_scatter_idx, TKp, efo[-1:])
        z_q, z_sc, _, _ = _up_projection(xg_q, a_sf, w1_q, w1_sf, efo, TKp, act)
    return z_q, z_sc


class _DownProjection(torch.autograd.Function):
    @classmethod
    def apply(cls, y1, z, w2, b2, topk_scores, selected_experts, expert_frequency_offset, T, K, stream_id,
              x_gather_idx, s_scatter_idx, s_reverse_scatter_idx, num_activated_expert_per_token_offset,
              is_varlen_K, activation_type, fp8_protocol, fp8_combine_grad_handle=None, fp8_config=None,
              router_score_source=None, router_score_src_idx=None):
        return super().apply(y1, z, w2, b2, topk_scores, selected_experts, expert_frequency_offset, T, K, stream_id,
                             x_gather_idx, s_scatter_idx, s_reverse_scatter_idx,
                             num_activated_expert_per_token_offset, is_varlen_K, activation_type, fp8_protocol,
                             fp8_combine_grad_handle, fp8_config, router_score_source, router_score_src_idx)

    @staticmethod
    def forward(ctx, y1, z, w2, b2, topk_scores, selected_experts, efo, T, K, stream_id, x_gather_idx, s_scatter_idx,
                s_rev, naept, is_varlen_K, activation_type, fp8_protocol, fp8_combine_grad_handle, fp8_config,
                router_score_source, router_score_src_idx):
        ctx.set_materialize_grads(False)
        _require_fp8()
        if b2 is not None:
            raise NotImplementedError("expert biases are not supported on the MXFP8 path")
        link = _handoff_take(z)
        y1_q, y1_sf = link.pop("y1")
        w2_q, w2_sf, _ = _weight_operand(w2, False, link.get("iso32", False))
        y2 = ops.gemm_varlen_m(y1_q, y1_sf, w2_q, w2_sf, efo)
        del y1_q, y1_sf
        o = ops.combine(y2, s_rev, naept, topk_scores, int(T), out=link.pop("out_buf", None))
        del y2
        _log_stage_memory(link.get("stagewise", False), "forward: after down-projection")
        ops.post_status(o.device)
        ctx.link = link
        ctx.T = int(T)
        ctx.grad_handle = fp8_combine_grad_handle
        ctx.score_source_shape = None if router_score_source is None else tuple(router_score_source.shape)
        ctx.save_for_backward(w2, topk_scores, efo, x_gather_idx, s_scatter_idx, s_rev, naept, router_score_src_idx)
        return o

    @staticmethod
    def backward(ctx, dout):
        w2, topk_scores, efo, x_gather_idx, s_scatter_idx, s_rev, naept, src_idx = ctx.saved_tensors
        link = ctx.link
        z_saved = link.pop("z")
        z_q, z_sc = z_saved if z_saved is not None else _recompute_z(link.pop("z_recompute"))
        E, H, I = w2.shape
        TKp = z_q.shape[0]
        s = ops.gather_scores(topk_scores, s_scatter_idx)
        payload = ctx.grad_handle.take() if ctx.grad_handle is not None else None
        if payload is not None:
            # dout arrives already as e4m3 + raw 1x32 scales (backward of an FP8 combine all-to-all);
            # the `dout` argument is then only a placeholder carrying the autograd edge
            dout_q, dout_raw = payload
            dout = None
        else:
            dout = dout.contiguous()
            if dout.dtype != torch.bfloat16:
                dout = dout.to(torch.bfloat16)
            dout_q = dout_raw = None
            if USE_TMA_GATHER and link.get("act", 0) == 0:
                dout_q, dout_raw, _ = ops.quant_rows(dout, raw=True)
        y1s_q = dout_c = None
        dout_c_rows = False
        act = link.get("act", 0)
        stagewise = link.get("stagewise", False)
        # memory-lean order: the column-quantised copy of dout is made after GemmDGated has run and z and the
        # gathered dout rows are freed, and dw2 runs (and frees its operands) before dx_expanded is allocated
        early_cols = not stagewise
        w2t_q, w2t_sf, kn = _weight_operand(w2, True, link.get("iso32", False))
        if kn:
            # GemmDGated reads B K-major only (its 192-column slices are no MN-major swizzle atoms): a transient
            # byte-transposed copy, freed after the GEMM (the reference does the same, functional/__init__.py:2160)
            w2t_q = ops.transpose_u8(w2t_q)
        if USE_TMA_GATHER and act == 0:
            a_sf = ops.gather_scales_isa(dout_raw, x_gather_idx, TKp, H)
            if early_cols and dout is not None and ctx.needs_input_grad[2] and _mn_wgrad_ok(E, I, H):
                dout_c, dout_sf, dout_c_rows = _col_operand(dout, x_gather_idx, TKp, efo[-1:], E, I, H)
            if FUSE_DGATED_QUANT and _mn_wgrad_ok(E, I, H):
                dz_q, dz_rsf, dz_csf, y1s_q, y1s_sf, dsp = ops.gemm_dgated_fused(
                    dout_q, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, TKp, a_idx=x_gather_idx)
                link["dz"] = (dz_q, dz_rsf, None, dz_csf)
                dz = y1s = None
            else:
                dz, y1s, dsp = ops.gemm_dgated(dout_q, x_gather_idx, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, TKp)
        else:
            if dout_q is not None:
                dg_q, a_sf = ops.scatter_rows_fp8(dout_q, dout_raw, naept, s_rev, s_scatter_idx, TKp, efo[-1:])
            else:
                # row scales in scatter form (each token read once: 68 us on T=8192, H=3072, K=8), column scales
                # in a second, gathered pass (93 us); the one-pass dual kernel measured 209 us there
                dg_q, a_sf = ops.quant_rows_scatter(dout, naept, s_rev, s_scatter_idx, TKp, efo[-1:])
                if early_cols and ctx.needs_input_grad[2] and _mn_wgrad_ok(E, I, H):
                    dout_c, dout_sf, dout_c_rows = _col_operand(dout, x_gather_idx, TKp, efo[-1:], E, I, H)
            if act != 0:
                # ReGLU / GEGLU: D from a plain GEMM, then the stand-alone activation-gradient kernel; dz / y1s in bf16
                # take the separate quantizers below
                D = ops.gemm_varlen_m(dg_q, a_sf, w2t_q, w2t_sf, efo)
                dz, y1s, dsp = ops.glu_bwd(D, z_q, z_sc, s, act)
                del D
            elif FUSE_DGATED_QUANT and _mn_wgrad_ok(E, I, H):
                # dz / y1s never exist in bf16: the epilogue emits the e4m3 operands of dgrad, dw1 and dw2,
                # row-major; the weight-gradient GEMMs read them MN-major (needs 256-multiples of I and H)
                dz_q, dz_rsf, dz_csf, y1s_q, y1s_sf, dsp = ops.gemm_dgated_fused(
                    dg_q, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, TKp)
                link["dz"] = (dz_q, dz_rsf, None, dz_csf)
                dz = y1s = None
            else:
                dz, y1s, dsp = ops.gemm_dgated(dg_q, None, a_sf, w2t_q, w2t_sf, efo, z_q, z_sc, s, TKp)
            del dg_q
        del z_q, z_sc, w2t_q, w2t_sf, a_sf
        _log_stage_memory(stagewise, "backward: after GemmDGated")
        dw2 = None
        if ctx.needs_input_grad[2]:
            if y1s is not None:
                y1s_t, y1s_sf = ops.quant_cols_t(y1s, None, TKp, valid_rows=efo[-1:])
                del y1s
            if dout_c is None:
                if dout is None:
                    dout_t, dout_sf = ops.requant_cols_t(dout_q, dout_raw, x_gather_idx, TKp, efo[-1:])
                elif _mn_wgrad_ok(E, I, H):
                    dout_c, dout_sf, dout_c_rows = _col_operand(dout, x_gather_idx, TKp, efo[-1:], E, I, H)
                else:
                    dout_t, dout_sf = ops.quant_cols_t(dout, x_gather_idx, TKp, valid_rows=efo[-1:])
            mg, base = _grad_target(w2, (E, I, H))
            a_op, a_rows = (y1s_q, True) if y1s_q is not None else (y1s_t, False)
            b_op, b_rows = (dout_c, dout_c_rows) if dout_c is not None else (dout_t, False)
            if mg is not None and link.get("up_runs_backward") and _DEFER_DW2 and not stagewise:
                # accumulation into main_grad returns no tensor: the GEMM is handed to _UpProjection.backward, which
                # runs it after dx so that it, too, lies underneath an enclosing exchange of dx
                def dw2_job(a_op=a_op, a_rows=a_rows, b_op=b_op, b_rows=b_rows, sf_a=y1s_sf, sf_b=dout_sf, mg=mg,
                            base=base, efo=efo):
                    _wgrad(a_op, sf_a, a_rows, b_op, sf_b, b_rows, efo, mg, True)
                    _after_accumulate(base)
                # the operands too, so that the first Function's backward can fold this GEMM into dw1's launch
                dw2_job.operands = dict(a_op=a_op, a_rows=a_rows, b_op=b_op, b_rows=b_rows, sf_a=y1s_sf, sf_b=dout_sf,
                                        mg=mg, base=base)
                link["dw2_job"] = dw2_job
            elif mg is not None:
                _wgrad(a_op, y1s_sf, a_rows, b_op, dout_sf, b_rows, efo, mg, True)
                _after_accumulate(base)
            else:
                out = torch.empty(E, I, H, dtype=torch.float32, device=s.device)
                _wgrad(a_op, y1s_sf, a_rows, b_op, dout_sf, b_rows, efo, out, False)
                dw2 = out.transpose(1, 2).to(w2.dtype)
            del a_op, b_op, y1s_q, dout_c
            _log_stage_memory(stagewise, "backward: after dw2")
        if dz is not None:
            link["dz"] = ops.quant_iso32(dz)
        else:      # the gradient edge of z still needs a tensor of its shape; its contents are never read
            dz = _placeholder(topk_scores, (TKp, 2 * I))
        # ds: token-major (length of the score buffer) and, when asked, scattered to the [T,K] source
        d_scores = d_source = None
        want_flat = ctx.needs_input_grad[4]
        want_src = ctx.needs_input_grad[19] and src_idx is not None
        if want_flat or want_src:
            TK = s_rev.numel()
            numel = 1
            if want_src:
                for d in ctx.score_source_shape:
                    numel *= d
            ds_tm, ds_src = ops.ds_finalize(dsp, s_rev, TK, naept[-1:], src_idx if want_src else None, numel)
            if want_flat:
                d_scores = torch.zeros_like(topk_scores)
                d_scores[:TK] = ds_tm
            if want_src:
                d_source = ds_src.view(ctx.score_source_shape)
        grads = [None] * 21
        grads[1] = dz
        grads[2] = dw2
        grads[4] = d_scores
        grads[19] = d_source
        return tuple(grads)


# ----------------------------------------------------------------------------
# router: top-k on logits, softmax over the K selected (forward.py:217-236,
# backward.py:572-641)
# ----------------------------------------------------------------------------
class _TopKSoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, K):
        scores, idx = ops.topk_softmax(logits.contiguous(), int(K))
        ctx.save_for_backward(scores, idx)
        ctx.E = logits.shape[1]
        ctx.mark_non_differentiable(idx)
        return scores, idx

    @staticmethod
    def backward(ctx, dscores, _didx):
        scores, idx = ctx.saved_tensors
        return ops.topk_softmax_bwd(scores, idx, dscores.contiguous().float(), ctx.E), None


def _expert_major(w: torch.Tensor) -> torch.Tensor:
    """[N,K,E] view (the layout the module passes) -> [E,N,K] contiguous."""
    w = w.permute(2, 0, 1)
    return w if w.is_contiguous() else w.contiguous()


def moe_TC_softmax_topk_layer(x, router_w, w1, b1, w2, b2, K, stream_id, activation_type=ActivationType.SWIGLU,
                              is_inference_mode_enabled=False, fp8_protocol=None):
    """Dense top-k MoE layer.  x [T,H]; router_w [E,H]; w1 [2I,H,E] and w2 [H,I,E] views of the expert-major
    parameters (rows of w1 interleaved gate0, up0, gate1, ...).  Returns (o [T,H], router_logits [T,E],
    expert_frequency [E] int32); differentiable w.r.t. x, router_w, w1, w2."""
    _require_fp8()
    activation_code(activation_type)
    ops.poll_status(x.device)         # a device-side failure of an earlier pass surfaces here, without a sync
    T, H = x.shape
    E = router_w.shape[0]
    w1_e, w2_e = _expert_major(w1), _expert_major(w2)
    logits = F.linear(x, router_w)
    scores, idx = _TopKSoftmax.apply(logits.float(), K)
    md = ops.topk_metadata(idx, scores.detach(), E, 128, TK_alloc=T * K, lane_order=1, pad_mode=1)
    y1, z = _UpProjection.apply(x, w1_e, b1, md["efo"], md["TKp_alloc"], K, stream_id, md["x_gather_idx"],
                                md["s_scatter_idx"], md["s_reverse_scatter_idx"], md["naept"], False,
                                activation_type, is_inference_mode_enabled)
    o = _DownProjection.apply(y1, z, w2_e, b2, md["topk_scores"], idx, md["efo"], T, K, stream_id,
                              md["x_gather_idx"], md["s_scatter_idx"], md["s_reverse_scatter_idx"], md["naept"],
                              False, activation_type, fp8_protocol, None, None, scores, md["score_src_idx"])
    return o, logits, md["counts"]


# ----------------------------------------------------------------------------
# general routing: a list of (token, expert, score) pairs instead of a [T,K] table
# ----------------------------------------------------------------------------
_MAX_PAIRS_PER_TOKEN = 16        # lanes per token the routing-metadata kernel handles


def _pairs_to_table(router_scores_selected, sorted_selected_T, selected_E, T):
    """(score, token, expert) pairs, sorted by token -> padded tables idx [T,Kmax] (-1 = no pair) and scores
    [T,Kmax]; the scatter into the score table is differentiable with respect to the pair scores."""
    tok = sorted_selected_T.long()
    per_tok = torch.bincount(tok, minlength=T)
    kmax = int(per_tok.max()) if tok.numel() else 1
    if kmax > _MAX_PAIRS_PER_TOKEN:
        raise NotImplementedError(f"a token routed to {kmax} experts: at most {_MAX_PAIRS_PER_TOKEN} are supported")
    kmax = max(kmax, 1)
    first = torch.cumsum(per_tok, 0) - per_tok
    lane = torch.arange(tok.numel(), device=tok.device) - first[tok]
    idx = torch.full((T, kmax), -1, dtype=torch.int32, device=tok.device)
    idx[tok, lane] = selected_E.to(torch.int32)
    scores = torch.zeros(T, kmax, dtype=torch.float32, device=tok.device).index_put((tok, lane),
                                                                                  router_scores_selected.float())
    return idx, scores


def general_routing_router_metadata(router_scores_selected, sorted_selected_T, selected_E, T: int, E: int):
    """Routing metadata for an arbitrary list of (token, expert) pairs sorted by token - same outputs as the
    reference's function of this name (sonicmoe/functional/__init__.py:740-773): (expert_frequency,
    expert_frequency_offset [E+1], x_gather_idx, s_scatter_idx, s_reverse_scatter_idx,
    num_activated_expert_per_token_offset [T+1]), all unpadded (alignment 1)."""
    idx, scores = _pairs_to_table(router_scores_selected.detach(), sorted_selected_T, selected_E, T)
    n = int(sorted_selected_T.numel())
    md = ops.topk_metadata(idx, scores, E, alignment=1, TK_alloc=n, TKp_alloc=n, lane_order=1, pad_mode=1)
    return (md["counts"], md["efo"], md["x_gather_idx"], md["s_scatter_idx"], md["s_reverse_scatter_idx"],
            md["naept"])


def moe_general_routing_inputs(x, router_scores, token_indices, expert_indices, w1, b1, w2, b2, E, stream_id,
                               activation_type=ActivationType.SWIGLU, is_inference_mode_enabled=False):
    """MoE layer on an explicit routing: pair i sends token `token_indices[i]` (ascending) to expert
    `expert_indices[i]` with weight `router_scores[i]`; a token may have any number of pairs up to 16 (what a
    token-rounding or expert-choice router produces).  x [T,H]; w1 [2I,H,E] and w2 [H,I,E] views of the
    expert-major parameters, as in `moe_TC_softmax_topk_layer`.  Returns (o [T,H], expert_frequency [E] int32);
    differentiable with respect to x, router_scores, w1 and w2.  Call sites in the reference:
    benchmarks/moe-token-rounding.py:103-118, tools/introspect.py:1511-1514."""
    from ..interface import run_sonic_moe
    _require_fp8()
    activation_code(activation_type)
    if b1 is not None or b2 is not None:
        raise NotImplementedError("expert biases are not supported on the MXFP8 path")
    T = x.shape[0]
    w1_e, w2_e = _expert_major(w1), _expert_major(w2)
    idx, scores = _pairs_to_table(router_scores, token_indices, expert_indices, T)
    counts = ops.count_cumsum(expert_indices.to(torch.int32).contiguous(), E, do_cumsum=False) if E % 4 == 0 \
        else torch.bincount(expert_indices.long(), minlength=E).to(torch.int32)
    o = run_sonic_moe(x, idx, scores, idx.shape[1], E, w1_e, w2_e, fp8=True, activation_type=activation_type,
                      sync_free_sizing=True)
    return o, counts
