"""`run_sonic_moe`: expert compute on pre-routed (dispatched) tokens - the
functional entry the host framework calls after its dispatch all-to-all
(sonicmoe/interface.py:69-345)."""
from __future__ import annotations

import torch

from . import ops
from .enums import ActivationType, activation_code
from .functional import (_DownProjection, _UpProjection, attach_preallocated_gated_outputs, enable_fp8,
                         place_results)


def scale_bytes(fp8_scale: torch.Tensor, H: int) -> torch.Tensor:
    """The 1x32 ue8m0 scales of an FP8 payload as one byte per group, u8 [N, H/32], from any of the formats the
    reference's dispatch delivers (sonicmoe/quack_utils/blockscaled_fp8_gemm.py:535-550, interface.py:135-187):
    uint8 / float8_e8m0fnu [N, H/32]; int32 [N, H/128] - four scale bytes per word, the compact form DeepEP
    transports as opaque int32; int32 [N, H/32] - one word per group."""
    groups = H // 32
    if fp8_scale.dtype == torch.uint8 and fp8_scale.shape[-1] == groups:
        return fp8_scale.contiguous()
    if fp8_scale.dtype == torch.int32 and fp8_scale.shape[-1] * 4 == groups:
        return fp8_scale.contiguous().view(torch.uint8)           # little-endian: byte j of a row is group j
    if fp8_scale.dtype == torch.int32 and fp8_scale.shape[-1] == groups:
        return fp8_scale.to(torch.uint8)
    if getattr(torch, "float8_e8m0fnu", None) is not None and fp8_scale.dtype == torch.float8_e8m0fnu \
            and fp8_scale.shape[-1] == groups:
        return fp8_scale.contiguous().view(torch.uint8)
    raise ValueError(f"fp8_scale {fp8_scale.dtype} {tuple(fp8_scale.shape)} is none of the 1x32 ue8m0 formats for "
                     f"H={H}: u8/e8m0 [N,{groups}], int32 [N,{groups // 4}] (packed words) or int32 [N,{groups}]")


def run_sonic_moe(hidden_states, topk_indices, topk_scores, K, E, w1, w2, fp8=False, tokens_per_expert=None,
                  fp8_scale=None, fp8_combine_grad_handle=None, fp8_config=None, release_fp8_weights=False,
                  activation_type=ActivationType.SWIGLU, sync_free_sizing=False, grad_holder=None, out=None,
                  dx_out=None):
    """hidden_states [N,H] bf16 (or e4m3 with `fp8_scale` = raw 1x32 ue8m0 bytes [N,H/32]);
    topk_indices [N,K] with -1 for slots whose expert is not local (a row's valid experts distinct);
    topk_scores [N,K] f32; w1 [E,2I,H]; w2 [E,H,I].  Returns [N,H] bf16.

    With an e4m3 `hidden_states` no gradient can flow to it (torch has no differentiable 8-bit tensors);
    `grad_holder` - a bf16 [N,H] tensor that requires grad, contents ignored - then receives dx in its place
    (the expert-parallel dispatch passes its placeholder here; not part of the reference signature).

    `out` / `dx_out` - contiguous bf16 [N,H] CUDA buffers that receive the forward output and, in the backward,
    dx (the returned tensor / the gradient ARE those buffers); used by the expert-parallel layer to leave both in
    memory its peers can read (not part of the reference signature).

    `tokens_per_expert` (host list / tensor) sizes the expert-sorted buffers exactly; with
    `sync_free_sizing` (or without counts) they are sized at the shape-only upper bound and no
    device-to-host copy happens."""
    if not fp8:
        raise NotImplementedError("run_sonic_moe: only fp8=True (MXFP8) is built")
    ops.poll_status(hidden_states.device)     # a device-side failure of an earlier pass surfaces here, without a sync
    N = hidden_states.shape[0]
    idx = topk_indices if topk_indices.dtype == torch.int32 else topk_indices.to(torch.int32)
    probs = topk_scores.detach()
    if probs.dtype != torch.float32:
        probs = probs.float()
    TK = TKp = None
    if tokens_per_expert is not None and not sync_free_sizing:
        counts = tokens_per_expert.tolist() if isinstance(tokens_per_expert, torch.Tensor) else list(tokens_per_expert)
        TK = int(sum(counts))
        TKp = int(sum(-(-c // 128) * 128 for c in counts if c > 0))
    md = ops.topk_metadata(idx.contiguous(), probs.contiguous(), E, 128, TK, TKp)
    stream_id = torch.cuda.current_stream().cuda_stream
    payload = None
    if fp8_scale is not None:
        H = hidden_states.shape[1]
        raw = scale_bytes(fp8_scale, H)
        payload = (hidden_states.view(torch.uint8), raw)
        gated_n = int(w1.shape[1])
        if activation_code(activation_type) == 0 and gated_n % 256 == 0 and H % 128 == 0 \
                and hidden_states.dtype in (torch.float8_e4m3fn, torch.uint8):
            # the scales gathered to expert-sorted rows and the four outputs of the up-projection are made together
            # with the metadata and travel with the payload (reference: interface.py:136-188,254-262; the output
            # allocation sits in its metadata op, deepep_topk_metadata_cuda/kernel.cu:982-1019)
            TKp_alloc = md["TKp_alloc"]
            packed = ops.gather_scales_isa(raw, md["x_gather_idx"], TKp_alloc, H)
            dev = hidden_states.device
            outs = (torch.empty(TKp_alloc, gated_n, dtype=hidden_states.dtype, device=dev),
                    torch.empty(TKp_alloc, gated_n // 2, dtype=hidden_states.dtype, device=dev),
                    torch.empty(TKp_alloc, gated_n // 32, dtype=torch.uint8, device=dev),
                    torch.empty(TKp_alloc // 128, gated_n // 256, 512, dtype=torch.uint8, device=dev))
            payload = (payload[0], raw, attach_preallocated_gated_outputs(packed, outs))
        hidden_states = grad_holder if grad_holder is not None else torch.empty(
            (), dtype=torch.bfloat16, device=hidden_states.device).expand(N, hidden_states.shape[1])
    need_router_grad = topk_scores.requires_grad
    with enable_fp8(True), place_results(out, dx_out):
        y1, z = _UpProjection.apply(hidden_states, w1, None, md["efo"], md["TKp_alloc"], K, stream_id,
                                    md["x_gather_idx"], md["s_scatter_idx"], md["s_reverse_scatter_idx"],
                                    md["naept"], True, activation_type, False, False, payload, fp8_config)
        out = _DownProjection.apply(y1, z, w2, None, md["topk_scores"], md["s_scatter_idx"], md["efo"], N, K,
                                    stream_id, md["x_gather_idx"], md["s_scatter_idx"],
                                    md["s_reverse_scatter_idx"], md["naept"], True, activation_type, None,
                                    fp8_combine_grad_handle, fp8_config,
                                    topk_scores if need_router_grad else None,
                                    md["score_src_idx"] if need_router_grad else None)
    return out
