"""`deepep_topk_to_sonic_metadata`: dispatched top-k indices/probs -> padded
routing metadata (sonicmoe/ernie_compat/deepep_metadata.py:180-358,593-799)."""
from __future__ import annotations

import torch

from .. import ops


def metadata_lanes_expert_sorted() -> bool:
    """A token's lanes are listed in ascending expert order (deepep_metadata.py:173-177)."""
    return True


def deepep_topk_to_sonic_metadata(dispatched_indices, dispatched_probs, tokens_per_expert, E, device="cuda",
                                  block: int = 128, sync_free_sizing: bool = False):
    """Returns (expert_frequency_offset [E+1], x_gather_idx [TK_padded], s_scatter_idx [TK_padded],
    s_reverse_scatter_idx [TK], num_activated_expert_per_token_offset [N+1], topk_scores [TK_padded],
    TK_padded, total_pad_rows, N_recv, score_src_idx [TK]).

    With `tokens_per_expert` given (host list or tensor) and `sync_free_sizing` False the outputs are
    sized exactly (a tensor argument is read back to the host, as in the reference); otherwise they are
    sized at the shape-only upper bound TK = N*min(K,E), TK_padded = roundup(TK,128) + E*block, and
    `total_pad_rows` is the bound minus TK.
    """
    if dispatched_indices.dtype != torch.int32:
        raise ValueError(f"dispatched_indices: expected int32, got {dispatched_indices.dtype}")
    if dispatched_probs.dtype != torch.float32:
        raise ValueError(f"dispatched_probs: expected float32, got {dispatched_probs.dtype}")
    if dispatched_indices.ndim != 2 or dispatched_probs.ndim != 2:
        raise ValueError("dispatched_indices and dispatched_probs must be 2D")
    if dispatched_probs.shape != dispatched_indices.shape:
        raise ValueError(f"shape mismatch: indices={tuple(dispatched_indices.shape)} vs "
                         f"probs={tuple(dispatched_probs.shape)}")
    N = dispatched_indices.shape[0]
    TK = TKp = None
    if not sync_free_sizing and tokens_per_expert is not None:
        counts = tokens_per_expert.tolist() if isinstance(tokens_per_expert, torch.Tensor) else list(tokens_per_expert)
        TK = int(sum(counts))
        TKp = int(sum(-(-c // block) * block for c in counts if c > 0))
    md = ops.topk_metadata(dispatched_indices.contiguous(), dispatched_probs.contiguous(), E, block, TK, TKp)
    return (md["efo"], md["x_gather_idx"], md["s_scatter_idx"], md["s_reverse_scatter_idx"], md["naept"],
            md["topk_scores"], md["TKp_alloc"], md["TKp_alloc"] - md["TK_alloc"], N, md["score_src_idx"])


def deepep_topk_to_sonic_metadata_with_scales(dispatched_indices, dispatched_probs, tokens_per_expert, E, raw_scales,
                                              cols, device="cuda", block: int = 128,
                                              pack_scales_in_scatter: bool = False,
                                              pack_scales_rowmajor: bool = False, gated_output_prototype=None,
                                              gated_n=None, gated_preact_bf16: bool = False,
                                              gated_allocate_z_scale: bool = True, sync_free_sizing: bool = False):
    """`deepep_topk_to_sonic_metadata` for an FP8 payload: the ten metadata values, then the payload's raw 1x32 ue8m0
    scales `raw_scales` (u8 / e8m0 [N, cols/32], or the compact int32 carrier [N, cols/128] with four scale bytes
    per word) gathered to expert-sorted rows in the ISA layout of (TK_padded, cols), then - when
    `gated_output_prototype` (an e4m3 tensor naming device and dtype) and `gated_n` (= 2I, a multiple of 256) are
    given - the four outputs of the up-projection allocated for this call: pre-activation [TK_padded, gated_n]
    (e4m3, or bf16 with `gated_preact_bf16`), post-activation e4m3 [TK_padded, gated_n/2], raw pre-activation scales
    u8 [TK_padded, gated_n/32] (empty without `gated_allocate_z_scale`) and post-activation ISA scales u8
    [TK_padded/128, gated_n/256, 512] (sonicmoe/ernie_compat/deepep_metadata.py:360-470,
    deepep_topk_metadata_cuda/kernel.cu:942-1019).  Each call returns fresh storage.  `pack_scales_in_scatter` /
    `pack_scales_rowmajor` select among the reference's kernels for the same bytes and change nothing here."""
    from ..interface import scale_bytes

    if (gated_output_prototype is None) != (gated_n is None):
        raise ValueError("gated_output_prototype and gated_n must be provided together")
    raw2d = raw_scales
    if raw2d.ndim == 3:
        if raw2d.shape[0] != 1:
            raise ValueError(f"raw_scales: expected batch=1, got shape {tuple(raw2d.shape)}")
        raw2d = raw2d.squeeze(0)
    if raw2d.ndim != 2:
        raise ValueError(f"raw_scales: expected rank 2, got shape {tuple(raw2d.shape)}")
    N = dispatched_indices.shape[0]
    if raw2d.shape[0] != N:
        raise ValueError(f"raw_scales row mismatch: expected {N}, got {raw2d.shape[0]}")
    cols = int(cols)
    if cols % 128:
        raise ValueError(f"cols must be a multiple of 128, got {cols}")
    raw_u8 = scale_bytes(raw2d, cols)            # raises on a shape / dtype that is none of the carriers
    if gated_output_prototype is not None:
        if "float8_e4m3" not in str(gated_output_prototype.dtype):
            raise ValueError(f"gated_output_prototype must use float8_e4m3, got {gated_output_prototype.dtype}")
        if int(gated_n) <= 0 or int(gated_n) % 256 != 0:
            raise ValueError(f"gated_n must be positive and divisible by 256, got {gated_n}")
    base = deepep_topk_to_sonic_metadata(dispatched_indices, dispatched_probs, tokens_per_expert, E, device, block,
                                         sync_free_sizing)
    x_gather_idx, TKp = base[1], base[6]
    packed = ops.gather_scales_isa(raw_u8, x_gather_idx, TKp, cols)
    if gated_output_prototype is None:
        return (*base, packed)
    dev, n = gated_output_prototype.device, int(gated_n)
    fp8 = gated_output_prototype.dtype
    preact = torch.empty(TKp, n, dtype=torch.bfloat16 if gated_preact_bf16 else fp8, device=dev)
    postact = torch.empty(TKp, n // 2, dtype=fp8, device=dev)
    z_scales = torch.empty((TKp, n // 32) if gated_allocate_z_scale else (0,), dtype=torch.uint8, device=dev)
    postact_scales = torch.empty(TKp // 128, n // 256, 512, dtype=torch.uint8, device=dev)
    return (*base, packed, preact, postact, z_scales, postact_scales)
