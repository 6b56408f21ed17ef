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
