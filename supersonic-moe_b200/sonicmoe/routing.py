"""Routers that produce (score, token, expert) pair lists for `moe_general_routing_inputs`.

`token_rounding_routing` restates the token-rounding router of the reference's benchmark
(benchmarks/moe-token-rounding.py:139-181): a token-choice top-K pass fixes each expert's load, the load is rounded
to a multiple of the GEMM row tile, and an expert-choice pass over the combined scores (top-K picks first, then the
rest by score) fills or trims every expert to exactly that many tokens.  With every count a multiple of the tile no
expert segment needs pad rows.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .count_cumsum import count_cumsum


def token_rounding_routing(router_logits: torch.Tensor, K: int, Mtile: int = 128, routing: str = "nr"):
    """router_logits [T,E] -> (scores of the selected pairs [nnz], token_indices [nnz] ascending, expert_indices
    [nnz]).  routing: "down" / "up" / "nr" (nearest) rounding of each expert's top-K load to a multiple of Mtile."""
    T, E = router_logits.shape
    dev = router_logits.device
    scores = F.softmax(router_logits, dim=-1, dtype=torch.float32)
    topk_values, topk_indices = scores.topk(K, dim=-1)
    flat = topk_indices.reshape(-1).to(torch.int32).contiguous()
    if flat.is_cuda and E % 4 == 0:
        freq = count_cumsum(flat, E, do_cumsum=False)
    else:
        freq = torch.bincount(flat.long(), minlength=E).to(torch.int32)
    if routing == "down":
        rounded = torch.div(freq, Mtile, rounding_mode="floor") * Mtile
    elif routing == "up":
        rounded = torch.div(freq + Mtile - 1, Mtile, rounding_mode="floor") * Mtile
    elif routing == "nr":
        rounded = torch.round(freq.float() / Mtile).to(torch.int32) * Mtile
    else:
        raise NotImplementedError(f"routing={routing!r}")
    rounded = rounded.clamp(max=T)
    topk_values = topk_values / topk_values.sum(dim=-1, keepdim=True)
    scores = scores.scatter(-1, topk_indices, topk_values)
    # expert-choice order: a token's top-K picks rank above everything else, each class by score
    combined = scores.detach() - 1
    combined.scatter_(1, topk_indices, topk_values.detach())
    order = combined.argsort(dim=0, descending=True).int()                       # [T,E]: per expert, tokens by rank
    keep = torch.arange(T, device=dev, dtype=torch.int32)[:, None] < rounded[None, :]
    token_indices = order[keep]
    expert_indices = torch.arange(E, device=dev, dtype=torch.int32)[None, :].expand(T, -1)[keep]
    by_token = token_indices.argsort(stable=True)
    token_indices, expert_indices = token_indices[by_token], expert_indices[by_token]
    return scores[token_indices.long(), expert_indices.long()].contiguous(), token_indices, expert_indices
