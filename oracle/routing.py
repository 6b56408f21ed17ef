"""CPU restatement of the reference's routing-metadata kernels (integer work).

TEST INFRASTRUCTURE ONLY - never imported by the product path.

Follows, function by function:

* `count_cumsum`         sonicmoe/count_cumsum/__init__.py:20-35, kernel.cu:96-152
* `topk_metadata`        sonicmoe/ernie_compat/deepep_topk_metadata_cuda/kernel.cu
                         :129-202 (histogram), :304-418 (padded offsets, naept),
                         :427-603 (scatter: stable ascending token order inside an
                         expert, ascending expert order inside a token), :604-668
                         (pad fill and over-allocated tails)
* `dense_topk_metadata`  sonicmoe/functional/triton_kernels/__init__.py:66-155
                         (rows of an expert ordered by ascending flat index t*K+k,
                         token-major index IS the flat index) followed by
                         `_pad_routing_metadata`, sonicmoe/functional/__init__.py:176-243
* sizing                 sonicmoe/ernie_compat/deepep_metadata.py:644-661
"""
from __future__ import annotations

import numpy as np
import torch


def count_cumsum(ids: torch.Tensor, E: int, do_cumsum: bool = True):
    """count[e] = #(ids == e), inclusive cumsum, both int32."""
    cnt = np.bincount(ids.reshape(-1).numpy().astype(np.int64), minlength=E)[:E].astype(np.int32)
    if not do_cumsum:
        return torch.from_numpy(cnt)
    return torch.from_numpy(cnt), torch.from_numpy(np.cumsum(cnt).astype(np.int32))


def sync_free_sizes(N: int, K: int, E: int, alignment: int = 128):
    """Shape-only upper bounds: TK = N*min(K,E), TKp = roundup(TK,128) + E*128."""
    TK = N * min(K, E)
    TKp = (TK + alignment - 1) // alignment * alignment + E * alignment
    return TK, TKp


def padded_offsets(counts: np.ndarray, alignment: int):
    pad = np.where(counts > 0, (counts + alignment - 1) // alignment * alignment, 0)
    efo = np.zeros(len(counts) + 1, dtype=np.int64)
    efo[1:] = np.cumsum(pad)
    return efo


def topk_metadata(idx: torch.Tensor, probs: torch.Tensor, E: int, alignment: int = 128,
                  TK_alloc: int | None = None, TKp_alloc: int | None = None,
                  lane_order: str = "expert", pad_mode: str = "sentinel"):
    """idx [N,K] int32 (valid iff 0 <= e < E; a row's valid experts distinct),
    probs [N,K] f32.

    lane_order "expert": a token's lanes are listed by ascending expert id (the
    CUDA kernel, kernel.cu:567-578); "slot": by top-k slot, so the token-major
    position of (t,k) is naept[t] + (#valid slots before k) - equal to the flat
    index t*K+k when every slot is valid (the dense Triton path).

    pad_mode "sentinel": pad rows' s_scatter_idx = real_TK (kernel.cu:611-650);
    "virtual": the i-th pad row (ascending position) gets real_TK + i
    (functional/__init__.py:226-234).

    Returns dict with efo[E+1], x_gather_idx[TKp], s_scatter_idx[TKp],
    s_reverse_scatter_idx[TK], naept[N+1], topk_scores[TKp], score_src_idx[TK],
    counts[E], real_TK, real_TKp.
    """
    idx_np = idx.numpy().astype(np.int64)
    pr_np = probs.numpy().astype(np.float32)
    N, K = idx_np.shape
    valid = (idx_np >= 0) & (idx_np < E)
    counts = np.bincount(idx_np[valid], minlength=E).astype(np.int64)
    efo = padded_offsets(counts, alignment)
    real_TK = int(valid.sum())
    real_TKp = int(efo[-1])
    TK = real_TK if TK_alloc is None else TK_alloc
    TKp = real_TKp if TKp_alloc is None else TKp_alloc
    assert TK >= real_TK and TKp >= real_TKp

    naept = np.zeros(N + 1, dtype=np.int64)
    naept[1:] = np.cumsum(valid.sum(axis=1))

    if lane_order == "expert":
        masked = np.where(valid, idx_np, np.iinfo(np.int64).max)
        rank = (masked[:, None, :] < masked[:, :, None]).sum(axis=2)  # [N,K]: #valid j with e_j < e_k
    else:
        rank = np.cumsum(valid, axis=1) - valid  # valid slots before k
    t_ids, k_ids = np.nonzero(valid)              # row-major: ascending t, then k
    e_ids = idx_np[t_ids, k_ids]
    order = np.argsort(e_ids, kind="stable")      # ascending expert, then ascending flat index
    if lane_order == "expert":
        # inside an expert rows are ascending token index; with distinct experts per
        # row that equals ascending flat index, which the stable sort already gives.
        pass
    t_s, k_s, e_s = t_ids[order], k_ids[order], e_ids[order]
    base = np.zeros(E, dtype=np.int64)
    base[1:] = np.cumsum(counts)[:-1]
    local = np.arange(real_TK) - base[e_s]
    pos = efo[e_s] + local                        # padded expert-sorted position
    tm = naept[t_s] + rank[t_s, k_s]              # token-major position

    x_gather = np.zeros(TKp, dtype=np.int32)
    s_scatter = np.full(TKp, real_TK, dtype=np.int32)
    s_rev = np.zeros(TK, dtype=np.int32)
    scores = np.zeros(TKp, dtype=np.float32)
    src = np.zeros(TK, dtype=np.int32)
    x_gather[pos] = t_s
    s_scatter[pos] = tm
    s_rev[tm] = pos
    scores[tm] = pr_np[t_s, k_s]
    src[tm] = t_s * K + k_s
    if pad_mode == "virtual":
        is_real = np.zeros(TKp, dtype=bool)
        is_real[pos] = True
        pads = np.nonzero(~is_real)[0]
        s_scatter[pads] = real_TK + np.arange(len(pads))
    out = dict(efo=efo.astype(np.int32), x_gather_idx=x_gather, s_scatter_idx=s_scatter,
               s_reverse_scatter_idx=s_rev, naept=naept.astype(np.int32), topk_scores=scores,
               score_src_idx=src, counts=counts.astype(np.int32))
    out = {k: torch.from_numpy(v) for k, v in out.items()}
    out["real_TK"] = real_TK
    out["real_TKp"] = real_TKp
    return out


def dense_topk_metadata(topk_idx: torch.Tensor, E: int):
    """Unpadded dense [T,K] metadata: efo[E+1], expert_frequency[E],
    x_gather_idx[TK] = token of the sorted entry, s_scatter_idx[TK] = flat t*K+k of
    the sorted entry, s_reverse_scatter_idx = inverse permutation."""
    T, K = topk_idx.shape
    flat = topk_idx.reshape(-1).numpy().astype(np.int64)
    order = np.argsort(flat, kind="stable")
    cnt = np.bincount(flat, minlength=E).astype(np.int32)
    efo = np.zeros(E + 1, dtype=np.int32)
    efo[1:] = np.cumsum(cnt)
    s_rev = np.empty(T * K, dtype=np.int32)
    s_rev[order] = np.arange(T * K, dtype=np.int32)
    return dict(expert_frequency=torch.from_numpy(cnt), efo=torch.from_numpy(efo),
                x_gather_idx=torch.from_numpy((order // K).astype(np.int32)),
                s_scatter_idx=torch.from_numpy(order.astype(np.int32)),
                s_reverse_scatter_idx=torch.from_numpy(s_rev))
