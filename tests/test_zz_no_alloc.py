"""The allocation-free routing-metadata entry point, smoe_topk_metadata_static.

Some callers of this library cannot allocate device memory at the moment they need routing metadata:
work that is being captured into a CUDA graph, code running from a stream callback, a serving process
that forbids cudaMalloc once it has started, or a host framework whose caching allocator the library
cannot reach.  For them the entry point keeps its scratch in a fixed array inside the library.  This
test drives it through the C ABI, twice in a row with different inputs (the array keeps the first
call's contents), and requires exactly the bytes the ordinary entry point writes.  It is collected last
so that a run stopping at the first failure has already executed everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
KEYS = ["efo", "x_gather_idx", "s_scatter_idx", "s_reverse_scatter_idx", "naept", "topk_scores", "score_src_idx",
        "counts"]


def _routing(N, K, E, p_mask, seed):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randn(N, E, generator=g).topk(K, dim=-1).indices.to(torch.int32)
    if p_mask > 0:
        idx = torch.where(torch.rand(N, K, generator=g) < p_mask, torch.full_like(idx, -1), idx)
    return idx, torch.rand(N, K, generator=g)


def _static_call(lib, idx, probs, E, TK, TKp):
    N, K = idx.shape
    mk = lambda n, dt=torch.int32: torch.full((n,), -7, dtype=dt, device=DEV)
    out = dict(efo=mk(E + 1), x_gather_idx=mk(TKp), s_scatter_idx=mk(TKp), s_reverse_scatter_idx=mk(TK),
               naept=mk(N + 1), topk_scores=mk(TKp, torch.float32), score_src_idx=mk(TK), counts=mk(E))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.smoe_topk_metadata_static(p(idx), p(probs), N, K, E, 128, TK, TKp, 0, 0, p(out["efo"]),
                                       p(out["x_gather_idx"]), p(out["s_scatter_idx"]),
                                       p(out["s_reverse_scatter_idx"]), p(out["naept"]), p(out["topk_scores"]),
                                       p(out["score_src_idx"]), p(out["counts"]),
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_scratch_entry_point_matches_the_allocating_one_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sonicmoe import ops
    from sonicmoe._lib import lib
    assert lib.smoe_topk_metadata_static_capacity() == 1 << 20
    # two calls in a row, the second smaller and sparser than the first: stale scratch must not leak through
    for N, K, E, p_mask, seed in [(8192, 8, 64, 0.1, 1), (1000, 4, 16, 0.6, 2)]:
        idx, probs = _routing(N, K, E, p_mask, seed)
        idx, probs = idx.to(DEV), probs.to(DEV)
        ref = ops.topk_metadata(idx, probs, E, 128)
        rc, got = _static_call(lib, idx, probs, E, ref["TK_alloc"], ref["TKp_alloc"])
        assert rc == 0
        torch.cuda.synchronize()
        for k in KEYS:
            assert torch.equal(got[k], ref[k]), k
    # a problem whose scratch need exceeds the fixed array is refused on the host, before any launch
    N, K, E = 65536, 8, 256
    assert lib.smoe_topk_metadata_workspace(N, E) > lib.smoe_topk_metadata_static_capacity()
    idx, probs = _routing(64, K, E, 0.0, 3)
    rc = lib.smoe_topk_metadata_static(None, None, N, K, E, 128, 0, 0, 0, 0, None, None, None, None, None, None, None,
                                       None, None)
    assert rc == 1      # SMOE_ERR_SHAPE
