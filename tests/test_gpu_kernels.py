"""GPU parity tests of the individual kernels (through the C ABI) against the CPU oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import moe as OM
from oracle import quant as Q
from oracle import routing as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sonicmoe import ops as _ops
    return _ops


DEV = "cuda"


def make_routing(N, K, E, p_mask=0.0, seed=0, skew=False):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(N, E, generator=g)
    if skew:
        p = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
        logits = logits + torch.log(p / p.sum())[torch.randperm(E, generator=g)]
    idx = logits.topk(K, dim=-1).indices.to(torch.int32)
    if p_mask > 0:
        idx = torch.where(torch.rand(N, K, generator=g) < p_mask, torch.full_like(idx, -1), idx)
    probs = torch.rand(N, K, generator=g, dtype=torch.float32)
    return idx, probs


MD_KEYS = ["efo", "x_gather_idx", "s_scatter_idx", "s_reverse_scatter_idx", "naept", "topk_scores", "score_src_idx",
           "counts"]


@pytest.mark.parametrize("N,K,E,p_mask,skew", [
    (256, 2, 8, 0.0, False), (8192, 8, 8, 0.0, False), (4096, 8, 128, 0.0, True), (1000, 8, 64, 0.4, False),
    (1, 8, 16, 0.0, False), (77, 6, 6, 1.0, False), (33, 4, 4, 0.9, False), (0, 4, 8, 0.0, False),
    (2048, 16, 256, 0.2, True)])
@pytest.mark.parametrize("lane_order,pad_mode", [(0, 0), (1, 1)])
def test_topk_metadata_bit_exact(ops, N, K, E, p_mask, skew, lane_order, pad_mode):
    idx, probs = make_routing(N, K, E, p_mask, seed=N + K + E, skew=skew)
    got = ops.topk_metadata(idx.to(DEV), probs.to(DEV), E, 128, lane_order=lane_order, pad_mode=pad_mode)
    ref = R.topk_metadata(idx, probs, E, 128, TK_alloc=got["TK_alloc"], TKp_alloc=got["TKp_alloc"],
                          lane_order=["expert", "slot"][lane_order], pad_mode=["sentinel", "virtual"][pad_mode])
    for k in MD_KEYS:
        assert torch.equal(got[k].cpu(), ref[k]), k
    # exact sizing too
    got = ops.topk_metadata(idx.to(DEV), probs.to(DEV), E, 128, TK_alloc=ref["real_TK"], TKp_alloc=ref["real_TKp"],
                            lane_order=lane_order, pad_mode=pad_mode)
    ref = R.topk_metadata(idx, probs, E, 128, lane_order=["expert", "slot"][lane_order],
                          pad_mode=["sentinel", "virtual"][pad_mode])
    for k in MD_KEYS:
        assert torch.equal(got[k].cpu(), ref[k]), k


def test_topk_metadata_alignment_one(ops):
    idx, probs = make_routing(500, 4, 16, 0.1, seed=9)
    got = ops.topk_metadata(idx.to(DEV), probs.to(DEV), 16, 1)
    ref = R.topk_metadata(idx, probs, 16, 1, TK_alloc=got["TK_alloc"], TKp_alloc=got["TKp_alloc"])
    for k in MD_KEYS:
        assert torch.equal(got[k].cpu(), ref[k]), k


@pytest.mark.parametrize("n,E,dt", [(65536, 8, torch.int32), (1000, 128, torch.int64), (0, 4, torch.int32),
                                    (131072, 50000, torch.int32)])
def test_count_cumsum(ops, n, E, dt):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, E, (n,), generator=g).to(dt)
    c, cs = ops.count_cumsum(ids.to(DEV), E)
    rc, rcs = R.count_cumsum(ids, E)
    assert torch.equal(c.cpu(), rc) and torch.equal(cs.cpu(), rcs)


def adversarial_rows(M, K, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[0] = 0.0                                     # all-zero groups -> scale byte 0
    x[1, :32] = 0.0
    x[1, 5] = 1.75 * 2.0 ** 3                      # exactly at the carry threshold
    x[2, :32] = 0.0
    x[2, 7] = 1.875 * 2.0 ** -5                    # just above it
    x[3] *= 1e-30                                  # tiny
    x[4] *= 1e30                                   # huge
    x[5, 3] = 448.0 * 2.0 ** 4
    x[6] *= 1e-3
    x[7, ::3] = 0.0
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("M,K", [(256, 256), (8192, 3072), (100, 128), (64, 1536)])
def test_quant_rows_bit_exact(ops, M, K):
    x = adversarial_rows(M, K, M + K)
    q, raw, isa = ops.quant_rows(x.to(DEV), raw=True, isa=True)
    rq, rs = Q.row_quant(x)
    assert torch.equal(q.cpu(), rq)
    assert torch.equal(raw.cpu(), rs)
    assert torch.equal(Q.unpack_isa(isa.cpu(), M, K), rs)


def test_gather_scales_isa(ops):
    T, K, rows = 300, 512, 1024
    g = torch.Generator().manual_seed(3)
    raw = torch.randint(0, 256, (T, K // 32), generator=g, dtype=torch.uint8)
    idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    got = ops.gather_scales_isa(raw.to(DEV), idx.to(DEV), rows, K)
    assert torch.equal(got.cpu(), Q.gather_scales_to_isa(raw, idx, K))


def test_quant_rows_gather_bit_exact(ops):
    T, K, rows, valid = 300, 1536, 1024, 900
    x = adversarial_rows(T, K, 21)
    g = torch.Generator().manual_seed(22)
    idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    q, isa = ops.quant_rows_gather(x.to(DEV), idx.to(DEV), rows, torch.tensor([valid], dtype=torch.int32).to(DEV))
    rq, rs = Q.row_quant(x)
    assert torch.equal(q.cpu()[:valid], rq[idx.long()][:valid])
    assert torch.equal(Q.unpack_isa(isa.cpu(), rows, K)[:valid], rs[idx.long()][:valid])


@pytest.mark.parametrize("N,K,E,H,p_mask", [(500, 4, 8, 512, 0.3), (2048, 8, 16, 3072, 0.0), (64, 2, 4, 6144, 0.5)])
def test_quant_rows_scatter_bit_exact(ops, N, K, E, H, p_mask):
    idx, probs = make_routing(N, K, E, p_mask, seed=N)
    md = R.topk_metadata(idx, probs, E, 128)
    x = adversarial_rows(N, H, N + 1)
    rows = md["real_TKp"] + 128                     # over-allocated tail stays untouched
    dev = lambda k: md[k].to(DEV)
    sscat = torch.cat([md["s_scatter_idx"], torch.full((128,), md["real_TK"], dtype=torch.int32)]).to(DEV)
    q, isa = ops.quant_rows_scatter(x.to(DEV), dev("naept"), dev("s_reverse_scatter_idx"), sscat, rows,
                                    dev("efo")[-1:])
    rq, rs = Q.row_quant(x)
    real = md["s_scatter_idx"] < md["real_TK"]
    xg = md["x_gather_idx"].long()
    got_q, got_s = q.cpu()[:md["real_TKp"]], Q.unpack_isa(isa.cpu(), rows, H)[:md["real_TKp"]]
    assert torch.equal(got_q[real], rq[xg][real]) and torch.equal(got_s[real], rs[xg][real])
    assert (got_q[~real] == 0).all() and (got_s[~real] == 0).all()


def test_gather_rows_fp8(ops):
    T, K, rows, valid = 300, 512, 1024, 896
    g = torch.Generator().manual_seed(8)
    q = torch.randint(0, 256, (T, K), generator=g, dtype=torch.uint8)
    raw = torch.randint(0, 256, (T, K // 32), generator=g, dtype=torch.uint8)
    idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    vr = torch.tensor([valid], dtype=torch.int32)
    out, isa = ops.gather_rows_fp8(q.to(DEV), raw.to(DEV), idx.to(DEV), rows, vr.to(DEV))
    assert torch.equal(out.cpu()[:valid], q[idx.long()][:valid])
    assert torch.equal(Q.unpack_isa(isa.cpu(), rows, K)[:valid], raw[idx.long()][:valid])


@pytest.mark.parametrize("N,K,E,topk,p_mask", [(300, 512, 8, 4, 0.3), (1000, 3072, 16, 8, 0.0), (64, 128, 4, 2, 0.9)])
def test_scatter_rows_fp8_matches_gather_form(ops, N, K, E, topk, p_mask):
    """Scatter form of the row copy = gather form on real rows; pad rows are zero (bytes and scales)."""
    idx, probs = make_routing(N, topk, E, p_mask, seed=N + K)
    md = ops.topk_metadata(idx.to(DEV), probs.to(DEV), E, 128)
    g = torch.Generator().manual_seed(K)
    q = torch.randint(0, 256, (N, K), generator=g, dtype=torch.uint8).to(DEV)
    raw = torch.randint(0, 256, (N, K // 32), generator=g, dtype=torch.uint8).to(DEV)
    rows = md["TKp_alloc"]
    valid = md["efo"][-1:]
    got_q, got_isa = ops.scatter_rows_fp8(q, raw, md["naept"], md["s_reverse_scatter_idx"], md["s_scatter_idx"],
                                          rows, valid)
    ref_q, ref_isa = ops.gather_rows_fp8(q, raw, md["x_gather_idx"], rows, valid)
    torch.cuda.synchronize()
    n = int(valid)
    real_tk = int(md["naept"][-1])
    real = (md["s_scatter_idx"][:n] < real_tk).cpu()
    assert torch.equal(got_q[:n].cpu()[real], ref_q[:n].cpu()[real])
    gs, rs = Q.unpack_isa(got_isa.cpu(), rows, K)[:n], Q.unpack_isa(ref_isa.cpu(), rows, K)[:n]
    assert torch.equal(gs[real], rs[real])
    assert (got_q[:n].cpu()[~real] == 0).all() and (gs[~real] == 0).all()


@pytest.mark.parametrize("T,dim,rows", [(256, 256, 512), (1000, 3072, 2048), (64, 64, 128)])
def test_quant_cols_transposed_bit_exact(ops, T, dim, rows):
    x = adversarial_rows(T, dim, T + dim)
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    q_t, isa = ops.quant_cols_t(x.to(DEV), idx.to(DEV), rows)
    rq, rs = Q.col_quant(x, idx)
    assert torch.equal(q_t.cpu(), rq.t().contiguous())
    assert torch.equal(Q.unpack_isa(isa.cpu(), dim, rows), rs)
    # without gather
    x2 = adversarial_rows(rows, dim, 11)
    q_t, isa = ops.quant_cols_t(x2.to(DEV), None, rows)
    rq, rs = Q.col_quant(x2)
    assert torch.equal(q_t.cpu(), rq.t().contiguous())
    assert torch.equal(Q.unpack_isa(isa.cpu(), dim, rows), rs)


@pytest.mark.parametrize("rows,cols", [(128, 128), (512, 3072), (1024, 256)])
def test_quant_iso32_bit_exact(ops, rows, cols):
    x = adversarial_rows(rows, cols, rows * 3 + cols)
    q, ri, q_t, ci = ops.quant_iso32(x.to(DEV))
    rq, bs = Q.iso32_quant(x)
    assert torch.equal(q.cpu(), rq)
    assert torch.equal(q_t.cpu(), rq.t().contiguous())
    assert torch.equal(Q.unpack_isa(ri.cpu(), rows, cols), bs.repeat_interleave(32, dim=0))
    assert torch.equal(Q.unpack_isa(ci.cpu(), cols, rows), bs.t().repeat_interleave(32, dim=0))


def test_combine_matches_oracle_and_repeats(ops):
    N, K, E, H = 512, 8, 16, 1024
    idx, probs = make_routing(N, K, E, 0.2, seed=2)
    md = R.topk_metadata(idx, probs, E, 128)
    g = torch.Generator().manual_seed(4)
    y2 = torch.randn(md["real_TKp"], H, generator=g).to(torch.bfloat16)
    for weighted in (True, False):
        ref = OM.combine(y2, md, N, weighted).to(torch.bfloat16)
        got = ops.combine(y2.to(DEV), md["s_reverse_scatter_idx"].to(DEV), md["naept"].to(DEV),
                          md["topk_scores"].to(DEV) if weighted else None, N)
        got2 = ops.combine(y2.to(DEV), md["s_reverse_scatter_idx"].to(DEV), md["naept"].to(DEV),
                           md["topk_scores"].to(DEV) if weighted else None, N)
        assert torch.equal(got, got2)
        # fp32 fma vs mul+add: at most 1 bf16 ulp apart
        d = (got.cpu().float() - ref.float()).abs()
        assert (d <= ref.float().abs() * 2 ** -7 + 1e-6).all()


@pytest.mark.parametrize("T,E,K", [(1000, 8, 8), (512, 128, 8), (64, 64, 1), (300, 256, 16)])
def test_topk_softmax_fwd_bwd(ops, T, E, K):
    g = torch.Generator().manual_seed(T)
    logits = torch.randn(T, E, generator=g)
    s, i = ops.topk_softmax(logits.to(DEV), K)
    rs, ri = OM.router_topk_softmax(logits, K)
    assert torch.equal(i.cpu(), ri)
    torch.testing.assert_close(s.cpu(), rs, rtol=1e-5, atol=1e-7)
    dsc = torch.randn(T, K, generator=g)
    dl = ops.topk_softmax_bwd(s, i, dsc.to(DEV), E)
    torch.testing.assert_close(dl.cpu(), OM.router_backward(s.cpu(), ri, dsc, E), rtol=1e-5, atol=1e-6)


def test_topk_softmax_rows_with_fewer_than_k_finite_logits(ops):
    """-inf-masked and NaN logits: the K indices stay distinct and in range (the finite ones first, then the lowest
    unused index with a score of exactly zero), the scores of the finite picks are their softmax, and the backward
    writes nothing outside [0, E)."""
    T, E, K = 64, 16, 4
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(T, E, generator=g)
    logits[0, :] = float("-inf")                           # nothing selectable
    logits[1, 2:] = float("-inf")                          # two finite logits
    logits[2, :] = float("nan")                            # NaN counts as -inf
    logits[3, 5] = float("nan")                            # one NaN among finite ones: never picked first
    logits[4, 3:] = float("-inf"); logits[4, 1] = float("nan")
    s, i = ops.topk_softmax(logits.to(DEV), K)
    s, i = s.cpu(), i.cpu()
    assert ((i >= 0) & (i < E)).all()
    assert all(len(set(row.tolist())) == K for row in i)
    assert torch.isfinite(s).all()
    assert (s[0] == 0).all() and i[0].tolist() == [0, 1, 2, 3]
    assert set(i[1, :2].tolist()) == {0, 1} and (s[1, 2:] == 0).all() and abs(float(s[1, :2].sum()) - 1) < 1e-6
    assert (s[2] == 0).all()
    assert 5 not in i[3].tolist()
    assert set(i[4, :2].tolist()) == {0, 2} and (s[4, 2:] == 0).all()
    clean = torch.nan_to_num(logits[5:], nan=float("-inf"))
    rs, ri = OM.router_topk_softmax(clean, K)
    assert torch.equal(i[5:], ri)
    torch.testing.assert_close(s[5:], rs, rtol=1e-5, atol=1e-7)
    # backward with a deliberately out-of-range index: ignored, neighbours untouched
    bad = i.clone()
    bad[0, 0] = 0x7fffffff
    bad[1, 1] = -3
    guard = torch.full((T + 2, E), 7.0, device=DEV)
    dl = guard[1:-1]
    from sonicmoe._lib import lib, check
    dsc = torch.randn(T, K, generator=g).to(DEV)
    sd, bd = s.to(DEV), bad.to(DEV)
    check(lib.smoe_topk_softmax_bwd(sd.data_ptr(), bd.data_ptr(), dsc.data_ptr(), T, E, K, dl.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream), "topk_softmax_bwd")
    torch.cuda.synchronize()
    assert (guard[0] == 7).all() and (guard[-1] == 7).all() and torch.isfinite(dl).all()


def test_topk_metadata_with_undersized_buffers_stays_in_bounds(ops):
    """Buffers sized from per-expert counts that are too small for what idx holds: the rows that do not fit are
    dropped and the published offsets are clamped - nothing is written past the allocations."""
    N, K, E = 512, 4, 8
    g = torch.Generator().manual_seed(3)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(N)]).to(torch.int32)
    probs = torch.rand(N, K, generator=g)
    TK, TKp = 1024, 1024                                    # the truth is 2048 routed pairs
    from sonicmoe._lib import lib, check
    dev = DEV
    e = lambda n, dt=torch.int32: torch.full((n + 64,), -77, dtype=dt, device=dev)
    efo, xg, ss, sr, na = e(E + 1), e(TKp), e(TKp), e(TK), e(N + 1)
    sc, si, cnt = torch.full((TKp + 64,), -77.0, device=dev), e(TK), e(E)
    ws = torch.empty(lib.smoe_topk_metadata_workspace(N, E), dtype=torch.uint8, device=dev)
    idx_d, probs_d = idx.to(dev), probs.to(dev)
    check(lib.smoe_topk_metadata(idx_d.data_ptr(), probs_d.data_ptr(), N, K, E, 128, TK, TKp, 0, 0,
                                 efo.data_ptr(), xg.data_ptr(), ss.data_ptr(), sr.data_ptr(), na.data_ptr(),
                                 sc.data_ptr(), si.data_ptr(), cnt.data_ptr(), ws.data_ptr(),
                                 torch.cuda.current_stream().cuda_stream), "topk_metadata")
    torch.cuda.synchronize()
    for buf, n in ((efo, E + 1), (xg, TKp), (ss, TKp), (sr, TK), (na, N + 1), (si, TK), (cnt, E)):
        assert (buf[n:] == -77).all()
    assert (sc[TKp:] == -77.0).all()
    assert int(efo[:E + 1].max()) <= TKp and int(cnt[:E].sum()) == N * K
    assert ((xg[:TKp] >= 0) & (xg[:TKp] < N)).all() and ((sr[:TK] >= 0) & (sr[:TK] < TKp)).all()


# ------------------------------------------------------------------ GEMMs
def rand_fp8(shape, g, lo_exp=118, hi_exp=126):
    """Random e4m3 bytes (no NaN) and random ue8m0 scale bytes per 1x32 group."""
    q = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8)
    q = torch.where((q & 0x7F) == 0x7F, q & 0xF0, q)
    sc = torch.randint(lo_exp, hi_exp + 1, shape[:-1] + (shape[-1] // 32,), generator=g, dtype=torch.uint8)
    return q, sc


def deq(q, sc):
    sh = q.shape
    return Q.dequant_rows(q.reshape(-1, sh[-1]), sc.reshape(-1, sh[-1] // 32)).reshape(sh)


def make_efo(counts128):
    efo = torch.zeros(len(counts128) + 1, dtype=torch.int32)
    efo[1:] = torch.cumsum(torch.tensor(counts128) * 128, 0)
    return efo


def stats(got, ref):
    got, ref = got.float().flatten(), ref.float().flatten()
    cos = float((got * ref).sum() / (got.norm() * ref.norm()).clamp(min=1e-30))
    rr = float((got - ref).norm() / ref.norm().clamp(min=1e-30))
    return cos, rr


# 384 = the 256 x 384 double-accumulator kernel (N % 384 == 0; other N fall back); bit 17 = the single-CTA kernel
@pytest.mark.parametrize("bn", [128, 192, 256, 384, 128 | (1 << 17), 256 | (1 << 17)])
@pytest.mark.parametrize("tiles,N,K", [([1, 0, 2, 1], 256, 128), ([3, 2, 0, 0, 4, 1, 1, 2], 512, 1024),
                                        ([40, 30, 50, 28], 1536, 768), ([5, 4, 0, 7], 768, 256), ([6, 5], 384, 512),
                                        ([3, 0, 1], 768, 640)])
def test_gemm_varlen_m(ops, bn, tiles, N, K):
    from sonicmoe._lib import lib
    g = torch.Generator().manual_seed(sum(tiles) + N + K)
    E = len(tiles)
    efo = make_efo(tiles)
    rows = int(efo[-1]) + 256                       # over-allocated tail must be ignored
    a_q, a_sc = rand_fp8((rows, K), g)
    b_q, b_sc = rand_fp8((E, N, K), g)
    a_sf = Q.pack_isa(a_sc, rows, K)
    b_sf = Q.pack_isa(b_sc.reshape(E * N, K // 32), E * N, K)
    lib.smoe_internal_gemm_knobs(bn)
    try:
        c = ops.gemm_varlen_m(a_q.to(DEV), a_sf.to(DEV), b_q.to(DEV), b_sf.to(DEV), efo.to(DEV))
        torch.cuda.synchronize()
        ops.check_status(DEV)
    finally:
        lib.smoe_internal_gemm_knobs(0)
    A, B = deq(a_q, a_sc).to(DEV), deq(b_q, b_sc).to(DEV)
    for e in range(E):
        a, b = int(efo[e]), int(efo[e + 1])
        if b > a:
            ref = (A[a:b] @ B[e].T)
            cos, rr = stats(c[a:b], ref)
            assert cos > 0.99999 and rr < 4e-3, (e, cos, rr)


def gated_inputs(T, H, I, tiles, seed):
    g = torch.Generator().manual_seed(seed)
    E = len(tiles)
    efo = make_efo(tiles)
    rows = int(efo[-1])
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    a_idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    return g, E, efo, rows, x, w1, a_idx


GATED_SHAPES = [(300, 256, 128, [1, 2, 0, 1]), (2000, 1024, 512, [5, 3, 9, 0, 0, 2, 1, 4]),
                (1000, 512, 768, [3, 1, 2])]
# A rows: "tma_gather" = fetched by index inside the GEMM (two-CTA kernel: cp.async load warps; with "4": TMA gather4;
# single-CTA kernel: TMA gather4); "gathered" = expert-sorted copy, tiled TMA; the "_1cta" variants run the
# single-CTA kernel
GATHER_MODES = ["tma_gather", "tma_gather4", "gathered", "tma_gather_1cta", "gathered_1cta"]


def _force(mode):
    from sonicmoe._lib import lib
    bits = (1 << 17) if mode.endswith("_1cta") else 0
    if mode == "tma_gather4":
        bits |= -(1 << 31)            # bit 31 of a 32-bit int
    lib.smoe_internal_gemm_knobs(bits)


@pytest.mark.parametrize("T,H,I,tiles", GATED_SHAPES)
def test_gemm_gated_same_bytes_for_every_column_tile(ops, T, H, I, tiles):
    """128-, 192- and 256-column tiles (two accumulator stages vs. one drained into registers) agree bit for bit."""
    from sonicmoe._lib import lib
    g, E, efo, rows, x, w1, a_idx = gated_inputs(T, H, I, tiles, 11)
    xq, xs = Q.row_quant(x)
    wq, ws = Q.row_quant(w1.reshape(E * 2 * I, H))
    args = (xq[a_idx.long()].contiguous().to(DEV), None, Q.gather_scales_to_isa(xs, a_idx, H).to(DEV),
            wq.reshape(E, 2 * I, H).to(DEV), Q.pack_isa(ws, E * 2 * I, H).to(DEV), efo.to(DEV), rows)
    outs = {}
    for bn in (128, 192, 256):
        lib.smoe_internal_gemm_knobs(bn)
        try:
            outs[bn] = ops.gemm_gated(*args)
            torch.cuda.synchronize()
            ops.check_status(DEV)
        finally:
            lib.smoe_internal_gemm_knobs(0)
    n = int(efo[-1])
    for bn in (192, 256):
        for got, want in zip(outs[bn], outs[128]):
            if got.ndim == 2:
                assert torch.equal(got[:n], want[:n]), bn
        assert torch.equal(Q.unpack_isa(outs[bn][3].cpu(), rows, I)[:n], Q.unpack_isa(outs[128][3].cpu(), rows, I)[:n])


@pytest.mark.parametrize("mode", GATHER_MODES)
@pytest.mark.parametrize("T,H,I,tiles", GATED_SHAPES)
def test_gemm_gated(ops, T, H, I, tiles, mode):
    g, E, efo, rows, x, w1, a_idx = gated_inputs(T, H, I, tiles, 7)
    xq, xs = Q.row_quant(x)
    wq, ws = Q.row_quant(w1.reshape(E * 2 * I, H))
    a_sf = Q.gather_scales_to_isa(xs, a_idx, H)
    w_sf = Q.pack_isa(ws, E * 2 * I, H)
    _force(mode)
    try:
        if mode.startswith("tma_gather"):
            a_in, idx_in = xq.to(DEV), a_idx.to(DEV)
        else:
            a_in, idx_in = xq[a_idx.long()].contiguous().to(DEV), None
        z_q, z_sc, y1_q, y1_sf = ops.gemm_gated(a_in, idx_in, a_sf.to(DEV), wq.reshape(E, 2 * I, H).to(DEV),
                                                w_sf.to(DEV), efo.to(DEV), rows)
    finally:
        _force("")
    torch.cuda.synchronize()
    ops.check_status(DEV)
    X = Q.dequant_rows(xq, xs)[a_idx.long()]
    W = Q.dequant_rows(wq, ws).reshape(E, 2 * I, H)
    z = torch.cat([X[int(efo[e]):int(efo[e + 1])] @ W[e].T for e in range(E)])
    rz_q, rz_s = Q.row_quant(z, amax_floor=1e-4)
    y1 = Q.bf16_rne(OM.swiglu(z))
    ry_q, ry_s = Q.row_quant(y1)
    # scale bytes agree except where the fp32 summation order moves amax across a rounding boundary
    zs_mis = (z_sc.cpu() != rz_s).float().mean().item()
    ys_mis = (Q.unpack_isa(y1_sf.cpu(), rows, I) != ry_s).float().mean().item()
    assert zs_mis < 2e-3 and ys_mis < 2e-3, (zs_mis, ys_mis)
    cos, rr = stats(Q.dequant_rows(z_q.cpu(), z_sc.cpu()), z)
    assert cos > 0.999 and rr < 0.04, (cos, rr)
    cos, rr = stats(Q.dequant_rows(y1_q.cpu(), Q.unpack_isa(y1_sf.cpu(), rows, I)), y1)
    assert cos > 0.999 and rr < 0.04, (cos, rr)
    # where scale bytes agree the payload bytes agree almost everywhere (1-ulp flips only)
    same = (z_sc.cpu() == rz_s).repeat_interleave(32, dim=1)
    byte_mis = ((z_q.cpu() != rz_q) & same).float().mean().item()
    assert byte_mis < 0.02, byte_mis


@pytest.mark.parametrize("mode", GATHER_MODES)
@pytest.mark.parametrize("T,H,I,tiles", GATED_SHAPES)
def test_gemm_dgated(ops, T, H, I, tiles, mode):
    g, E, efo, rows, dout, _, a_idx = gated_inputs(T, H, I, tiles, 13)
    w2t = (torch.randn(E, I, H, generator=g) * 0.05).to(torch.bfloat16)
    z = torch.randn(rows, 2 * I, generator=g)
    zq, zs = Q.row_quant(z, amax_floor=1e-4)
    s = torch.rand(rows, generator=g)
    s[::7] = 0.0
    dq, dsc = Q.row_quant(dout)
    wq, ws = Q.row_quant(w2t.reshape(E * I, H))
    a_sf = Q.gather_scales_to_isa(dsc, a_idx, H)
    w_sf = Q.pack_isa(ws, E * I, H)
    _force(mode)
    try:
        if mode.startswith("tma_gather"):
            a_in, idx_in = dq.to(DEV), a_idx.to(DEV)
        else:
            a_in, idx_in = dq[a_idx.long()].contiguous().to(DEV), None
        dz, y1s, dsp = ops.gemm_dgated(a_in, idx_in, a_sf.to(DEV), wq.reshape(E, I, H).to(DEV), w_sf.to(DEV),
                                       efo.to(DEV), zq.to(DEV), zs.to(DEV), s.to(DEV), rows)
    finally:
        _force("")
    torch.cuda.synchronize()
    ops.check_status(DEV)
    Dm = Q.dequant_rows(dq, dsc)[a_idx.long()]
    W = Q.dequant_rows(wq, ws).reshape(E, I, H)
    D = torch.cat([Dm[int(efo[e]):int(efo[e + 1])] @ W[e].T for e in range(E)])
    rdz, y = OM.dswiglu(Q.dequant_rows(zq, zs), s.unsqueeze(1) * D)
    for got, ref in ((dz, rdz), (y1s, s.unsqueeze(1) * y), (dsp.sum(0), (y * D).sum(1))):
        cos, rr = stats(got.cpu(), ref)
        assert cos > 0.9999 and rr < 6e-3, (cos, rr)
    assert (dz.cpu()[s == 0] == 0).all() and (y1s.cpu()[s == 0] == 0).all()


@pytest.mark.parametrize("bn", [128, 192, 256, 384, 128 | (1 << 17), 256 | (1 << 17)])
@pytest.mark.parametrize("M,N,tiles", [(128, 256, [1, 0, 2, 1]), (512, 768, [3, 2, 0, 0, 4, 1, 1, 2]), (768, 384, [2, 1, 3]),
                                       (256, 1152, [5, 0, 9, 4])])
def test_gemm_wgrad(ops, bn, M, N, tiles):
    from sonicmoe._lib import lib
    g = torch.Generator().manual_seed(M + N)
    E = len(tiles)
    efo = make_efo(tiles)
    TKp = int(efo[-1]) + 128
    a_q, a_sc = rand_fp8((M, TKp), g)
    b_q, b_sc = rand_fp8((N, TKp), g)
    a_sf, b_sf = Q.pack_isa(a_sc, M, TKp), Q.pack_isa(b_sc, N, TKp)
    A, B = deq(a_q, a_sc).to(DEV), deq(b_q, b_sc).to(DEV)
    init = torch.randn(E, M, N, generator=g)
    lib.smoe_internal_gemm_knobs(bn)
    try:
        out = init.clone().to(DEV)
        ops.gemm_wgrad(a_q.to(DEV), a_sf.to(DEV), b_q.to(DEV), b_sf.to(DEV), efo.to(DEV), out, accumulate=True)
        fresh = torch.full((E, M, N), 7.0, device=DEV)
        ops.gemm_wgrad(a_q.to(DEV), a_sf.to(DEV), b_q.to(DEV), b_sf.to(DEV), efo.to(DEV), fresh, accumulate=False)
        torch.cuda.synchronize()
        ops.check_status(DEV)
    finally:
        lib.smoe_internal_gemm_knobs(0)
    for e in range(E):
        a, b = int(efo[e]), int(efo[e + 1])
        ref = A[:, a:b] @ B[:, a:b].T if b > a else torch.zeros(M, N, device=DEV)
        if b > a:
            cos, rr = stats(fresh[e], ref)
            assert cos > 0.99999 and rr < 1e-4, (e, cos, rr)
        else:
            assert (fresh[e] == 0).all()
        torch.testing.assert_close(out[e], init[e].to(DEV) + ref, rtol=1e-4, atol=1e-2 * ref.abs().max().item() + 1e-6)


@pytest.mark.parametrize("T,K,rows,valid", [(64, 256, 256, 256), (300, 768, 1024, 896), (128, 512, 384, 128)])
def test_quant_dual_gather_matches_single_direction_kernels(ops, T, K, rows, valid):
    """One pass over gathered rows = the bytes of quant_rows_gather (row-wise) and quant_cols_t (column-wise)."""
    g = torch.Generator().manual_seed(T + K)
    x = (torch.randn(T, K, generator=g) * torch.exp(2 * torch.randn(T, 1, generator=g))).to(torch.bfloat16)
    x[3] = 0
    idx = torch.randint(0, T, (rows,), generator=g, dtype=torch.int32)
    xd, idxd = x.to(DEV), idx.to(DEV)
    vr = torch.tensor([valid], dtype=torch.int32, device=DEV)
    q_row, row_isa, q_col, col_isa = ops.quant_dual_gather(xd, idxd, rows, vr)
    c_only = ops.quant_dual_gather(xd, idxd, rows, vr, with_rows=False)
    r_q, r_isa = ops.quant_rows_gather(xd, idxd, rows, vr)
    r_qt, r_cisa = ops.quant_cols_t(xd, idxd, rows)
    torch.cuda.synchronize()
    assert c_only[0] is None and torch.equal(c_only[2][:valid], q_col[:valid])
    assert torch.equal(q_row[:valid], r_q[:valid])
    assert torch.equal(Q.unpack_isa(row_isa.cpu(), rows, K)[:valid], Q.unpack_isa(r_isa.cpu(), rows, K)[:valid])
    assert torch.equal(q_col[:valid].t(), r_qt[:, :valid])
    got, want = Q.unpack_isa(col_isa.cpu(), K, rows), Q.unpack_isa(r_cisa.cpu(), K, rows)
    assert torch.equal(got[:, :valid // 32], want[:, :valid // 32])
    assert torch.equal(Q.unpack_isa(c_only[3].cpu(), K, rows)[:, :valid // 32], want[:, :valid // 32])
    # against the CPU restatement
    o_q, o_sc = Q.col_quant(x[idx[:valid].long()].float())
    assert torch.equal(q_col[:valid].cpu(), o_q) and torch.equal(got[:, :valid // 32], o_sc)


@pytest.mark.parametrize("layout", [1, 2, 3])
@pytest.mark.parametrize("M,N,tiles", [(256, 256, [1, 0, 2, 1]), (512, 768, [3, 2, 0, 0, 4, 1, 1, 2]), (768, 256, [2, 1, 3])])
def test_gemm_wgrad_mn_major_operands(ops, layout, M, N, tiles):
    """Operands kept [TKp, dim] (MN-major for the tensor core) give the bits of the transposed-copy path."""
    g = torch.Generator().manual_seed(M + N + layout)
    E = len(tiles)
    efo = make_efo(tiles)
    TKp = int(efo[-1]) + 128
    a_q, a_sc = rand_fp8((M, TKp), g)
    b_q, b_sc = rand_fp8((N, TKp), g)
    a_sf, b_sf = Q.pack_isa(a_sc, M, TKp).to(DEV), Q.pack_isa(b_sc, N, TKp).to(DEV)
    a_d, b_d, efo_d = a_q.to(DEV), b_q.to(DEV), efo.to(DEV)
    a_in = a_d.t().contiguous() if layout & 1 else a_d
    b_in = b_d.t().contiguous() if layout & 2 else b_d
    init = torch.randn(E, M, N, generator=g).to(DEV)
    for accumulate in (False, True):
        want = init.clone()
        ops.gemm_wgrad(a_d, a_sf, b_d, b_sf, efo_d, want, accumulate=accumulate)
        got = init.clone()
        ops.gemm_wgrad_mn(a_in, a_sf, b_in, b_sf, efo_d, got, accumulate, bool(layout & 1), bool(layout & 2))
        torch.cuda.synchronize()
        ops.check_status(DEV)
        assert torch.equal(got, want), (accumulate, (got - want).abs().max().item())
    A, B = deq(a_q, a_sc).to(DEV), deq(b_q, b_sc).to(DEV)
    for e in range(E):
        a, b = int(efo[e]), int(efo[e + 1])
        if b > a:
            cos, rr = stats(got[e] - init[e], A[:, a:b] @ B[:, a:b].T)
            assert cos > 0.9999 and rr < 1e-3, (e, cos, rr)


# I = 2048 is not a multiple of 192: the fused kernel runs 11 column tiles, the last one ragged (128 of 192 columns)
@pytest.mark.parametrize("bn", [0, 128])
@pytest.mark.parametrize("T,H,I,tiles", GATED_SHAPES + [(600, 256, 2048, [2, 1, 3])])
def test_gemm_dgated_fused_quantizers_match_separate_kernels(ops, T, H, I, tiles, bn):
    """The fused epilogue must emit exactly the bytes of dgated -> quant_iso32(dz) / quant_cols_t(y1s)."""
    from sonicmoe._lib import lib
    g, E, efo, rows, dout, _, a_idx = gated_inputs(T, H, I, tiles, 17)
    w2t = (torch.randn(E, I, H, generator=g) * 0.05).to(torch.bfloat16)
    z = torch.randn(rows, 2 * I, generator=g)
    zq, zs = Q.row_quant(z, amax_floor=1e-4)
    s = torch.rand(rows, generator=g)
    s[::5] = 0.0
    dq, dsc = Q.row_quant(dout)
    wq, ws = Q.row_quant(w2t.reshape(E * I, H))
    a_sf = Q.gather_scales_to_isa(dsc, a_idx, H).to(DEV)
    w_sf = Q.pack_isa(ws, E * I, H).to(DEV)
    a_in = dq[a_idx.long()].contiguous().to(DEV)
    args = (a_sf, wq.reshape(E, I, H).to(DEV), w_sf, efo.to(DEV), zq.to(DEV), zs.to(DEV), s.to(DEV), rows)
    lib.smoe_internal_gemm_knobs(bn)
    try:
        dz, y1s, dsp = ops.gemm_dgated(a_in, None, *args)
        f_dzq, f_rsf, f_csf, f_yq, f_ysf, f_dsp = ops.gemm_dgated_fused(a_in, *args)
        torch.cuda.synchronize()
        ops.check_status(DEV)
    finally:
        lib.smoe_internal_gemm_knobs(0)
    r_q, r_rsf, r_qt, r_csf = ops.quant_iso32(dz)
    r_yt, r_ysf = ops.quant_cols_t(y1s, None, rows)
    n = int(efo[-1])          # rows of real segments (the tail of the allocation is never written)
    assert torch.equal(f_dzq[:n], r_q[:n]) and torch.equal(f_dzq[:n].t(), r_qt[:, :n])
    assert torch.equal(f_yq[:n].t(), r_yt[:, :n])
    assert torch.equal(Q.unpack_isa(f_rsf.cpu(), rows, 2 * I)[:n], Q.unpack_isa(r_rsf.cpu(), rows, 2 * I)[:n])
    assert torch.equal(Q.unpack_isa(f_csf.cpu(), 2 * I, rows)[:, :n // 32], Q.unpack_isa(r_csf.cpu(), 2 * I, rows)[:, :n // 32])
    assert torch.equal(Q.unpack_isa(f_ysf.cpu(), I, rows)[:, :n // 32], Q.unpack_isa(r_ysf.cpu(), I, rows)[:, :n // 32])
    # ds partials are summed over column tiles of different widths in the two kernels: fp32 re-association only
    a, b = f_dsp.sum(0)[:n], dsp.sum(0)[:n]
    assert torch.equal(a, b) or torch.allclose(a, b, rtol=1e-5, atol=1e-5 * float(b.abs().max()))
    # rows fetched by index inside the kernel (cp.async load warps) instead of the gathered copy: the same bits
    lib.smoe_internal_gemm_knobs(bn)
    try:
        g_out = ops.gemm_dgated_fused(dq.to(DEV), *args, a_idx=a_idx.to(DEV))
        torch.cuda.synchronize()
        ops.check_status(DEV)
    finally:
        lib.smoe_internal_gemm_knobs(0)
    for name, got, want in zip(("dz_q", "dz_rsf", "dz_csf", "y1s_q", "y1s_sf"), g_out[:5],
                               (f_dzq, f_rsf, f_csf, f_yq, f_ysf)):
        if got.ndim == 2:
            assert torch.equal(got[:n], want[:n]), name
    assert torch.equal(Q.unpack_isa(g_out[1].cpu(), rows, 2 * I)[:n], Q.unpack_isa(f_rsf.cpu(), rows, 2 * I)[:n])
    assert torch.equal(Q.unpack_isa(g_out[4].cpu(), I, rows)[:, :n // 32], Q.unpack_isa(f_ysf.cpu(), I, rows)[:, :n // 32])
    assert torch.equal(g_out[5].sum(0)[:n], f_dsp.sum(0)[:n])


@pytest.mark.parametrize("T,K,E,world", [(333, 4, 16, 4), (1000, 8, 8, 8), (64, 2, 6, 2)])
def test_ep_dispatch_plan_from_metadata_kernels_matches_torch_construction(ops, T, K, E, world):
    """The plan built with the routing-metadata kernels (destination ranks as experts) equals the device-agnostic
    torch construction; the count exchange is replaced by a loop-back so one GPU suffices."""
    from sonicmoe.ep import DispatchPlan

    class LoopbackPlan(DispatchPlan):
        def _exchange_counts(self, rows_to, pairs, world):
            self.send_counts = rows_to.tolist()
            self.recv_counts = list(self.send_counts)
            self.tokens_per_local_expert = pairs.view(world, -1).sum(0).tolist()
            self.n_send = self.n_recv = sum(self.send_counts)
            self.send_off = [sum(self.send_counts[:r]) for r in range(world)]

    g = torch.Generator().manual_seed(T)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    idx[::7, -1] = -1                                 # dropped slots
    got = LoopbackPlan(idx.to(DEV), E, None, world=world)
    want = LoopbackPlan(idx, E, None, world=world)
    assert got.send_counts == want.send_counts and got.n_send == want.n_send
    assert torch.equal(got.send_tok.cpu(), want.send_tok)
    assert torch.equal(got.send_rank.cpu().long(), want.send_rank.long())
    assert torch.equal(got.send_idx.cpu(), want.send_idx)
    assert torch.equal(got.copy_off.cpu(), want.copy_off)
    assert torch.equal(got.copy_pos.cpu(), want.copy_pos)
    assert got.tokens_per_local_expert == want.tokens_per_local_expert


@pytest.mark.parametrize("T,K,E,world,H", [(333, 4, 16, 4, 256), (500, 8, 8, 8, 512), (64, 2, 6, 2, 128)])
def test_ep_combine_pull_on_one_gpu_with_local_stand_ins_for_the_peers(ops, T, K, E, world, H):
    """The peer-memory combine kernel with every 'peer' buffer on this GPU: result = sum of a token's copies in
    ascending rank order, rows addressed as first_row[rank] + (i - send_off[rank])."""
    from sonicmoe.ep import DispatchPlan

    class LoopbackPlan(DispatchPlan):
        def _exchange_counts(self, rows_to, pairs, world):
            self.send_counts = rows_to.tolist()
            self.recv_counts = list(self.send_counts)
            self.tokens_per_local_expert = pairs.view(world, -1).sum(0).tolist()
            self.n_send = self.n_recv = sum(self.send_counts)
            self.send_off = [sum(self.send_counts[:r]) for r in range(world)]

    g = torch.Generator().manual_seed(T + H)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32)
    idx[::5, 0] = -1
    plan = LoopbackPlan(idx.to(DEV), E, None, world=world)
    first_row = [int(v) for v in torch.randint(0, 50, (world,), generator=g)]      # this rank's rows start anywhere
    bufs = [torch.randn(first_row[r] + plan.send_counts[r] + 7, H, generator=g).to(torch.bfloat16).to(DEV)
            for r in range(world)]
    out = ops.ep_combine_pull([b.data_ptr() for b in bufs], first_row, plan.send_off, plan.copy_pos, plan.copy_off,
                              plan.send_rank, T, H, torch.device(DEV))
    torch.cuda.synchronize()
    want = torch.zeros(T, H)
    send_rank, copy_pos, copy_off = plan.send_rank.cpu(), plan.copy_pos.cpu(), plan.copy_off.cpu()
    for t in range(T):
        for c in range(int(copy_off[t]), int(copy_off[t + 1])):
            i = int(copy_pos[c]); r = int(send_rank[i])
            want[t] += bufs[r][first_row[r] + i - plan.send_off[r]].float().cpu()
    assert torch.equal(out.cpu(), want.to(torch.bfloat16))


def test_transpose_u8_and_plain_gemm_with_b_stored_kn(ops):
    """`transpose_u8` is a byte transpose; `gemm_varlen_m_bt` reads B[e] stored [K,N] (the single ISO32 weight
    buffer) and gives the bits of the K-major GEMM on the byte-transposed copy, and the dequantised fp32 product."""
    g = torch.Generator().manual_seed(77)
    t = torch.randint(0, 256, (3, 128, 192), generator=g, dtype=torch.uint8).to(DEV)
    assert torch.equal(ops.transpose_u8(t), t.transpose(1, 2).contiguous())
    for E, N, K, seg in ((4, 256, 384, (256, 0, 128, 384)), (2, 768, 256, (384, 128))):
        rows = sum(seg)
        efo = torch.tensor([0] + list(torch.tensor(seg).cumsum(0)), dtype=torch.int32, device=DEV)
        a = torch.randn(rows, K, generator=g).to(torch.bfloat16).to(DEV)
        # B logical [E, N, K]; stored as W [E, K, N] quantised with 32x32-block scales
        w = (torch.randn(E, K, N, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
        a_q, _, a_sf = ops.quant_rows(a, raw=False, isa=True)
        q = torch.empty(E, K, N, dtype=torch.uint8, device=DEV)
        per_r, per_c = ops.isa_bytes(K, N), ops.isa_bytes(N, K)
        rsf = torch.empty(E * per_r, dtype=torch.uint8, device=DEV)
        csf = torch.empty(E * per_c, dtype=torch.uint8, device=DEV)
        for e in range(E):
            qq, ri, qt, ci = ops.quant_iso32(w[e])
            ops.quant_iso32(w[e], out=(q[e], rsf[e * per_r:(e + 1) * per_r], csf[e * per_c:(e + 1) * per_c]))
            assert torch.equal(q[e], qq) and torch.equal(qt, qq.t().contiguous())
            assert torch.equal(rsf[e * per_r:(e + 1) * per_r], ri) and torch.equal(csf[e * per_c:(e + 1) * per_c], ci)
        got = ops.gemm_varlen_m_bt(a_q, a_sf, q, csf, efo)
        ref = ops.gemm_varlen_m(a_q, a_sf, ops.transpose_u8(q), csf, efo)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        assert torch.equal(got, ref)
        # dequantised fp32 product
        aq, asc = Q.row_quant(a.float().cpu())
        ad = Q.dequant_rows(aq, asc)
        want = torch.zeros(rows, N)
        for e in range(E):
            wq, ws = Q.iso32_quant(w[e].float().cpu())
            wd = Q.e4m3_bytes_to_f32(wq) * Q.dequant_scale_from_e8m0(ws).repeat_interleave(32, 0).repeat_interleave(32, 1)
            lo, hi = int(efo[e]), int(efo[e + 1])
            want[lo:hi] = ad[lo:hi] @ wd
        gd, wd64 = got.double().cpu(), want.double()
        cos = float((gd * wd64).sum() / (gd.norm() * wd64.norm()))
        assert cos > 0.99999, cos


def test_payload_only_scatter_and_caller_owned_gated_outputs(ops):
    """`scatter_rows_fp8(with_scales=False)` writes the same payload bytes; `gemm_gated(out=...)` fills the
    caller's buffers with the same bytes and rejects buffers of the wrong size."""
    g = torch.Generator().manual_seed(78)
    T, H, N2, E, K = 256, 256, 512, 4, 2
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    probs = torch.rand(T, K, generator=g).to(DEV)
    md = ops.topk_metadata(idx, probs, E)
    TKp = md["TKp_alloc"]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    q, raw, _ = ops.quant_rows(x, raw=True)
    full, isa = ops.scatter_rows_fp8(q, raw, md["naept"], md["s_reverse_scatter_idx"], md["s_scatter_idx"], TKp,
                                     md["efo"][-1:])
    only, none = ops.scatter_rows_fp8(q, raw, md["naept"], md["s_reverse_scatter_idx"], md["s_scatter_idx"], TKp,
                                      md["efo"][-1:], with_scales=False)
    n = int(md["efo"][-1])
    assert none is None and torch.equal(full[:n], only[:n])
    w = (torch.randn(E, N2, H, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    wq, _, wsf = ops.quant_rows(w.view(E * N2, H), raw=False, isa=True)
    wq = wq.view(E, N2, H)
    ref = ops.gemm_gated(full, None, isa, wq, wsf, md["efo"], TKp)
    bufs = (torch.zeros(TKp, N2, dtype=torch.float8_e4m3fn, device=DEV),
            torch.zeros(TKp, N2 // 32, dtype=torch.uint8, device=DEV),
            torch.zeros(TKp, N2 // 2, dtype=torch.float8_e4m3fn, device=DEV),
            torch.zeros(TKp // 128, N2 // 256, 512, dtype=torch.uint8, device=DEV))
    got = ops.gemm_gated(full, None, isa, wq, wsf, md["efo"], TKp, out=bufs)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert got[0].data_ptr() == bufs[0].data_ptr() and got[3].data_ptr() == bufs[3].data_ptr()
    nb = n // 128 * (N2 // 2 // 128) * 512
    assert torch.equal(ref[0][:n], got[0][:n]) and torch.equal(ref[1][:n], got[1][:n])
    assert torch.equal(ref[2][:n], got[2][:n]) and torch.equal(ref[3][:nb], got[3][:nb])
    with pytest.raises(ValueError):
        ops.gemm_gated(full, None, isa, wq, wsf, md["efo"], TKp, out=(bufs[0], bufs[1], bufs[2], bufs[3][:-1]))


def test_two_weight_gradients_in_one_launch_give_the_bits_of_two_launches(ops):
    """`gemm_wgrad_pair`: dw1 and dw2 share a launch of the 256 x 384 kernel; every output element has the same single
    writer and the same K order as in its own launch, so the results are bit-identical, overwriting or accumulating,
    with an empty expert and with the A operands stored either way."""
    g = torch.Generator().manual_seed(303)
    E, N, M1, M2 = 4, 768, 512, 256
    seg = (256, 0, 384, 128)
    TKp = sum(seg)
    efo = torch.tensor([0] + list(torch.tensor(seg).cumsum(0)), dtype=torch.int32, device=DEV)
    rnd = lambda *s: torch.randint(0, 256, s, generator=g, dtype=torch.uint8).to(DEV)
    finite = lambda t: torch.where((t & 0x7F) == 0x7F, t & 0xFE, t)          # no e4m3 NaN patterns
    sfr = lambda n: torch.randint(118, 130, (n,), generator=g, dtype=torch.uint8).to(DEV)
    b1, b2 = finite(rnd(N, TKp)), finite(rnd(N, TKp))
    b1_sf, b2_sf = sfr(ops.isa_bytes(N, TKp)), sfr(ops.isa_bytes(N, TKp))
    for a_rows_tk in (True, False):
        a1 = finite(rnd(TKp, M1) if a_rows_tk else rnd(M1, TKp))
        a2 = finite(rnd(TKp, M2) if a_rows_tk else rnd(M2, TKp))
        a1_sf, a2_sf = sfr(ops.isa_bytes(M1, TKp)), sfr(ops.isa_bytes(M2, TKp))
        for accumulate in (False, True):
            base1 = torch.randn(E, M1, N, generator=g).to(DEV)
            base2 = torch.randn(E, M2, N, generator=g).to(DEV)
            r1, r2 = base1.clone(), base2.clone()
            ops.gemm_wgrad_mn(a1, a1_sf, b1, b1_sf, efo, r1, accumulate, a_rows_tk, False)
            ops.gemm_wgrad_mn(a2, a2_sf, b2, b2_sf, efo, r2, accumulate, a_rows_tk, False)
            o1, o2 = base1.clone(), base2.clone()
            ops.gemm_wgrad_pair(a1, a1_sf, b1, b1_sf, o1, a2, a2_sf, b2, b2_sf, o2, efo, accumulate, a_rows_tk)
            torch.cuda.synchronize()
            ops.check_status(DEV)
            assert torch.equal(o1, r1) and torch.equal(o2, r2), (a_rows_tk, accumulate)
            if not accumulate:
                assert bool((o1[1] == 0).all()) and bool((o2[1] == 0).all())      # the empty expert
