"""The expert-parallel data movers on ONE GPU: the ranks of a group are emulated as separate buffers of the same
device (the kernels wait on nothing, so each "rank's" launch simply runs after the buffers are filled), and every
result is compared bit for bit with a host-side restatement of the exchange it replaces: rows ordered by source rank
and, inside a source, by that source's send order (what an all-to-all delivers)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from sonicmoe import ops as _ops
    return _ops


def _align(n):
    return (n + 255) // 256 * 256


class _Rank:
    """What one rank leaves in its mapped buffer (same byte layout on every rank) plus host copies for the check."""

    def __init__(self, ops, r, world, T, t_cap, H, K, E, seed, starve=None):
        g = torch.Generator().manual_seed(seed + r)
        self.T = T
        logits = torch.randn(T, E, generator=g)
        if starve is not None:                                    # nobody routes to the experts of rank `starve`
            El = E // world
            logits[:, starve * El:(starve + 1) * El] = float("-inf")
        self.idx = logits.topk(K, dim=-1).indices.to(torch.int32)
        self.probs = torch.rand(T, K, generator=g)
        self.x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        cap = t_cap * min(K, world)
        idx_d = self.idx.to(DEV)
        dest_u, _ = ops.ep_plan_dest(idx_d, E, world)
        md = ops.topk_metadata(dest_u, dest_u.view(torch.float32), world, alignment=1, TK_alloc=T * min(K, world),
                               TKp_alloc=T * min(K, world) + world)
        n_cap = T * min(K, world)
        self.send_tok = md["x_gather_idx"][:n_cap]
        self.send_idx, self.send_rank = ops.ep_plan_send_idx(idx_d, self.send_tok, md["efo"], n_cap, E, world)
        self.counts, self.seg = md["counts"], md["efo"]
        self.copy_pos, self.copy_off = md["s_reverse_scatter_idx"][:n_cap], md["naept"]
        q, raw, _ = ops.quant_rows(self.x.to(DEV), raw=True)
        self.q, self.raw = q, raw
        # byte layout: q | raw | tok | idx | probs | counts | seg
        at, self.off = 0, {}
        for name, nbytes in (("q", t_cap * H), ("raw", t_cap * (H // 32)), ("tok", cap * 4), ("idx", cap * K * 4),
                             ("probs", t_cap * K * 4), ("counts", 256), ("seg", 256)):
            self.off[name] = at
            at += _align(nbytes)
        buf = torch.zeros(at, dtype=torch.uint8, device=DEV)
        o = self.off
        buf[o["q"]:o["q"] + T * H] = q.view(-1)
        buf[o["raw"]:o["raw"] + T * (H // 32)] = raw.view(-1)
        buf[o["tok"]:o["tok"] + n_cap * 4] = self.send_tok.contiguous().view(torch.uint8)
        buf[o["idx"]:o["idx"] + n_cap * K * 4] = self.send_idx.contiguous().view(torch.uint8).view(-1)
        buf[o["probs"]:o["probs"] + T * K * 4] = self.probs.to(DEV).contiguous().view(torch.uint8).view(-1)
        buf[o["counts"]:o["counts"] + world * 4] = self.counts[:world].contiguous().view(torch.uint8)
        buf[o["seg"]:o["seg"] + (world + 1) * 4] = self.seg[:world + 1].contiguous().view(torch.uint8)
        self.buf = buf
        self.layout = (o["q"], o["raw"], o["tok"], o["idx"], o["probs"])


@pytest.mark.parametrize("world,starve", [(4, None), (2, None), (4, 3)])
def test_dispatch_and_combine_pulls_against_the_exchange_they_replace(ops, world, starve):
    H, K, E = 512, 4, 16
    tokens = [384, 257, 512, 130][:world]                         # ranks hold different numbers of tokens
    t_cap = max(tokens)
    ranks = [_Rank(ops, r, world, tokens[r], t_cap, H, K, E, 500, starve) for r in range(world)]
    ptrs = [rk.buf.data_ptr() for rk in ranks]
    layout = ranks[0].layout
    assert all(rk.layout == layout for rk in ranks)
    counts = [rk.counts[:world].cpu().tolist() for rk in ranks]   # counts[s][r]: rows s sends to r
    segs = [rk.seg[:world + 1].cpu().tolist() for rk in ranks]
    n_bound = world * t_cap
    received = []
    for me in range(world):
        # what an all-to-all would deliver to `me`
        exp_q, exp_raw, exp_idx, exp_p = [], [], [], []
        for s, rk in enumerate(ranks):
            lo, n = segs[s][me], counts[s][me]
            tok = rk.send_tok[lo:lo + n].long()
            exp_q.append(rk.q[tok]); exp_raw.append(rk.raw[tok])
            exp_idx.append(rk.send_idx[lo:lo + n]); exp_p.append(rk.probs.to(DEV)[tok])
        exp_q, exp_raw, exp_idx, exp_p = (torch.cat(v) for v in (exp_q, exp_raw, exp_idx, exp_p))
        n_recv = exp_q.shape[0]
        received.append(n_recv)
        recv_counts = [counts[s][me] for s in range(world)]
        src_off = [segs[s][me] for s in range(world)]
        q, raw, idx, p = ops.ep_dispatch_pull(ptrs, recv_counts, src_off, me, layout, H, K, DEV)
        assert q.shape[0] == n_recv
        assert torch.equal(q, exp_q) and torch.equal(raw, exp_raw) and torch.equal(idx, exp_idx) and torch.equal(p, exp_p)
        q2, raw2, none_i, none_p = ops.ep_dispatch_pull(ptrs, recv_counts, src_off, me, layout, H, K, DEV, with_meta=False)
        assert none_i is None and none_p is None and torch.equal(q2, exp_q) and torch.equal(raw2, exp_raw)
        # the same without host-side counts: tables from the counts every rank left in its buffer
        tab = ops.ep_tables(ptrs, me, ranks[0].off["counts"], ranks[0].off["seg"], DEV)
        qd, rawd, idxd, pd = ops.ep_dispatch_pull_dev(ptrs, tab, me, layout, H, K, n_bound, DEV)
        assert qd.shape[0] == n_bound
        assert torch.equal(qd[:n_recv], exp_q) and torch.equal(rawd[:n_recv], exp_raw)
        assert torch.equal(idxd[:n_recv], exp_idx) and torch.equal(pd[:n_recv], exp_p)
        assert bool((idxd[n_recv:] == -1).all()) and bool((pd[n_recv:] == 0).all())      # rows that did not arrive
    if starve is not None:
        assert received[starve] == 0 and min(r for i, r in enumerate(received) if i != starve) > 0

    # ---- return: every rank holds one bf16 row per received row; the source adds its tokens' copies, ascending rank
    g = torch.Generator().manual_seed(77)
    partial = [torch.randn(max(received[r], 1), H, generator=g).to(torch.bfloat16).to(DEV) for r in range(world)]
    pptrs = [t.data_ptr() for t in partial]
    for me, rk in enumerate(ranks):
        first_row = [sum(counts[s][r] for s in range(me)) for r in range(world)]
        send_off = segs[me][:world]
        n_send = segs[me][world]
        # host restatement: outgoing row i went to send_rank[i] and sits there at first_row + (i - send_off)
        sr = rk.send_rank[:n_send].cpu().tolist()
        back = torch.zeros(max(n_send, 1), H, dtype=torch.float32)
        for i in range(n_send):
            r = sr[i]
            back[i] = partial[r][first_row[r] + i - send_off[r]].float().cpu()
        pos, off = rk.copy_pos[:n_send].cpu().long(), rk.copy_off.cpu().long()
        want = torch.zeros(rk.T, H, dtype=torch.float32)
        for t in range(rk.T):
            for j in range(int(off[t]), int(off[t + 1])):          # ascending destination rank, fp32 accumulate
                want[t] += back[pos[j]]
        want = want.to(torch.bfloat16)
        got = ops.ep_combine_pull(pptrs, first_row, send_off, rk.copy_pos[:n_send].contiguous(), rk.copy_off,
                                  rk.send_rank[:n_send].contiguous(), rk.T, H, DEV)
        assert torch.equal(got.cpu(), want)
        tab = ops.ep_tables(ptrs, me, ranks[0].off["counts"], ranks[0].off["seg"], DEV)
        got_dev = ops.ep_combine_pull_dev(pptrs, tab, rk.copy_pos, rk.copy_off, rk.send_rank, rk.T, H, DEV)
        assert torch.equal(got_dev, got)
    torch.cuda.synchronize()


def test_pull_entry_points_refuse_what_they_cannot_run(ops):
    from sonicmoe._lib import lib
    import ctypes
    one = (ctypes.c_void_p * 1)(0)
    cnt = (ctypes.c_int32 * 1)(0)
    assert lib.smoe_ep_dispatch_pull(one, cnt, cnt, 17, 0, 0, 0, 0, 0, 0, 512, 4, None, None, None, None, None) != 0
    assert lib.smoe_ep_dispatch_pull(one, cnt, cnt, 1, 0, 0, 0, 0, 0, 0, 100, 4, None, None, None, None, None) != 0
    assert lib.smoe_ep_dispatch_pull(one, cnt, cnt, 1, 0, 8, 0, 0, 0, 0, 512, 4, None, None, None, None, None) != 0
    # nothing to receive: fine without any buffer
    assert lib.smoe_ep_dispatch_pull(one, cnt, cnt, 1, 0, 0, 0, 0, 0, 0, 512, 4, None, None, None, None, None) == 0
    assert lib.smoe_ep_tables(one, 1, 0, 0, 0, None, None) != 0
    assert lib.smoe_ep_tables_bytes() >= 4 * (17 + 16 * 3 + 1)


def test_plans_with_counts_in_flight_resolve_to_their_own_counts(ops):
    """A plan built without a read-back keeps its counts in a pinned host buffer of its own until something asks for
    them.  Twelve such plans are built back to back (more than a pipeline's forwards in flight would be) and resolved
    in reverse order: each must give exactly what a plan built with an immediate read-back gives.  One-rank group:
    the plan's kernels, its all-gather and the side-stream copy run as on many ranks."""
    import socket
    import torch.distributed as dist
    from sonicmoe import ep

    if dist.is_initialized():
        pytest.skip("a process group exists already")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    torch.cuda.set_device(0)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                            device_id=torch.device("cuda", 0))
    try:
        E, K = 8, 4
        g = torch.Generator().manual_seed(31)
        problems = []
        for i in range(12):
            T = 64 + 8 * i
            idx = torch.randn(T, E, generator=g).topk(K, dim=-1).indices.to(torch.int32)
            idx[torch.rand(T, K, generator=g) < 0.2] = -1          # masked slots
            idx[i:T:7] = -1                                        # tokens that go nowhere
            problems.append(idx.to(DEV))
        in_flight = [ep.DispatchPlan(idx, E, dist.group.WORLD, deferred=True) for idx in problems]
        assert all(p.deferred and p._pending is not None for p in in_flight)
        assert len({p._pending[0].data_ptr() for p in in_flight}) == len(in_flight)
        for idx, p in reversed(list(zip(problems, in_flight))):
            now = ep.DispatchPlan(idx, E, dist.group.WORLD, deferred=False)
            for name in ("send_counts", "recv_counts", "tokens_per_local_expert", "n_send", "n_recv", "tokens_all",
                         "first_row_at", "src_seg_off", "send_off", "max_recv_rows"):
                assert getattr(p, name) == getattr(now, name), name
            assert p._pending is None
            assert 0 < p.n_send < idx.shape[0]
            for name in ("send_tok", "send_idx", "send_rank", "copy_pos", "copy_off"):
                assert torch.equal(getattr(p, name), getattr(now, name)), name
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()
