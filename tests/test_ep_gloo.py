"""Expert-parallel dispatch / combine on CPU: two gloo ranks, bf16 payload, an fp32 stand-in for the
per-rank expert compute.  Checks the plan, the exchanges and their backward against a single-process
oracle of the whole problem, and the host-side failure handling (a rank with inconsistent sizes)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as OM
from oracle import routing as R

T, H, I, E, K = 96, 64, 32, 8, 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(rank, world):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g)
    dy = torch.randn(T, H, generator=g)
    logits = torch.randn(T, E, generator=g)
    scores, idx = OM.router_topk_softmax(logits, K)
    gw = torch.Generator().manual_seed(7)
    w1 = torch.randn(E, 2 * I, H, generator=gw) * 0.1
    w2 = torch.randn(E, H, I, generator=gw) * 0.1
    return x, dy, scores, idx, w1, w2


def _expert_fn_fp32(rows, local_idx, probs, w1, w2, fp8_scale, handle):
    """Differentiable fp32 stand-in of run_sonic_moe on (rows, masked local indices, probs)."""
    El = w1.shape[0]
    out = torch.zeros(rows.shape[0], rows.shape[1])
    for k in range(local_idx.shape[1]):
        for e in range(El):
            sel = (local_idx[:, k] == e).nonzero().flatten()
            if sel.numel():
                z = rows[sel] @ w1[e].T
                y = (z[:, 0::2] * torch.sigmoid(z[:, 0::2])) * z[:, 1::2]
                out = out.index_add(0, sel, probs[sel, k:k + 1] * (y @ w2[e].T))
    return out


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sonicmoe.ep import DispatchPlan, ExpertParallelMoE
    x, dy, scores, idx, w1, w2 = _inputs(rank, world)
    El = E // world
    x = x.requires_grad_(True)
    scores = scores.requires_grad_(True)
    w1l = w1[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    w2l = w2[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    ep = ExpertParallelMoE(E, K, dist.group.WORLD, payload="bf16", expert_fn=_expert_fn_fp32)
    out = ep(x, idx, scores, w1l, w2l)
    out.backward(dy)
    plan = DispatchPlan(idx, E, dist.group.WORLD)
    res = dict(out=out.detach(), dx=x.grad, ds=scores.grad, dw1=w1l.grad, dw2=w2l.grad,
               n_send=plan.n_send, n_recv=plan.n_recv, send_counts=plan.send_counts,
               copies=(plan.copy_off[1:] - plan.copy_off[:-1]).clone(),
               per_expert=list(plan.tokens_per_local_expert), first_row_at=list(plan.first_row_at),
               recv_counts=list(plan.recv_counts), send_off=list(plan.send_off), max_recv=plan.max_recv_rows)
    # host-side failure: an exchange whose split sizes disagree with the buffer is refused before any data moves
    try:
        plan.send_counts = [c + 1 for c in plan.send_counts]
        plan.a2a(torch.zeros(plan.n_send, 4))
        res["bad_split_raises"] = False
    except Exception:
        res["bad_split_raises"] = True
    out_q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


def _launch(world, attempts=2):
    """Run the ranks as spawned processes; a rendezvous that fails (the probed port was taken in between, a slow
    first import) is retried once on a fresh port.  Numerical mismatches are not retried: they are checked by the
    caller on the returned tensors."""
    ctx = mp.get_context("spawn")
    last = None
    for _ in range(attempts):
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
        for p in procs:
            p.start()
        try:
            results = dict(q.get(timeout=240) for _ in range(world))
            for p in procs:
                p.join(timeout=120)
            if all(p.exitcode == 0 for p in procs):
                return results
            last = RuntimeError(f"rank exit codes {[p.exitcode for p in procs]}")
        except Exception as exc:  # queue timeout: a rank died or never joined
            last = exc
        for p in procs:
            if p.is_alive():
                p.kill()
            p.join(timeout=30)
    raise last


def test_ep_two_ranks_matches_single_process_oracle():
    world = 2
    results = _launch(world)
    El = E // world
    dw1_tot = [torch.zeros(El, 2 * I, H) for _ in range(world)]
    dw2_tot = [torch.zeros(El, H, I) for _ in range(world)]
    for rank in range(world):
        x, dy, scores, idx, w1, w2 = _inputs(rank, world)
        md = R.topk_metadata(idx, scores, E, 1)
        gold = OM.moe_fp32(x, w1, w2, md, dy)
        r = results[rank]
        torch.testing.assert_close(r["out"], gold["o"], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(r["dx"], gold["dx"], rtol=1e-4, atol=1e-4)
        ds = torch.zeros(T * K)
        ds[md["score_src_idx"].long()] = gold["ds"]
        torch.testing.assert_close(r["ds"].flatten(), ds, rtol=1e-4, atol=1e-4)
        # plan: one copy of a token per destination rank
        dest = torch.div(idx, El, rounding_mode="floor")
        n_dest = torch.tensor([len(set(row.tolist())) for row in dest])
        assert torch.equal(r["copies"].long(), n_dest)
        # routed pairs per local expert, summed over all source ranks (sizes the expert-sorted buffers)
        all_idx = torch.cat([_inputs(rk, world)[3] for rk in range(world)])
        want = torch.bincount(all_idx.flatten(), minlength=E)[rank * El:(rank + 1) * El]
        assert r["per_expert"] == want.tolist()
        # the count matrix every rank holds: where this rank's rows start in each peer's receive order
        sent = [results[s]["send_counts"] for s in range(world)]
        assert r["recv_counts"] == [sent[s][rank] for s in range(world)]
        assert r["first_row_at"] == [sum(sent[s][d] for s in range(rank)) for d in range(world)]
        assert r["send_off"] == [sum(sent[rank][:d]) for d in range(world)]
        assert r["max_recv"] == max(sum(sent[s][d] for s in range(world)) for d in range(world))
        assert r["n_send"] == int(n_dest.sum()) and sum(r["send_counts"]) == r["n_send"]
        assert r["bad_split_raises"]
        # this rank's tokens contribute to every rank's expert gradients
        for o in range(world):
            dw1_tot[o] += gold["dw1"][o * El:(o + 1) * El]
            dw2_tot[o] += gold["dw2"][o * El:(o + 1) * El]
    for o in range(world):
        torch.testing.assert_close(results[o]["dw1"], dw1_tot[o], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(results[o]["dw2"], dw2_tot[o], rtol=1e-4, atol=1e-4)
    assert results[0]["n_recv"] == results[0]["send_counts"][0] + results[1]["send_counts"][0]


def test_deferred_counts_buffers_are_owned_per_plan(monkeypatch):
    """The host copy of a plan's counts lives in a pinned buffer the plan owns until it has read it: any number of
    plans may be in flight (a pipeline schedule runs many forwards before the first backward), each resolves to its
    own counts, and a buffer returns to the pool when its plan has read it or dies unread."""
    import gc
    from sonicmoe import ep

    monkeypatch.setattr(ep, "_alloc_pinned_i64", lambda shape: torch.empty(shape, dtype=torch.int64))
    monkeypatch.setattr(ep, "_PINNED_FREE", {})
    monkeypatch.setattr(ep.dist, "get_rank", lambda group=None: 0)
    monkeypatch.setattr(ep.DispatchPlan, "_finish_cuda", lambda self: None)

    class Arrived:
        def synchronize(self):
            pass

    world, El = 2, 2
    key = (0, (world, world + world * El + 1))

    def plan_in_flight(i):
        p = object.__new__(ep.DispatchPlan)
        p.El, p.world, p.group = El, world, None
        host = ep._pinned_take(key)
        # rows of the gathered matrix: [rows to rank 0, rows to rank 1, pairs per expert (4), tokens]
        host.copy_(torch.tensor([[i, i + 1, 1, 2, 3, 4, 100 + i], [i + 2, i + 3, 5, 6, 7, 8, 200 + i]]))
        p._pending = (host, Arrived(), key)
        return p

    plans = [plan_in_flight(i) for i in range(12)]
    assert len({p._pending[0].data_ptr() for p in plans}) == 12
    for i, p in reversed(list(enumerate(plans))):
        assert p.send_counts == [i, i + 1]
        assert p.recv_counts == [i, i + 2]
        assert p.tokens_per_local_expert == [1 + 5, 2 + 6]
        assert p.tokens_all == [100 + i, 200 + i]
        assert p.src_seg_off == [0, 0] and p.first_row_at == [0, 0]
        assert p._pending is None
    assert len(ep._PINNED_FREE[key]) == 12
    unread = plan_in_flight(99)
    assert len(ep._PINNED_FREE[key]) == 11
    del unread
    gc.collect()
    assert len(ep._PINNED_FREE[key]) == 12
    with pytest.raises(AttributeError):
        plans[0].no_such_field
