"""Expert-parallel step on 2 GPUs (NCCL all-to-all, FP8 dispatch payload) against the single-GPU layer
run on the same tokens with all experts local."""
import os
import queue
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q, peer, starve, dispatch="pull"):
    try:
        import datetime
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        import sonicmoe.ep as ep_mod
        # return exchanges over mapped peer memory ("1": both, "fwd": the forward's only) vs NCCL all-to-all ("0")
        ep_mod.USE_PEER_COMBINE, ep_mod.PEER_COMBINE_BACKWARD = peer in ("1", "fwd"), peer == "1"
        ep_mod.DISPATCH = "pull" if dispatch == "both" else dispatch   # FP8 rows fetched from the peers vs all-to-all
        res = ep_mod.parity_against_single_gpu(dist.group.WORLD, dev, starve_last_rank=starve)
        if dispatch == "both":
            res["modes_bit_identical"] = _same_bits_either_dispatch(ep_mod, dev, rank, world)
        q.put((rank, res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:                           # the parent fails fast instead of waiting for a result that never comes
        q.put((rank, traceback.format_exc()))
        raise


def _same_bits_either_dispatch(ep_mod, dev, rank, world):
    """The same expert-parallel step, twice each way and interleaved (forward A, forward B, backward A, backward
    B on one layer object): rows fetched from the peers' memory give the bits of the NCCL all-to-all path."""
    import torch.distributed as dist
    T, H, I, K, El = 768, 512, 256, 4, 4
    E = El * world
    g = torch.Generator().manual_seed(900 + rank)
    gw = torch.Generator().manual_seed(899)
    w1 = (torch.randn(E, 2 * I, H, generator=gw) * 0.02).to(torch.bfloat16)[rank * El:(rank + 1) * El].contiguous()
    w2 = (torch.randn(E, H, I, generator=gw) * 0.02).to(torch.bfloat16)[rank * El:(rank + 1) * El].contiguous()
    batches = []
    for _ in range(2):
        x = torch.randn(T, H, generator=g).to(torch.bfloat16)
        dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
        vals, idx = torch.randn(T, E, generator=g).topk(K, dim=-1)
        batches.append((x, dy, torch.softmax(vals, -1), idx.to(torch.int32)))

    def run(mode):
        ep_mod.DISPATCH = mode
        ep_mod.DX_RETURN = "copy" if mode == "pull" else "nccl"      # the all-NCCL data path against the default one
        layer = ep_mod.ExpertParallelMoE(E, K, dist.group.WORLD)
        w1d, w2d = w1.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True)
        live = []
        for x, dy, sc, idx in batches:          # both forwards before either backward
            xd, sd = x.to(dev).requires_grad_(True), sc.to(dev).requires_grad_(True)
            live.append((layer(xd, idx.to(dev), sd, w1d, w2d), xd, sd, dy))
        outs = []
        for out, xd, sd, dy in live:
            out.backward(dy.to(dev))
            outs += [out.detach(), xd.grad, sd.grad]
        torch.cuda.synchronize(dev)
        assert (layer._disp is not None) == (mode == "pull")
        # the first call sized the mapped buffers from its counts; the second ran without reading any back
        assert layer._plan.deferred == (mode == "pull")
        return outs + [w1d.grad, w2d.grad]

    a, b = run("nccl"), run("pull")
    return all(torch.equal(u, v) for u, v in zip(a, b))


def _launch(world, peer, starve, dispatch="pull"):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, peer, starve, dispatch)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            try:
                rank, res = q.get(timeout=300)
            except queue.Empty:
                pytest.fail("a rank produced no result within 300 s")
            if isinstance(res, str):
                pytest.fail(f"rank {rank} raised:\n{res}")
            results[rank] = res
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        # no rank may outlive the test: a survivor would sit in a collective with kernels in flight
        for p in procs:
            if p.is_alive():
                p.kill()
            p.join(timeout=30)
    return results


@pytest.mark.parametrize("peer", ["0", "fwd", "1"])
def test_ep_two_gpus_matches_single_gpu_layer(peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sonicmoe.ep import PARITY_LIMITS
    for rank, res in _launch(2, peer, False).items():
        assert res.pop("used_peer") == (peer != "0"), "the requested return-exchange path was not the one that ran"
        assert res.pop("used_pull_dispatch") is True
        # with both peer-memory paths on, the forward reads no counts back (they are looked at in the backward)
        assert res.pop("forward_without_readback") == (peer != "0")
        assert res.pop("dx_returned_by_copies") == (peer != "1")      # "1" pulls dx from the owners instead
        assert res.pop("rows_received") > 0
        for name, (cos, rr) in res.items():
            cmin, rmax = PARITY_LIMITS[name]
            assert cos > cmin and rr < rmax, (rank, name, cos, rr)


def test_ep_rank_that_receives_no_tokens():
    """Every token routes to rank 0's experts: rank 1 runs the whole step on zero rows (zero-row GEMM calls,
    empty exchanges) while rank 0 does all the work; both must finish and agree with the single-GPU layer,
    rank 1's weight gradients being exactly zero."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sonicmoe.ep import PARITY_LIMITS
    results = _launch(2, "fwd", True)
    assert results[1]["rows_received"] == 0 and results[0]["rows_received"] > 0
    for rank, res in results.items():
        res.pop("used_peer"), res.pop("rows_received"), res.pop("used_pull_dispatch")
        assert res.pop("dx_returned_by_copies") is True
        assert res.pop("forward_without_readback") is True
        for name, (cos, rr) in res.items():
            cmin, rmax = PARITY_LIMITS[name]
            assert cos > cmin and rr < rmax, (rank, name, cos, rr)


def test_ep_dispatch_through_nccl_and_both_dispatch_paths_give_the_same_bits():
    """SONIC_MOE_EP_DISPATCH=nccl (rows gathered and sent through all-to-alls) still matches the single-GPU layer, and
    the default (rows fetched by the destination from the sources' mapped memory) reproduces it bit for bit, also
    with two forwards of one layer in flight before their backwards."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sonicmoe.ep import PARITY_LIMITS
    for rank, res in _launch(2, "0", False, "nccl").items():
        assert res.pop("used_pull_dispatch") is False and res.pop("forward_without_readback") is False
        res.pop("used_peer"), res.pop("rows_received"), res.pop("dx_returned_by_copies")
        for name, (cos, rr) in res.items():
            cmin, rmax = PARITY_LIMITS[name]
            assert cos > cmin and rr < rmax, (rank, name, cos, rr)
    for rank, res in _launch(2, "fwd", False, "both").items():
        assert res["modes_bit_identical"] is True, rank
