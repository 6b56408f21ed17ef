"""Expert-parallel step on 2 GPUs (NCCL all-to-all, FP8 dispatch payload) against the single-GPU layer
run on the same tokens with all experts local."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu
T, H, I, E, K = 1024, 512, 256, 16, 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _inputs(rank):
    g = torch.Generator().manual_seed(200 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    vals, idx = logits.topk(K, dim=-1)
    scores = torch.softmax(vals, -1)
    gw = torch.Generator().manual_seed(5)
    w1 = (torch.randn(E, 2 * I, H, generator=gw) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=gw) * 0.02).to(torch.bfloat16)
    return x, dy, scores, idx.to(torch.int32), w1, w2


def _worker(rank, world, port, q, peer):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import sonicmoe
    import sonicmoe.ep as ep_mod
    from sonicmoe.ep import ExpertParallelMoE
    ep_mod.USE_PEER_COMBINE = peer          # return exchanges over mapped peer memory vs NCCL all-to-all
    x, dy, scores, idx, w1, w2 = _inputs(rank)
    El = E // world
    xd = x.to(dev).requires_grad_(True)
    sd = scores.to(dev).requires_grad_(True)
    w1l = w1[rank * El:(rank + 1) * El].contiguous().to(dev).requires_grad_(True)
    w2l = w2[rank * El:(rank + 1) * El].contiguous().to(dev).requires_grad_(True)
    ep = ExpertParallelMoE(E, K, dist.group.WORLD)
    out = ep(xd, idx.to(dev), sd, w1l, w2l)
    out.backward(dy.to(dev))
    torch.cuda.synchronize()
    sonicmoe.ops.check_status(dev)
    used_peer = ep._arena is not None
    # every rank's tokens through the single-GPU layer with all experts local; weight gradients of the local
    # expert slice summed over both ranks' tokens
    dw1_ref = torch.zeros(El, 2 * I, H, device=dev)
    dw2_ref = torch.zeros(El, H, I, device=dev)
    mine = None
    for r in range(world):
        xr, dyr, sr, ir, _, _ = _inputs(r)
        xa = xr.to(dev).requires_grad_(True)
        sa = sr.to(dev).requires_grad_(True)
        w1a, w2a = w1.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True)
        o = sonicmoe.run_sonic_moe(xa, ir.to(dev), sa, K, E, w1a, w2a, fp8=True)
        o.backward(dyr.to(dev))
        dw1_ref += w1a.grad[rank * El:(rank + 1) * El].float()
        dw2_ref += w2a.grad[rank * El:(rank + 1) * El].float()
        if r == rank:
            mine = (o.detach(), xa.grad, sa.grad)
    torch.cuda.synchronize()

    def st(a, b):
        a, b = a.float().flatten(), b.float().flatten()
        return float((a * b).sum() / (a.norm() * b.norm())), float((a - b).norm() / b.norm())
    res = dict(out=st(out, mine[0]), dx=st(xd.grad, mine[1]), ds=st(sd.grad, mine[2]), dw1=st(w1l.grad, dw1_ref),
               dw2=st(w2l.grad, dw2_ref))
    res["used_peer"] = used_peer
    q.put((rank, res))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("peer", [False, True])
def test_ep_two_gpus_matches_single_gpu_layer(peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, peer)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, res in results.items():
        assert res.pop("used_peer") == peer, "the requested return-exchange path was not the one that ran"
        for name, (cos, rr) in res.items():
            # same quantisation points; differences: bf16 rounding of the per-rank partial sums (out, dx) and
            # the column-wise re-quantisation of the FP8 payload for the weight gradients
            lim = 0.04 if name in ("dw1", "dw2") else 0.01
            assert cos > 0.999 and rr < lim, (rank, name, cos, rr)
