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


def _worker(rank, world, port, q, peer, starve):
    try:
        import datetime
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                                timeout=datetime.timedelta(seconds=120))
        import sonicmoe.ep as ep_mod
        ep_mod.USE_PEER_COMBINE = peer          # return exchanges over mapped peer memory vs NCCL all-to-all
        res = ep_mod.parity_against_single_gpu(dist.group.WORLD, dev, starve_last_rank=starve)
        q.put((rank, res))
        dist.barrier()
        dist.destroy_process_group()
    except Exception:                           # the parent fails fast instead of waiting for a result that never comes
        q.put((rank, traceback.format_exc()))
        raise


def _launch(world, peer, starve):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, peer, starve)) for r in range(world)]
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


@pytest.mark.parametrize("peer", [False, True])
def test_ep_two_gpus_matches_single_gpu_layer(peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from sonicmoe.ep import PARITY_LIMITS
    for rank, res in _launch(2, peer, False).items():
        assert res.pop("used_peer") == peer, "the requested return-exchange path was not the one that ran"
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
    results = _launch(2, False, True)
    assert results[1]["rows_received"] == 0 and results[0]["rows_received"] > 0
    for rank, res in results.items():
        res.pop("used_peer"), res.pop("rows_received")
        for name, (cos, rr) in res.items():
            cmin, rmax = PARITY_LIMITS[name]
            assert cos > cmin and rr < rmax, (rank, name, cos, rr)
