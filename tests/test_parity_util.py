"""The two carve-out constructions of tests/parity_util.py, proven on the CPU oracles alone: the small layer's
results are bit-identical to the corresponding pieces of the full layer, for the fp32 gold and for the
FP8-emulating oracle (so every quantisation group of the full layer re-appears unchanged in the small one)."""
import pytest
import torch

from oracle import moe as OM
from oracle import routing as R
from parity_util import block_closure, ds_by_slot, oracles_on, single_expert


def _layer(T, H, I, E, K, seed, skew):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    if skew:
        p = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
        logits = logits + torch.log(p / p.sum())[torch.randperm(E, generator=g)]
    scores, idx = OM.router_topk_softmax(logits, K)
    return x, dy, w1, w2, idx.to(torch.int32), scores.float()


@pytest.mark.parametrize("T,H,I,E,K,skew", [(1024, 128, 64, 8, 8, False), (2048, 128, 64, 32, 4, True)])
def test_block_closure_reproduces_the_full_layer_bit_for_bit(T, H, I, E, K, skew):
    x, dy, w1, w2, idx, scores = _layer(T, H, I, E, K, 11, skew)
    md, gold, emu = oracles_on(x, dy, w1, w2, idx, scores, E)
    sample = torch.randperm(T, generator=torch.Generator().manual_seed(1))[:6].sort().values
    U, idx_m, sc_m, used, where = block_closure(idx, scores, md, sample, E)
    assert U.numel() < T
    md_m, gold_m, emu_m = oracles_on(x[U], dy[U], w1[used], w2[used], idx_m, sc_m, len(used))
    for full, mini in ((emu, emu_m), (gold, gold_m)):
        exact = full is emu                     # fp32 matmuls over different row counts may block differently
        for key in ("o", "dx"):
            a, b = full[key][sample].float(), mini[key][where].float()
            assert torch.equal(a, b) if exact else torch.allclose(a, b, rtol=1e-4, atol=1e-6), key
        a = ds_by_slot(full["ds"], md, T, K)[sample]
        b = ds_by_slot(mini["ds"], md_m, U.numel(), K)[where]
        assert torch.equal(a, b) if exact else torch.allclose(a, b, rtol=1e-4, atol=1e-6)


def test_single_expert_reproduces_its_weight_gradients_bit_for_bit():
    T, H, I, E, K = 1024, 128, 64, 16, 4
    x, dy, w1, w2, idx, scores = _layer(T, H, I, E, K, 12, True)
    md, gold, emu = oracles_on(x, dy, w1, w2, idx, scores, E)
    e = int(torch.bincount(idx.flatten().long(), minlength=E).argmax())
    tok, idx1, sc1 = single_expert(idx, scores, e)
    _, gold1, emu1 = oracles_on(x[tok], dy[tok], w1[e:e + 1], w2[e:e + 1], idx1, sc1, 1)
    assert torch.equal(emu["dw1"][e], emu1["dw1"][0]) and torch.equal(emu["dw2_IH"][e], emu1["dw2_IH"][0])
    assert torch.allclose(gold["dw1"][e], gold1["dw1"][0], rtol=1e-4, atol=1e-6)
