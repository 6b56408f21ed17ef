"""The oracle's MoE restatements against each other and against autograd (CPU only).

Config C1 of the benchmark set: T=256, H=256, I=128, E=8, K=2, seed 0."""
import torch

from oracle import moe as OM
from oracle import quant as Q
from oracle import routing as R


def _c1(seed=0, T=256, H=256, I=128, E=8, K=2):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    scores, idx = OM.router_topk_softmax(logits, K)
    return x, dy, w1, w2, logits, scores, idx, E, K


def stats(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return float((a * b).sum() / (a.norm() * b.norm())), float((a - b).norm() / b.norm())


def test_fp32_gold_matches_autograd_of_the_reference_torch_path():
    x, dy, w1, w2, logits, scores, idx, E, K = _c1()
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    # autograd of the reference's pure-PyTorch expert path (sonicmoe/moe.py:739-758), fp32
    xf = x.float().requires_grad_(True)
    w1f, w2f = w1.float().requires_grad_(True), w2.float().requires_grad_(True)
    sc = scores.clone().requires_grad_(True)
    sel = idx.flatten().long()
    order = sel.sort(stable=True).indices
    freq = sel.bincount(minlength=E).tolist()
    fan_in = order // K
    h = xf[fan_in].split(freq)
    h = [torch.nn.functional.linear(h[e], w1f[e]) for e in range(E)]
    h = [t[..., 1::2] * torch.nn.functional.silu(t[..., ::2]) for t in h]
    h = torch.cat([torch.nn.functional.linear(h[e], w2f[e]) for e in range(E)])
    h = h * sc.flatten()[order].unsqueeze(-1)
    out = torch.zeros_like(xf).index_add(0, fan_in, h)
    out.backward(dy.float())
    torch.testing.assert_close(gold["o"], out.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gold["dx"], xf.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gold["dw1"], w1f.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gold["dw2"], w2f.grad, rtol=1e-4, atol=1e-5)
    ds = torch.zeros(sc.numel())
    ds[md["score_src_idx"].long()] = gold["ds"]
    torch.testing.assert_close(ds.view_as(sc), sc.grad, rtol=1e-4, atol=1e-5)


def test_fp8_emulated_dataflow_is_within_the_published_tolerance_of_the_gold():
    x, dy, w1, w2, logits, scores, idx, E, K = _c1()
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    for k_emu, k_gold in (("o", "o"), ("dx", "dx"), ("dw1", "dw1"), ("dw2_IH", "dw2_IH"), ("ds", "ds")):
        cos, rr = stats(emu[k_emu], gold[k_gold])
        assert cos > 0.996 and rr < 0.09, (k_emu, cos, rr)
    # pad rows carry exactly zero gradient (tests/ops/test_pad_gradient_integrity.py)
    s = md["topk_scores"][md["s_scatter_idx"].long()]
    assert (emu["dz"][s == 0] == 0).all() and (emu["y1s"][s == 0] == 0).all()
    # z is quantised with the 1e-4 amax floor, y1 without
    assert emu["z_scales"].min() >= 105


def test_router_backward_matches_autograd():
    x, dy, w1, w2, logits, scores, idx, E, K = _c1()
    lg = logits.clone().requires_grad_(True)
    vals, ix = lg.topk(K, dim=-1)
    s = torch.softmax(vals, -1)
    g = torch.randn(s.shape, generator=torch.Generator().manual_seed(3))
    s.backward(g)
    torch.testing.assert_close(OM.router_backward(scores, idx, g, E), lg.grad, rtol=1e-5, atol=1e-6)


def test_torch_baseline_module_matches_gold_on_its_own_routing():
    b = OM.TorchMoEBaseline(8, 2, 64, 32, seed=1, dtype=torch.float32)
    x = torch.randn(50, 64, generator=torch.Generator().manual_seed(2))
    out, logits = b(x)
    scores, idx = OM.router_topk_softmax(logits.detach(), 2)
    md = R.topk_metadata(idx, scores, 8, 1)
    gold = OM.moe_fp32(x, b.w1.detach(), b.w2.detach(), md)
    torch.testing.assert_close(out.detach(), gold["o"], rtol=1e-4, atol=1e-5)
