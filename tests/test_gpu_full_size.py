"""The reference-shape layer (T=8192, H=3072, I=1536, E=8, K=8, seed 0) at FULL size on the GPU.

The CPU oracle cannot run the whole layer at this size in seconds, so parity is checked through properties that do
not depend on the size:

* routing metadata: bit-exact against the (vectorised) CPU restatement at full size;
* forward output of a token depends on that token alone (row-wise quantizers, per-row GEMMs): a seeded sample of
  tokens is pushed through the FP8-emulating oracle and the fp32 gold as a tiny layer of its own and must meet the
  same two gates as the small configs;
* determinism: a repeated step is bit-identical, including the fp32 main_grad increments;
* power-of-two homogeneity of the backward: every quantizer uses power-of-two scales, so doubling dy must double dx,
  dscores and the main_grad increments exactly (a checksum over the whole backward dataflow);
* pad rows and the over-allocated tail never leak: gradients of the scores of real slots are finite everywhere.
"""
import pytest
import torch

from oracle import moe as OM
from oracle import routing as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
T, H, I, E, K, SEED = 8192, 3072, 1536, 8, 8, 0


def stats(got, ref):
    got, ref = got.detach().float().cpu().flatten(), ref.detach().float().cpu().flatten()
    cos = float((got * ref).sum() / (got.norm() * ref.norm()).clamp(min=1e-30))
    rr = float((got - ref).norm() / ref.norm().clamp(min=1e-30))
    return cos, rr


@pytest.fixture(scope="module")
def layer():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sonicmoe
    g = torch.Generator().manual_seed(SEED)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    scores, idx = OM.router_topk_softmax(logits, K)
    w1d, w2d = torch.nn.Parameter(w1.to(DEV)), torch.nn.Parameter(w2.to(DEV))
    w1d.main_grad = torch.zeros(E, 2 * I, H, dtype=torch.float32, device=DEV)
    w2d.main_grad = torch.zeros(E, I, H, dtype=torch.float32, device=DEV)
    xd, dyd, idxd = x.to(DEV), dy.to(DEV), idx.to(torch.int32).to(DEV)

    def step(dy_scale=1.0):
        xg = xd.detach().requires_grad_(True)
        sg = scores.to(DEV).requires_grad_(True)
        w1d.main_grad.zero_()          # increments are compared exactly: start every step from zero
        w2d.main_grad.zero_()
        out = sonicmoe.run_sonic_moe(xg, idxd, sg, K, E, w1d, w2d, fp8=True)
        out.backward(dyd * dy_scale)
        torch.cuda.synchronize()
        sonicmoe.ops.check_status(DEV)
        return dict(out=out.detach(), dx=xg.grad, ds=sg.grad, dw1=w1d.main_grad.clone(), dw2=w2d.main_grad.clone())

    return dict(sm=sonicmoe, x=x, dy=dy, w1=w1, w2=w2, idx=idx, scores=scores, step=step, first=step())


def test_routing_metadata_full_size_bit_exact(layer):
    ops = layer["sm"].ops
    idx, scores = layer["idx"].to(torch.int32), layer["scores"].float()
    md = ops.topk_metadata(idx.to(DEV), scores.to(DEV), E, 128)
    ref = R.topk_metadata(idx, scores, E, 128, TK_alloc=md["TK_alloc"], TKp_alloc=md["TKp_alloc"])
    for key in ("efo", "x_gather_idx", "s_scatter_idx", "s_reverse_scatter_idx", "naept", "topk_scores",
                "score_src_idx"):
        assert torch.equal(md[key].cpu(), ref[key]), key
    assert int(md["efo"][-1]) % 128 == 0 and bool((md["efo"][1:] >= md["efo"][:-1]).all())
    tk = T * K
    # inverse-permutation property: position -> slot -> position
    rev = md["s_reverse_scatter_idx"][:tk].long()
    assert torch.equal(torch.sort(rev).values, torch.sort(torch.unique(rev)).values)      # no position used twice


def test_sampled_tokens_forward_matches_oracles(layer):
    """out[t] depends on token t only: a sample of tokens, run through the oracles as a 48-token layer, must agree."""
    g = torch.Generator().manual_seed(123)
    sample = torch.randperm(T, generator=g)[:48]
    x, idx, scores = layer["x"][sample], layer["idx"][sample].to(torch.int32), layer["scores"][sample].float()
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, layer["w1"], layer["w2"], md)["o"]
    emu = OM.moe_fp8_emulated(x, layer["w1"], layer["w2"], md)["o"]
    got = layer["first"]["out"].cpu()[sample]
    c_e, r_e = stats(got, emu)
    assert c_e >= 0.9995 and r_e <= 0.03, ("vs FP8-emulating oracle", c_e, r_e)
    c_g, r_g = stats(got, gold)
    e_c, e_r = stats(emu, gold)
    assert c_g >= min(0.997, e_c - 5e-4) and r_g <= max(0.076, 1.03 * e_r), ("vs fp32 gold", c_g, r_g, e_c, e_r)


def test_repeat_is_bit_exact(layer):
    a, b = layer["first"], layer["step"]()
    for k in ("out", "dx", "ds", "dw1", "dw2"):
        assert torch.equal(a[k], b[k]), k
    assert torch.isfinite(a["ds"]).all() and torch.isfinite(a["dx"].float()).all()
    assert a["dw1"].abs().sum() > 0 and a["dw2"].abs().sum() > 0


def test_backward_is_exactly_homogeneous_in_powers_of_two(layer):
    """Every quantizer scale is a power of two and every reduction is a sum: dy -> 2 dy doubles the whole backward
    (dx in bf16, dscores and the main_grad increments in fp32) bit for bit."""
    a, b = layer["first"], layer["step"](2.0)
    assert torch.equal(b["out"], a["out"])
    assert torch.equal(b["dx"].float(), a["dx"].float() * 2)
    assert torch.equal(b["ds"], a["ds"] * 2)
    assert torch.equal(b["dw1"], a["dw1"] * 2) and torch.equal(b["dw2"], a["dw2"] * 2)
