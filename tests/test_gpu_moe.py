"""End-to-end parity of the MoE layer (module and functional API) on the GPU against the CPU oracle.

Two gates per tensor (out, dx, drouter, dw1, dw2):

* against the FP8-emulating oracle (same quantisation points, GEMMs as dequantise -> fp32 matmul):
  cosine >= 0.9995 and RRMSE <= 3 % - the CUDA path reproduces the reference dataflow;
* against the fp32 gold: the tolerance the reference publishes for its FP8 path (README.md:321-334),
  cosine >= 0.997 and RRMSE <= 7.6 %.  That figure is a property of the FP8 dataflow AND the data: on some of
  the seeded N(0,1)/softmax inputs used here the bit-faithful CPU emulation of the reference dataflow itself sits
  at 7.7 % (dw2), so the bound applied is max(7.6 %, 1.03 x the emulation's own error) and
  min(0.997, the emulation's cosine - 5e-4): never looser than what the reference dataflow delivers on the
  same inputs."""
import pytest
import torch

from oracle import moe as OM
from oracle import quant as Q
from oracle import routing as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
COS_MIN, RRMSE_MAX = 0.997, 0.076


@pytest.fixture(scope="module")
def sm():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import sonicmoe
    return sonicmoe


def stats(got, ref):
    got, ref = got.detach().float().cpu().flatten(), ref.detach().float().cpu().flatten()
    cos = float((got * ref).sum() / (got.norm() * ref.norm()).clamp(min=1e-30))
    rr = float((got - ref).norm() / ref.norm().clamp(min=1e-30))
    return cos, rr


def check(name, got, ref, cos_min=COS_MIN, rr_max=RRMSE_MAX, emu=None):
    cos, rr = stats(got, ref)
    if emu is not None:
        ecos, err = stats(emu, ref)
        # summation order differs between the kernels and the emulation: allow 5e-4 / 3 % around its own error
        cos_min, rr_max = min(cos_min, ecos - 5e-4), max(rr_max, 1.03 * err)
        c2, r2 = stats(got, emu)
        assert c2 >= 0.9995 and r2 <= 0.03, f"{name} vs FP8-emulating oracle: cos {c2:.5f} rrmse {r2:.5f}"
    assert cos >= cos_min and rr <= rr_max, f"{name}: cos {cos:.5f} rrmse {rr:.5f} (need {cos_min:.5f} / {rr_max:.5f})"


def make_layer(T, H, I, E, K, seed, skew=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) * 0.02).to(torch.bfloat16)
    # router weight scaled so that logits are ~N(0,1)
    wr = (torch.randn(E, H, generator=g) / H ** 0.5).to(torch.bfloat16)
    if skew:
        p = torch.arange(1, E + 1, dtype=torch.float32) ** -1.2
        bias = torch.log(p / p.sum())[torch.randperm(E, generator=g)]
    else:
        bias = None
    return x, dy, w1, w2, wr, bias


def oracle_dense(x, dy, w1, w2, wr, K, logits):
    """fp32 gold of the whole layer: router + experts, explicit backward.  `logits` are the router logits as the
    module computes them (bf16 linear on the GPU): a CPU matmul rounds differently and would flip the top-k choice
    of tokens whose K-th and (K+1)-th logits nearly tie, which is a property of the test, not of the layer."""
    E = wr.shape[0]
    xf, wrf = x.float(), wr.float()
    scores, idx = OM.router_topk_softmax(logits, K)
    md = R.topk_metadata(idx, scores, E, 128, lane_order="slot", pad_mode="virtual")
    r = OM.moe_fp32(x, w1, w2, md, dy)
    dscores = r["ds"].view(-1, K)
    dlogits = OM.router_backward(scores, idx, dscores, E)
    r["dx_total"] = r["dx"] + dlogits @ wrf
    r["dwr"] = dlogits.T @ xf
    r["dlogits"] = dlogits
    r["idx"], r["scores"], r["md"] = idx, scores, md
    # the same layer through the FP8-emulating dataflow (router stays in bf16/fp32 as in the module)
    e = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    e_dlogits = OM.router_backward(scores, idx, e["ds"].view(-1, K), E)
    r["emu"] = dict(o=e["o"], dx_total=e["dx"].float() + e_dlogits @ wrf, dw1=e["dw1"],
                    dw2=e["dw2_IH"].transpose(1, 2), dwr=e_dlogits.T @ xf)
    return r


@pytest.mark.parametrize("T,H,I,E,K,seed", [(256, 256, 128, 8, 2, 0), (1024, 512, 256, 16, 4, 1),
                                             (512, 1024, 384, 8, 8, 2)])
def test_moe_module_fwd_bwd_vs_fp32_oracle(sm, T, H, I, E, K, seed):
    x, dy, w1, w2, wr, _ = make_layer(T, H, I, E, K, seed)
    moe = sm.MoE(E, K, H, I, sm.ActivationType.SWIGLU, add_bias=False, std=0.02).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        moe.router.weight.copy_(wr)
        moe.c_fc.weight.copy_(w1)
        moe.c_proj.weight.copy_(w2)
    xd = x.to(DEV).requires_grad_(True)
    out, aux = moe(xd, use_fp8=True)
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    with torch.no_grad():
        logits = torch.nn.functional.linear(x.to(DEV), moe.router.weight).float().cpu()
    ref = oracle_dense(x, dy, w1, w2, wr, K, logits)
    emu = ref["emu"]
    check("out", out, ref["o"], emu=emu["o"])
    check("dx", xd.grad, ref["dx_total"], emu=emu["dx_total"])
    check("dw1", moe.c_fc.weight.grad, ref["dw1"], emu=emu["dw1"])
    check("dw2", moe.c_proj.weight.grad, ref["dw2"], emu=emu["dw2"])
    check("drouter", moe.router.weight.grad, ref["dwr"], emu=emu["dwr"])
    assert aux is not None and torch.isfinite(aux)
    # aux loss = E * sum(normalize1(sum_t softmax(logits)) * normalize1(freq))
    freq = torch.bincount(ref["idx"].flatten().long(), minlength=E).float()
    exp = E * (torch.nn.functional.normalize(torch.softmax(logits, -1).sum(0), p=1, dim=0) *
               torch.nn.functional.normalize(freq, p=1, dim=0)).sum()
    assert abs(float(aux.detach()) - float(exp)) < 1e-3 * abs(float(exp))


def test_module_rejects_non_fp8_and_other_backends(sm):
    moe = sm.MoE(8, 2, 256, 128, sm.ActivationType.SWIGLU, add_bias=False, std=0.02).to(DEV).to(torch.bfloat16)
    x = torch.randn(64, 256, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        moe(x)
    with pytest.raises(NotImplementedError):
        moe(x, kernel_backend_moe=sm.KernelBackendMoE.torch, use_fp8=True)


def masked_routing(T, E, K, E_local, seed, bias=None):
    """Global top-k routing; experts >= E_local are 'not local' (-1), as an EP rank sees it."""
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if bias is not None:
        logits = logits + bias
    scores, idx = OM.router_topk_softmax(logits, K)
    idx = torch.where(idx < E_local, idx, torch.full_like(idx, -1))
    return idx, scores


@pytest.mark.parametrize("sizing", ["exact", "sync_free"])
def test_run_sonic_moe_masked_skewed_vs_oracles(sm, sizing):
    T, H, I, E, K = 2048, 512, 256, 32, 8
    x, dy, w1, w2, _, bias = make_layer(T, H, I, E, K, 5, skew=True)
    E_local = 24                                       # 8 experts "remote"; Zipf skew leaves some local ones empty
    idx, scores = masked_routing(T, E, K, E_local, 6, bias * 3)
    w1, w2 = w1[:E_local].contiguous(), w2[:E_local].contiguous()
    counts = torch.bincount(idx[idx >= 0].long(), minlength=E_local)
    assert (counts == 0).any(), "test wants at least one empty expert"
    md = R.topk_metadata(idx, scores, E_local, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)

    xd = x.to(DEV).requires_grad_(True)
    w1d = w1.to(DEV).requires_grad_(True)
    w2d = w2.to(DEV).requires_grad_(True)
    sd = scores.to(DEV).requires_grad_(True)
    kw = dict(tokens_per_expert=counts.tolist()) if sizing == "exact" else dict(sync_free_sizing=True)
    out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E_local, w1d, w2d, fp8=True, **kw)
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    ds_ref = torch.zeros(T * K)
    ds_ref[md["score_src_idx"][:md["real_TK"]].long()] = gold["ds"][:md["real_TK"]]
    ds_emu = torch.zeros(T * K)
    ds_emu[md["score_src_idx"][:md["real_TK"]].long()] = emu["ds"][:md["real_TK"]]
    for name, got, ref, em in [("out", out, gold["o"], emu["o"]), ("dx", xd.grad, gold["dx"], emu["dx"]),
                               ("dw1", w1d.grad, gold["dw1"], emu["dw1"]),
                               ("dw2", w2d.grad, gold["dw2"], emu["dw2_IH"].transpose(1, 2)),
                               ("ds", sd.grad.flatten(), ds_ref, ds_emu)]:
        check(name, got, ref, emu=em)
    # empty experts: exactly-zero weight gradients; masked slots: exactly-zero score gradients
    empty = (counts == 0).nonzero().flatten()
    assert (w1d.grad[empty.to(DEV)] == 0).all() and (w2d.grad[empty.to(DEV)] == 0).all()
    assert (sd.grad.cpu()[idx < 0] == 0).all()


def test_main_grad_accumulation_and_bit_exact_repeat(sm):
    T, H, I, E, K = 1024, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 9)
    idx, scores = masked_routing(T, E, K, E, 10)
    w1d = torch.nn.Parameter(w1.to(DEV))
    w2d = torch.nn.Parameter(w2.to(DEV))
    hooks = []
    for w, shape in ((w1d, (E, 2 * I, H)), (w2d, (E, I, H))):
        w.main_grad = torch.zeros(shape, dtype=torch.float32, device=DEV)
        w._apply_backward_hook = lambda: hooks.append(1)

    def step():
        xd = x.to(DEV).requires_grad_(True)
        sd = scores.to(DEV).requires_grad_(True)
        out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True)
        out.backward(dy.to(DEV))
        return out.detach().clone(), xd.grad.clone(), sd.grad.clone()

    o1, dx1, ds1 = step()
    g1 = (w1d.main_grad.clone(), w2d.main_grad.clone())
    assert w1d.grad is None and w2d.grad is None and len(hooks) == 2
    o2, dx2, ds2 = step()
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    assert torch.equal(o1, o2) and torch.equal(dx1, dx2) and torch.equal(ds1, ds2)
    # second step added exactly the same increment
    assert torch.equal(w1d.main_grad - g1[0], g1[0]) and torch.equal(w2d.main_grad - g1[1], g1[1])
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    check("main_grad w1", g1[0], gold["dw1"], emu=emu["dw1"])
    check("main_grad w2 [E,I,H]", g1[1], gold["dw2_IH"], emu=emu["dw2_IH"])


def test_all_masked_and_single_token(sm):
    H, I, E, K = 256, 128, 8, 2
    x, dy, w1, w2, _, _ = make_layer(64, H, I, E, K, 3)
    idx = torch.full((64, K), -1, dtype=torch.int32)
    scores = torch.rand(64, K)
    xd = x.to(DEV).requires_grad_(True)
    w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
    out = sm.run_sonic_moe(xd, idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True)
    out.backward(dy.to(DEV))
    assert (out == 0).all() and (xd.grad == 0).all() and (w1d.grad == 0).all() and (w2d.grad == 0).all()
    # one token
    idx = torch.tensor([[3, 5]], dtype=torch.int32)
    scores = torch.tensor([[0.7, 0.3]])
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x[:1], w1, w2, md, dy[:1])
    xd = x[:1].to(DEV).requires_grad_(True)
    out = sm.run_sonic_moe(xd, idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True)
    out.backward(dy[:1].to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    check("out", out, gold["o"], cos_min=0.99, rr_max=0.12)     # 256 values: loose statistics
    check("dx", xd.grad, gold["dx"], cos_min=0.99, rr_max=0.12)


def test_mlp_node_split_half_experts_and_main_grad_flush(sm):
    """SonicMoEMlpNode on dispatched rows: per-expert split-half weights in, per-expert main_grad in the
    framework's layouts out (after step()), two micro-batches accumulated."""
    from sonicmoe.ernie_compat import SonicMoEMlpNode
    T, H, I, E, K = 768, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 21)
    idx, scores = masked_routing(T, E, K, E, 22)

    class Lin:
        def __init__(self, w):
            self.weight = w

    class Expert:
        def __init__(self, e):
            # split-half [H, 2I]: gates are the even rows of the interleaved w1, ups the odd rows
            self.up_gate_proj = Lin(torch.cat([w1[e, 0::2].T, w1[e, 1::2].T], dim=1).contiguous().to(DEV))
            self.down_proj = Lin(w2[e].T.contiguous().to(DEV))

    experts = [Expert(e) for e in range(E)]
    node = SonicMoEMlpNode(experts, E, H, I)
    counts = torch.bincount(idx[idx >= 0].long(), minlength=E)
    outs = []
    for _ in range(2):
        xd = x.to(DEV).requires_grad_(True)
        pd = scores.to(DEV).requires_grad_(True)
        out = node(xd, counts.tolist(), idx.to(DEV), pd)
        out.backward(dy.to(DEV))
        outs.append((out.detach(), xd.grad, pd.grad))
    node.step()
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    check("node out", outs[0][0], gold["o"], emu=emu["o"])
    check("node dx", outs[0][1], gold["dx"], emu=emu["dx"])
    # per-expert main_grad, framework layouts, two micro-batches
    g1 = torch.stack([e.up_gate_proj.weight.main_grad for e in experts]).cpu() / 2       # [E, H, 2I] split-half
    g2 = torch.stack([e.down_proj.weight.main_grad for e in experts]).cpu() / 2          # [E, I, H]
    to_split = lambda d: torch.cat([d[:, 0::2].transpose(1, 2), d[:, 1::2].transpose(1, 2)], dim=2)
    check("node dw1 (split-half)", g1, to_split(gold["dw1"]), emu=to_split(emu["dw1"]))
    check("node dw2 [E,I,H]", g2, gold["dw2_IH"], emu=emu["dw2_IH"])
    # a second step() without a backward in between must not flush again
    before = experts[0].up_gate_proj.weight.main_grad.clone()
    node.step()
    assert torch.equal(before, experts[0].up_gate_proj.weight.main_grad)


def test_recompute_z_gives_the_same_bits_and_does_not_keep_z(sm):
    """`SonicMoEConfig(recompute_z=True)`: z is dropped after the forward and regenerated in the backward by the
    same kernels, so every output and gradient is bit-identical to the default (z saved)."""
    T, H, I, E, K = 1024, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 31)
    idx, scores = masked_routing(T, E, K, E, 32)

    def run(cfg):
        xd = x.to(DEV).requires_grad_(True)
        sd = scores.to(DEV).requires_grad_(True)
        w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
        out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True, fp8_config=cfg)
        links = [f for f in (out.grad_fn, ) if f is not None]
        out.backward(dy.to(DEV))
        torch.cuda.synchronize()
        sm.ops.check_status(DEV)
        return out.detach(), xd.grad, sd.grad, w1d.grad, w2d.grad

    base = run(None)
    rec = run(sm.SonicMoEConfig(use_fp8=True, recompute_z=True))
    for name, a, b in zip(("out", "dx", "ds", "dw1", "dw2"), base, rec):
        assert torch.equal(a, b), name
    # and through the thread-local activation, as the reference's callers set it
    with sm.SonicMoEConfig(use_fp8=True, recompute_z=True).activate():
        act = run(None)
    for a, b in zip(base, act):
        assert torch.equal(a, b)


def test_weight_cache_is_not_fooled_by_a_recycled_address(sm):
    """A weight that is freed and another of the same shape allocated at the same address (the caching allocator
    does that) must not be served the first one's FP8 copy."""
    from sonicmoe.functional import weight_fp8
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(4, 256, 128, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    qa = weight_fp8(a, False)[0].clone()
    ptr = a.data_ptr()
    del a
    b = (torch.randn(4, 256, 128, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    if b.data_ptr() != ptr:
        pytest.skip("allocator did not recycle the address")
    qb = weight_fp8(b, False)[0]
    want = sm.ops.quant_rows(b.view(4 * 256, 128), raw=False, isa=True)[0].view(4, 256, 128)
    assert torch.equal(qb, want) and not torch.equal(qb, qa)


def test_caller_owned_buffers_for_output_and_dx(sm):
    """`run_sonic_moe(out=..., dx_out=...)`: the forward output and dx are written straight into the caller's bf16
    buffers (the expert-parallel layer points them at memory its peers read), with the same bits as without."""
    T, H, I, E, K = 512, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 41)
    idx, scores = masked_routing(T, E, K, E, 42)
    w1d, w2d = w1.to(DEV), w2.to(DEV)

    def run(**kw):
        xd = x.to(DEV).requires_grad_(True)
        out = sm.run_sonic_moe(xd, idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True, **kw)
        out.backward(dy.to(DEV))
        torch.cuda.synchronize()
        return out, xd.grad

    ref_out, ref_dx = run()
    buf_o = torch.full((T, H), 7.0, dtype=torch.bfloat16, device=DEV)
    buf_dx = torch.full((T, H), 7.0, dtype=torch.bfloat16, device=DEV)
    out, dx = run(out=buf_o, dx_out=buf_dx)
    # (a leaf's .grad is autograd's own copy; a non-leaf consumer, like the EP dispatch, gets the buffer itself)
    assert out.data_ptr() == buf_o.data_ptr() and torch.equal(buf_dx, ref_dx)
    assert torch.equal(out, ref_out) and torch.equal(dx, ref_dx)
    one = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)          # one region used in turn, as the EP layer does
    out, dx = run(out=one, dx_out=one)
    assert torch.equal(dx, ref_dx) and torch.equal(one, ref_dx)
    with pytest.raises(ValueError):
        run(out=torch.empty(T, H + 8, dtype=torch.bfloat16, device=DEV))
    # nothing leaks into the next call
    out, dx = run()
    assert out.data_ptr() not in (buf_o.data_ptr(), one.data_ptr()) and torch.equal(out, ref_out)


def test_exact_sizing_with_nothing_routed(sm):
    """`tokens_per_expert` all zero (what an expert-parallel rank passes when it received no routed pairs): every
    expert-sorted buffer has zero rows, the GEMM entry points return without a launch, out / dx are zero and the
    weight gradients are exactly zero - returned, and accumulated into main_grad."""
    H, I, E, K = 256, 128, 8, 2
    x, dy, w1, w2, _, _ = make_layer(64, H, I, E, K, 3)
    idx = torch.full((64, K), -1, dtype=torch.int32)
    scores = torch.rand(64, K)
    xd = x.to(DEV).requires_grad_(True)
    sd = scores.to(DEV).requires_grad_(True)
    w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
    out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True, tokens_per_expert=[0] * E)
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    assert (out == 0).all() and (xd.grad == 0).all() and (sd.grad == 0).all()
    assert (w1d.grad == 0).all() and (w2d.grad == 0).all()
    # with main_grad: the accumulators are left as they were
    w1p, w2p = torch.nn.Parameter(w1.to(DEV)), torch.nn.Parameter(w2.to(DEV))
    w1p.main_grad = torch.full((E, 2 * I, H), 3.0, dtype=torch.float32, device=DEV)
    w2p.main_grad = torch.full((E, I, H), 5.0, dtype=torch.float32, device=DEV)
    out = sm.run_sonic_moe(x.to(DEV).requires_grad_(True), idx.to(DEV), scores.to(DEV), K, E, w1p, w2p, fp8=True,
                           tokens_per_expert=torch.zeros(E, dtype=torch.int64))
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    assert (w1p.main_grad == 3.0).all() and (w2p.main_grad == 5.0).all()
    # the C ABI itself: zero rows are not an error, an overwriting weight gradient stores zeros
    from sonicmoe._lib import lib
    st = sm.ops.status_word(DEV)
    assert lib.smoe_gemm_varlen_m(None, None, None, None, None, None, 0, 256, 128, E, st.data_ptr(), None) == 0
    assert lib.smoe_gemm_gated(None, 0, None, None, None, None, None, None, None, None, None, 0, 256, 128, E,
                               st.data_ptr(), None) == 0
    c = torch.full((E, 256, 256), 9.0, dtype=torch.float32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.smoe_gemm_wgrad_mn(None, None, None, None, None, c.data_ptr(), 256, 256, 0, E, 0, 3, st.data_ptr(),
                                  stream) == 0
    assert lib.smoe_gemm_wgrad(None, None, None, None, None, c.data_ptr(), 256, 256, 0, E, 1, st.data_ptr(),
                               stream) == 0
    torch.cuda.synchronize()
    assert (c == 0).all()


def test_two_layers_forward_interleaved_before_their_backwards(sm):
    """Two layers (different weights, different tokens) whose `_UpProjection`s both run before either
    `_DownProjection`, and whose backwards run in the opposite order: each pair must find its own FP8 payloads
    (reference: tests/ops/test_mlpnode_multilayer.py; hand-off keyed per invocation)."""
    from sonicmoe import ops
    from sonicmoe.functional import _DownProjection, _UpProjection, enable_fp8
    T, H, I, E, K = 512, 512, 256, 8, 4
    layers = []
    for seed in (51, 52):
        x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, seed)
        idx, scores = masked_routing(T, E, K, E, seed + 10)
        layers.append(dict(x=x, dy=dy, w1=w1, w2=w2, idx=idx, scores=scores))

    def alone(L):
        xd = L["x"].to(DEV).requires_grad_(True)
        w1d, w2d = L["w1"].to(DEV).requires_grad_(True), L["w2"].to(DEV).requires_grad_(True)
        out = sm.run_sonic_moe(xd, L["idx"].to(DEV), L["scores"].to(DEV), K, E, w1d, w2d, fp8=True)
        out.backward(L["dy"].to(DEV))
        return out.detach(), xd.grad, w1d.grad, w2d.grad

    want = [alone(L) for L in layers]
    st = []
    with enable_fp8(True):
        for L in layers:                                    # both up-projections first
            xd = L["x"].to(DEV).requires_grad_(True)
            w1d, w2d = L["w1"].to(DEV).requires_grad_(True), L["w2"].to(DEV).requires_grad_(True)
            md = ops.topk_metadata(L["idx"].to(DEV), L["scores"].to(DEV), E, 128)
            y1, z = _UpProjection.apply(xd, w1d, None, md["efo"], md["TKp_alloc"], K, 0, md["x_gather_idx"],
                                        md["s_scatter_idx"], md["s_reverse_scatter_idx"], md["naept"], True,
                                        sm.ActivationType.SWIGLU, False)
            st.append(dict(xd=xd, w1d=w1d, w2d=w2d, md=md, y1=y1, z=z))
        for L, s in zip(layers, st):                        # then both down-projections
            md = s["md"]
            s["out"] = _DownProjection.apply(s["y1"], s["z"], s["w2d"], None, md["topk_scores"], md["s_scatter_idx"],
                                             md["efo"], T, K, 0, md["x_gather_idx"], md["s_scatter_idx"],
                                             md["s_reverse_scatter_idx"], md["naept"], True,
                                             sm.ActivationType.SWIGLU, None)
        for L, s in reversed(list(zip(layers, st))):        # backwards in the opposite order
            s["out"].backward(L["dy"].to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    for w, s in zip(want, st):
        for name, a, b in zip(("out", "dx", "dw1", "dw2"), w, (s["out"].detach(), s["xd"].grad, s["w1d"].grad,
                                                                 s["w2d"].grad)):
            assert torch.equal(a, b), name
    # a z that did not come from _UpProjection is refused instead of silently pairing with someone else's payload
    with enable_fp8(True), pytest.raises(RuntimeError):
        md = st[0]["md"]
        _DownProjection.apply(torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), st[0]["w2d"], None,
                              md["topk_scores"], md["s_scatter_idx"], md["efo"], T, K, 0, md["x_gather_idx"],
                              md["s_scatter_idx"], md["s_reverse_scatter_idx"], md["naept"], True,
                              sm.ActivationType.SWIGLU, None)


def test_weight_update_through_data_copy_is_seen_after_invalidation(sm):
    """`param.data.copy_(master)` does not move the tensor version counter the FP8 weight cache looks at: the
    cached copy stays in use until `drop_weight_fp8` / `clear_weight_cache` is called, and `SonicMoEMlpNode.step()`
    drops its stacked weights and their FP8 copies itself."""
    from sonicmoe.ernie_compat import SonicMoEMlpNode
    T, H, I, E, K = 256, 256, 128, 8, 2
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 61)
    idx, scores = masked_routing(T, E, K, E, 62)
    w1d, w2d = w1.to(DEV), w2.to(DEV)
    run = lambda: sm.run_sonic_moe(x.to(DEV), idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True)
    a = run().clone()
    w1d.data.copy_(w1d * 2)                       # invisible to the version counter
    stale = run().clone()
    sm.drop_weight_fp8(w1d)
    fresh = run().clone()
    assert torch.equal(a, stale) and not torch.equal(a, fresh)

    class Lin:
        def __init__(self, w):
            self.weight = w

    class Expert:
        def __init__(self, e):
            self.up_gate_proj = Lin(torch.cat([w1[e, 0::2].T, w1[e, 1::2].T], dim=1).contiguous().to(DEV))
            self.down_proj = Lin(w2[e].T.contiguous().to(DEV))

    experts = [Expert(e) for e in range(E)]
    node = SonicMoEMlpNode(experts, E, H, I)
    counts = torch.bincount(idx[idx >= 0].long(), minlength=E).tolist()
    o1 = node(x.to(DEV), counts, idx.to(DEV), scores.to(DEV)).detach().clone()
    node.step()
    for e in experts:                             # "optimizer step" through .data
        e.down_proj.weight.data.copy_(e.down_proj.weight * 2)
    o2 = node(x.to(DEV), counts, idx.to(DEV), scores.to(DEV)).detach()
    torch.cuda.synchronize()
    c, r = stats(o2, o1 * 2)
    assert not torch.equal(o1, o2) and c > 0.9999 and r < 0.01


def test_device_failure_code_surfaces_at_the_next_call_without_a_sync(sm):
    """The layer posts the GEMM status word to pinned host memory at the end of each pass and looks at it on the
    next entry: a non-zero code (here written by hand; a kernel writes it when a bounded wait runs out) raises."""
    T, H, I, E, K = 256, 256, 128, 8, 2
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 71)
    idx, scores = masked_routing(T, E, K, E, 72)
    w1d, w2d = w1.to(DEV), w2.to(DEV)
    run = lambda: sm.run_sonic_moe(x.to(DEV), idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True)
    run()
    torch.cuda.synchronize()
    run()                                          # healthy: the posted copy is zero, nothing raises
    sm.ops.status_word(DEV).fill_(202)
    run()                                          # this pass posts the non-zero word ...
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="202"):
        run()                                      # ... and the next entry reports it
    torch.cuda.synchronize()
    assert int(sm.ops.status_word(DEV).item()) == 0
    run()
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)


def make_layer_reference_bench(T, H, I, E, K, seed):
    """Inputs as the reference's own benchmark draws them (tests/ops/bench_mlpnode_topk_nsys.py:113-200), the
    distribution its published precision (cos >= 0.997, RRMSE < 7.6 %) was measured on: x = randn * 0.02,
    dy = randn * 0.01, weights = randn / sqrt(fan_in), experts = top-k of randn(T,E), probabilities = U(0.5,1)
    normalised over the K slots."""
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(E, 2 * I, H, generator=g) / H ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn(E, H, I, generator=g) / I ** 0.5).to(torch.bfloat16)
    _, idx = torch.randn(T, E, generator=g).topk(K, dim=-1)
    p = torch.rand(T, K, generator=g) * 0.5 + 0.5
    p = (p / p.sum(dim=1, keepdim=True)).float()
    x = (torch.randn(T, H, generator=g) * 0.02).to(torch.bfloat16)
    dy = (torch.randn(T, H, generator=g) * 0.01).to(torch.bfloat16)
    return x, dy, w1, w2, idx.to(torch.int32), p


@pytest.mark.parametrize("T,H,I,E,K,seed", [(1024, 512, 256, 16, 4, 42), (512, 1024, 384, 8, 8, 123),
                                             (2048, 512, 256, 8, 8, 777)])
def test_reference_bench_distribution_meets_the_published_tolerance_as_it_stands(sm, T, H, I, E, K, seed):
    """On the reference's own input distribution every tensor - out, dx, dscores, dw1, dw2 - must meet the published
    bound itself: cosine >= 0.997 and RRMSE <= 7.6 % against the fp32 gold, no emulation-relative widening.  (The
    CPU emulation of the reference dataflow lands on the reference's published per-tensor figures here: out 0.9978,
    dx 0.9975, ds 0.9972, dw1 0.9977, dw2 0.9972.)"""
    from parity_util import gate
    x, dy, w1, w2, idx, p = make_layer_reference_bench(T, H, I, E, K, seed)
    md = R.topk_metadata(idx, p, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    xd = x.to(DEV).requires_grad_(True)
    pd = p.to(DEV).requires_grad_(True)
    w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
    counts = torch.bincount(idx.flatten().long(), minlength=E).tolist()
    out = sm.run_sonic_moe(xd, idx.to(DEV), pd, K, E, w1d, w2d, fp8=True, tokens_per_expert=counts)
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    tk = md["real_TK"]
    ds_of = lambda r: torch.zeros(T * K).index_put_((md["score_src_idx"][:tk].long(),), r["ds"][:tk].float())
    report = []
    for name, got, ref, em in [("out", out, gold["o"], emu["o"]), ("dx", xd.grad, gold["dx"], emu["dx"]),
                               ("ds", pd.grad.flatten(), ds_of(gold), ds_of(emu)),
                               ("dw1", w1d.grad, gold["dw1"], emu["dw1"]),
                               ("dw2", w2d.grad, gold["dw2"], emu["dw2_IH"].transpose(1, 2))]:
        gate(name, got, ref, em, strict=True, report=report)
    print("\n" + "\n".join(f"refdist {T}x{H}x{I} E{E} K{K} {n}: gpu cos {a:.5f} rrmse {b:.5f} | emulation "
                           f"{c:.5f} {d:.5f} | gpu vs emulation {e:.5f} {f:.5f}" for n, a, b, c, d, e, f in report))


@pytest.mark.parametrize("routing", ["down", "up", "nr"])
def test_token_rounding_router_through_general_routing(sm, routing):
    """`token_rounding_routing` -> `moe_general_routing_inputs`: every expert's row count is a multiple of 128, so the
    padded layout has no pad row at all, and out / dx / dscores / dw1 / dw2 meet both oracles
    (reference: benchmarks/moe-token-rounding.py:103-181)."""
    from parity_util import gate
    T, H, I, E, K = 1024, 512, 256, 16, 4
    x, dy, w1, w2, wr, _ = make_layer(T, H, I, E, K, 81)
    logits = torch.nn.functional.linear(x.float(), wr.float())
    s, tok, exp = sm.token_rounding_routing(logits.to(DEV), K, 128, routing)
    counts = torch.bincount(exp.long(), minlength=E).cpu()
    assert bool((counts % 128 == 0).all()) and int(counts.sum()) == tok.numel()
    # the same pairs as a padded table for the oracles
    from sonicmoe.functional import _pairs_to_table, general_routing_router_metadata
    idx, sc = _pairs_to_table(s.cpu(), tok.cpu(), exp.cpu(), T)
    md = R.topk_metadata(idx, sc, E, 128)
    assert md["real_TKp"] == md["real_TK"] == tok.numel(), "no pad rows"
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy)
    xd = x.to(DEV).requires_grad_(True)
    sd = s.detach().clone().requires_grad_(True)
    moe = sm.MoE(E, K, H, I, sm.ActivationType.SWIGLU, add_bias=False, std=0.02).to(DEV).to(torch.bfloat16)
    with torch.no_grad():
        moe.c_fc.weight.copy_(w1)
        moe.c_proj.weight.copy_(w2)
    with sm.enable_fp8():
        o, freq = sm.moe_general_routing_inputs(xd, sd, tok, exp, moe.c_fc.weight.permute(1, 2, 0), None,
                                                moe.c_proj.weight.permute(1, 2, 0), None, E, 0,
                                                sm.ActivationType.SWIGLU, False)
    o.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    assert torch.equal(freq.cpu().long(), counts)
    tk = md["real_TK"]
    # pair i of the (token-sorted) list <-> table slot (token, lane): the oracle's ds is token-major over the table
    flat = torch.zeros(idx.numel())
    ds_pairs = lambda r: flat.clone().index_put_((md["score_src_idx"][:tk].long(),), r["ds"][:tk].float())[
        (idx.flatten() >= 0)]
    for name, got, ref, em in [("out", o, gold["o"], emu["o"]), ("dx", xd.grad, gold["dx"], emu["dx"]),
                               ("ds", sd.grad, ds_pairs(gold), ds_pairs(emu)),
                               ("dw1", moe.c_fc.weight.grad, gold["dw1"], emu["dw1"]),
                               ("dw2", moe.c_proj.weight.grad, gold["dw2"], emu["dw2_IH"].transpose(1, 2))]:
        gate(f"token-rounding {routing} {name}", got, ref, em, strict=False)
    # the unpadded metadata of the reference's general-routing helper: a permutation sorted by expert, tokens
    # ascending inside an expert, and its inverse
    freq2, efo, xg, ss, srev, naept = general_routing_router_metadata(s, tok, exp, T, E)
    n = tok.numel()
    assert torch.equal(freq2.cpu().long(), counts) and int(efo[-1]) == n and int(naept[-1]) == n
    e_sorted = exp.cpu()[ss.cpu().long()]
    assert bool((e_sorted[1:] >= e_sorted[:-1]).all())
    assert torch.equal(xg.cpu()[:n], tok.cpu()[ss.cpu().long()])
    assert torch.equal(ss.cpu()[srev.cpu().long()], torch.arange(n, dtype=torch.int32))


def test_fp8_payload_scale_formats(sm):
    """An FP8 dispatch payload with its scales as u8 [N,H/32], as compact int32 words [N,H/128] (four ue8m0 bytes per
    word) or as int32 [N,H/32] gives bit-identical results (reference: blockscaled_fp8_gemm.py:535-550)."""
    from sonicmoe.quack_utils import quantize_activation_blockscaled_fast as quant
    T, H, I, E, K = 512, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 91)
    idx, scores = masked_routing(T, E, K, E, 92)
    w1d, w2d = w1.to(DEV), w2.to(DEV)
    xd = x.to(DEV)
    q, raw = quant(xd)
    q2, words = quant(xd, pack_scale_words=True)
    q3, wide = quant(xd, scale_dtype=torch.int32)
    assert words.dtype == torch.int32 and tuple(words.shape) == (T, H // 128)
    assert wide.dtype == torch.int32 and tuple(wide.shape) == (T, H // 32)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(words.view(torch.uint8), raw)
    run = lambda sc: sm.run_sonic_moe(q, idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True, fp8_scale=sc)
    base = run(raw)
    assert torch.equal(base, run(words)) and torch.equal(base, run(wide))
    ref = sm.run_sonic_moe(xd, idx.to(DEV), scores.to(DEV), K, E, w1d, w2d, fp8=True)
    assert torch.equal(base, ref)                      # same bytes as quantising inside the layer
    with pytest.raises(ValueError):
        run(raw[:, :-1].contiguous())


@pytest.mark.parametrize("act", ["reglu", "geglu", "swiglu"])
def test_other_gated_activations_match_oracles(sm, act):
    """ReGLU and GEGLU (reference: sonicmoe/enums.py:18-33) run as plain GEMMs + stand-alone activation kernels;
    SwiGLU through the same module path for comparison.  Both oracles take the activation by name."""
    from parity_util import gate
    T, H, I, E, K = 1024, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 101)
    w1 = (w1.float() * 4).to(torch.bfloat16)          # gate values of order one, so the activations differ visibly
    idx, scores = masked_routing(T, E, K, E, 102)
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy, act=act)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy, act=act)
    xd = x.to(DEV).requires_grad_(True)
    sd = scores.to(DEV).requires_grad_(True)
    w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
    out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True, activation_type=sm.ActivationType(act))
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    tk = md["real_TK"]
    ds_of = lambda r: torch.zeros(T * K).index_put_((md["score_src_idx"][:tk].long(),), r["ds"][:tk].float())
    for name, got, ref, em in [("out", out, gold["o"], emu["o"]), ("dx", xd.grad, gold["dx"], emu["dx"]),
                               ("ds", sd.grad.flatten(), ds_of(gold), ds_of(emu)),
                               ("dw1", w1d.grad, gold["dw1"], emu["dw1"]),
                               ("dw2", w2d.grad, gold["dw2"], emu["dw2_IH"].transpose(1, 2))]:
        gate(f"{act} {name}", got, ref, em, strict=False)
    if act != "swiglu":
        sw = OM.moe_fp32(x, w1, w2, md, dy, act="swiglu")["o"]
        assert stats(gold["o"], sw)[1] > 0.05, "the test data must tell the activations apart"
    with pytest.raises(NotImplementedError):
        sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True, activation_type=sm.ActivationType.SITU_GLU)


def test_in_kernel_row_gather_writes_no_gathered_copy_and_gives_the_same_bits(sm):
    """SONIC_MOE_A_GATHER=cpasync: x and dout are quantised once as [T,H] and the GEMMs fetch their rows by index
    (four cp.async load warps per CTA) - no expert-sorted [TKp,H] copy is written or read - with results bit-identical
    to the gathered-copy path."""
    import sonicmoe.functional as Fn
    T, H, I, E, K = 1024, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 111)
    idx, scores = masked_routing(T, E, K, 6, 112)          # two experts remote: masked slots, pad rows
    w1d, w2d = w1[:6].contiguous().to(DEV), w2[:6].contiguous().to(DEV)

    def run(mode):
        prev = (Fn.A_GATHER, Fn.USE_TMA_GATHER)
        Fn.A_GATHER, Fn.USE_TMA_GATHER = mode, mode == "cpasync"
        rec = []
        sm.ops.set_recorder(rec)
        try:
            xd = x.to(DEV).requires_grad_(True)
            sd = scores.to(DEV).requires_grad_(True)
            a, b = w1d.detach().requires_grad_(True), w2d.detach().requires_grad_(True)
            out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, 6, a, b, fp8=True)
            out.backward(dy.to(DEV))
            torch.cuda.synchronize()
            sm.ops.check_status(DEV)
        finally:
            sm.ops.set_recorder(None)
            Fn.A_GATHER, Fn.USE_TMA_GATHER = prev
        return (out.detach(), xd.grad, sd.grad, a.grad, b.grad), [n for n, _, _ in rec]

    base, ops_copy = run("copy")
    got, ops_cp = run("cpasync")
    assert "quant_rows_scatter" in ops_copy
    assert not {"quant_rows_scatter", "gather_rows_fp8", "scatter_rows_fp8", "quant_rows_gather"} & set(ops_cp)
    # x and dout are quantised once each as [T,H] (the other quant_rows calls are the weight copies of either mode)
    assert ops_cp.count("quant_rows") == ops_copy.count("quant_rows") + 2 and ops_cp.count("gather_scales_isa") == 2
    for name, a, b in zip(("out", "dx", "ds", "dw1", "dw2"), base, got):
        assert torch.equal(a, b), name


def test_transposed_weight_copy_without_a_transposed_bf16_tensor(sm):
    """`weight_fp8(w, transposed=True)` quantises W^T row-wise by running the column quantizer over W as it lies:
    same bytes and scale bytes as transposing first and quantising rows."""
    from sonicmoe.functional import clear_weight_cache, weight_fp8
    g = torch.Generator().manual_seed(121)
    for E, N, K in ((4, 256, 128), (3, 384, 256), (2, 128, 384)):
        w = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
        clear_weight_cache()
        q, sf = weight_fp8(w, True)
        wt = w.transpose(1, 2).contiguous()
        rq, _, rsf = sm.ops.quant_rows(wt.view(E * K, N), raw=False, isa=True)
        assert tuple(q.shape) == (E, K, N) and torch.equal(q.view(E * K, N), rq)
        got = torch.stack([Q.unpack_isa(sf.cpu()[e * sm.ops.isa_bytes(K, N):(e + 1) * sm.ops.isa_bytes(K, N)], K, N)
                           for e in range(E)])
        assert torch.equal(sf, rsf)                      # per-expert ISA blocks concatenated = the (E*K, N) layout
        assert torch.equal(got, Q.unpack_isa(rsf.cpu(), E * K, N).view(E, K, N // 32))
        oq, osc = Q.row_quant(wt.view(E * K, N).float().cpu())
        assert torch.equal(q.view(E * K, N).cpu(), oq) and torch.equal(got.view(E * K, N // 32), osc)


def _layer_run(sm, x, dy, w1, w2, idx, scores, K, E, cfg=None, main_grad=False):
    xd = x.to(DEV).requires_grad_(True)
    sd = scores.to(DEV).requires_grad_(True)
    w1d, w2d = w1.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
    if main_grad:
        w1d.main_grad = torch.zeros(w1.shape, dtype=torch.float32, device=DEV)
        w2d.main_grad = torch.zeros(w2.shape[0], w2.shape[2], w2.shape[1], dtype=torch.float32, device=DEV)
    out = sm.run_sonic_moe(xd, idx.to(DEV), sd, K, E, w1d, w2d, fp8=True, fp8_config=cfg)
    out.backward(dy.to(DEV))
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)
    if main_grad:
        return out.detach(), xd.grad, sd.grad, w1d.main_grad, w2d.main_grad
    return out.detach(), xd.grad, sd.grad, w1d.grad, w2d.grad


@pytest.mark.parametrize("T,H,I,E,K,seed", [(1024, 512, 256, 8, 4, 131), (512, 384, 256, 4, 2, 132)])
def test_iso32_weight_cache_one_buffer_per_weight(sm, T, H, I, E, K, seed):
    """`SonicMoEConfig(iso32_weight=True)`: each weight is quantised once with one scale per 32x32 block; the forward
    GEMMs read that buffer K-major and the activation-gradient GEMM reads the same bytes MN-major (H % 256 == 0) or
    through a transient byte transpose.  Half the cached FP8 weight bytes, results equal to the CPU emulation of
    the same dataflow, and inside the reference's FP8 thresholds against fp32 (tests/ops/test_moe_module.py:56-61:
    RRMSE < 0.10, cosine > 0.99)."""
    import sonicmoe.functional as Fn
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, seed)
    idx, scores = masked_routing(T, E, K, E, seed + 1)
    md = R.topk_metadata(idx, scores, E, 128)
    gold = OM.moe_fp32(x, w1, w2, md, dy)
    emu = OM.moe_fp8_emulated(x, w1, w2, md, dy, iso32_weight=True)

    def cached_bytes():
        return sum(v[1].numel() for v in Fn._WEIGHT_CACHE.values())

    Fn.clear_weight_cache()
    base = _layer_run(sm, x, dy, w1, w2, idx, scores, K, E)
    two_copies = cached_bytes()
    Fn.clear_weight_cache()
    rec = []
    sm.ops.set_recorder(rec)
    try:
        got = _layer_run(sm, x, dy, w1, w2, idx, scores, K, E, sm.SonicMoEConfig(use_fp8=True, iso32_weight=True))
    finally:
        sm.ops.set_recorder(None)
    names = [n for n, _, _ in rec]
    assert cached_bytes() * 2 == two_copies
    assert all(k[3] == "iso32" for k in Fn._WEIGHT_CACHE)
    fused = H % 256 == 0 and I % 256 == 0            # else dz takes the stand-alone 32x32-block quantizer once
    assert names.count("quant_iso32") == 2 * E + (0 if fused else 1) and "quant_rows" not in names
    assert ("gemm_varlen_m_bt" in names) == (H % 256 == 0) and names.count("transpose_u8") == (1 if H % 256 == 0 else 2)
    ds_ref, ds_emu = torch.zeros(T * K), torch.zeros(T * K)
    ds_ref[md["score_src_idx"][:md["real_TK"]].long()] = gold["ds"][:md["real_TK"]]
    ds_emu[md["score_src_idx"][:md["real_TK"]].long()] = emu["ds"][:md["real_TK"]]
    refs = dict(out=(gold["o"], emu["o"]), dx=(gold["dx"], emu["dx"]), ds=(ds_ref, ds_emu),
                dw1=(gold["dw1"], emu["dw1"]), dw2=(gold["dw2"], emu["dw2_IH"].transpose(1, 2)))
    for (name, (g, e)), t in zip(refs.items(), got):
        t = t.flatten() if name == "ds" else t
        c, r = stats(t, e)
        assert c >= 0.9995 and r <= 0.03, f"{name} vs emulation: cos {c:.5f} rrmse {r:.5f}"
        c, r = stats(t, g)
        assert c >= 0.99 and r <= 0.10, f"{name} vs fp32: cos {c:.5f} rrmse {r:.5f}"
    # the environment switch selects the same path
    import os
    os.environ["SONIC_MOE_FP8_ISO32_WEIGHT"] = "1"
    try:
        env = _layer_run(sm, x, dy, w1, w2, idx, scores, K, E)
    finally:
        del os.environ["SONIC_MOE_FP8_ISO32_WEIGHT"]
    for a, b in zip(got, env):
        assert torch.equal(a, b)
    # coarser scales: the scale bytes differ from the 1x32 copy's (the layer's results may still coincide bit for bit:
    # a power-of-two scale twice as large costs an e4m3 value nothing until it turns subnormal)
    w1d = w1.to(DEV)
    q32, rsf32, _ = Fn.weight_fp8_iso32(w1d)
    q1, sf1 = Fn.weight_fp8(w1d, False)
    assert not torch.equal(rsf32, sf1)
    for a, b in zip(base, got):
        c, r = stats(b, a)
        assert c >= 0.9999 and r <= 0.02
    Fn.clear_weight_cache()


def test_stagewise_memory_same_bits_lower_backward_peak_and_a_stage_record(sm):
    """`SonicMoEConfig(stagewise_memory=True)`: the backward makes each operand right before its one consumer and
    frees it right after (dout's column-quantised copy after GemmDGated has released z and the gathered rows; dw2
    before dx_expanded is allocated).  Bit-identical results, a lower peak, and a per-stage memory record."""
    import sonicmoe.functional as Fn
    T, H, I, E, K = 4096, 1024, 512, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 141)
    idx, scores = masked_routing(T, E, K, E, 142)

    def run(cfg):
        _layer_run(sm, x, dy, w1, w2, idx, scores, K, E, cfg, main_grad=True)      # warm the weight cache
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        before = torch.cuda.memory_allocated()
        res = _layer_run(sm, x, dy, w1, w2, idx, scores, K, E, cfg, main_grad=True)
        return res, torch.cuda.max_memory_allocated() - before

    base, peak_default = run(None)
    del Fn.STAGE_MEMORY_LOG[:]
    lean, peak_lean = run(sm.SonicMoEConfig(use_fp8=True, stagewise_memory=True))
    for name, a, b in zip(("out", "dx", "ds", "dw1", "dw2"), base, lean):
        assert torch.equal(a, b), name
    stages = [s for s, _, _ in Fn.STAGE_MEMORY_LOG]
    for want in ("forward: after up-projection", "forward: after down-projection", "backward: after GemmDGated",
                 "backward: after dw2", "backward: after dx", "backward: after dw1"):
        assert want in stages, (want, stages)
    assert stages.index("backward: after dw2") < stages.index("backward: after dx")
    TKp = T * K + E * 128
    # the default holds dout's column copy and y1s (TKp*(H+I) bytes) while dx_expanded (2*TKp*H) is live
    assert peak_lean < peak_default - TKp * I // 2, (peak_lean, peak_default)


def test_metadata_with_scales_and_preallocated_gated_outputs(sm):
    """`deepep_topk_to_sonic_metadata_with_scales`: the ten metadata values, the payload's scales gathered to
    expert-sorted rows in the ISA layout (u8 and compact int32 carriers give the same bytes), and the four
    up-projection outputs allocated for the call; a payload carrying them makes `_UpProjection` write there."""
    from sonicmoe.ernie_compat import deepep_topk_to_sonic_metadata, deepep_topk_to_sonic_metadata_with_scales
    from sonicmoe.functional import attach_preallocated_gated_outputs
    from sonicmoe.quack_utils import quantize_activation_blockscaled_fast as quant
    T, H, I, E, K = 512, 512, 256, 8, 4
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 151)
    idx, scores = masked_routing(T, E, K, 6, 152)
    idx_d, sc_d = idx.to(DEV), scores.to(DEV)
    counts = torch.bincount(idx[idx >= 0].long(), minlength=6).tolist()
    q, raw = quant(x.to(DEV))
    _, words = quant(x.to(DEV), pack_scale_words=True)
    base = deepep_topk_to_sonic_metadata(idx_d, sc_d, counts, 6)
    res = deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw, H)
    assert len(res) == 11
    for a, b in zip(base, res[:10]):
        assert (torch.equal(a, b) if isinstance(a, torch.Tensor) else a == b)
    TKp = res[6]
    want = Q.gather_scales_to_isa(raw.cpu(), base[1].cpu(), H)
    assert torch.equal(res[10].cpu().view(-1), want.view(-1))
    res_w = deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, words, H, gated_output_prototype=q,
                                                      gated_n=2 * I)
    assert len(res_w) == 15 and torch.equal(res_w[10], res[10])
    pre, post, zs, ps = res_w[11:]
    assert pre.dtype == q.dtype and tuple(pre.shape) == (TKp, 2 * I) and tuple(post.shape) == (TKp, I)
    assert zs.dtype == torch.uint8 and tuple(zs.shape) == (TKp, 2 * I // 32)
    assert tuple(ps.shape) == (TKp // 128, 2 * I // 256, 512)
    bf = deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw, H, gated_output_prototype=q,
                                                   gated_n=2 * I, gated_preact_bf16=True,
                                                   gated_allocate_z_scale=False)
    assert bf[11].dtype == torch.bfloat16 and bf[13].numel() == 0
    with pytest.raises(ValueError):
        deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw, H, gated_n=2 * I)
    with pytest.raises(ValueError):
        deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw, H, gated_output_prototype=q, gated_n=384)
    with pytest.raises(ValueError):
        deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw[:-1], H)
    with pytest.raises(ValueError):
        deepep_topk_to_sonic_metadata_with_scales(idx_d, sc_d, counts, 6, raw, H, gated_output_prototype=x.to(DEV),
                                                  gated_n=2 * I)
    # the up-projection writes into the buffers the payload carries
    w1d = w1[:6].contiguous().to(DEV)
    for t in (pre, post, zs, ps):
        t.view(torch.uint8).fill_(0x55)
    payload = (q, raw, attach_preallocated_gated_outputs(res_w[10], (pre, post, zs, ps)))
    holder = torch.empty((), dtype=torch.bfloat16, device=DEV).expand(T, H)
    with sm.enable_fp8(True):
        sm.functional._UpProjection.apply(holder, w1d, None, res_w[0], TKp, K, 0, res_w[1], res_w[2], res_w[3],
                                          res_w[4], True, sm.ActivationType.SWIGLU, True, False, payload, None)
    link = sm.functional._HANDOFF.popitem()[1]
    assert link["z"][0].data_ptr() == pre.data_ptr() and link["y1"][0].data_ptr() == post.data_ptr()
    assert link["z"][1].data_ptr() == zs.data_ptr() and link["y1"][1].data_ptr() == ps.data_ptr()
    with sm.enable_fp8(True):
        sm.functional._UpProjection.apply(holder, w1d, None, res_w[0], TKp, K, 0, res_w[1], res_w[2], res_w[3],
                                          res_w[4], True, sm.ActivationType.SWIGLU, True, False, (q, raw), None)
    ref = sm.functional._HANDOFF.popitem()[1]
    n = int(res_w[0][-1])                               # rows of the experts' segments (the rest is never written)
    assert torch.equal(ref["z"][0][:n], pre.view(torch.uint8)[:n])
    assert torch.equal(ref["y1"][0][:n], post.view(torch.uint8)[:n])
    nb = n // 128 * (I // 128) * 512                    # the ISA scale tiles of those rows
    assert torch.equal(ref["z"][1][:n], zs[:n]) and torch.equal(ref["y1"][1][:nb], ps.view(-1)[:nb])
    torch.cuda.synchronize()
    sm.ops.check_status(DEV)


def test_paired_weight_gradient_launch_changes_no_bit(sm):
    """dw2 folded into dw1's launch (the default when both accumulate into `main_grad` and H is a multiple of 384)
    against the two separate launches: identical main_grad, and the op list shows the one launch."""
    import sonicmoe.functional as Fn
    T, H, I, E, K = 1024, 768, 256, 4, 2
    x, dy, w1, w2, _, _ = make_layer(T, H, I, E, K, 161)
    idx, scores = masked_routing(T, E, K, E, 162)

    def run(pair):
        prev = Fn._PAIR_WGRADS
        Fn._PAIR_WGRADS = pair
        rec = []
        sm.ops.set_recorder(rec)
        try:
            res = _layer_run(sm, x, dy, w1, w2, idx, scores, K, E, None, main_grad=True)
        finally:
            sm.ops.set_recorder(None)
            Fn._PAIR_WGRADS = prev
        return res, [n for n, _, _ in rec]

    base, names_two = run(False)
    got, names_one = run(True)
    assert "gemm_wgrad_pair" in names_one and "gemm_wgrad_pair" not in names_two
    assert names_two.count("gemm_wgrad_mn") == 2 and "gemm_wgrad_mn" not in names_one
    for name, a, b in zip(("out", "dx", "ds", "dw1", "dw2"), base, got):
        assert torch.equal(a, b), name
