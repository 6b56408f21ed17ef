"""CPU restatement of the reference's MoE layer forward + backward.

TEST INFRASTRUCTURE ONLY - never imported by the product path (bench.py's
`cpu_baseline` leg and the tests are the only callers).

Three restatements, each on CPU torch tensors:

* `router_topk_softmax` / `router_backward`
      sonicmoe/moe.py:664-677,764-770 (top-k on logits, fp32 softmax over the K
      selected logits), sonicmoe/functional/backward.py:572-641 (Jacobian).
* `moe_fp32`   explicit fp32 forward/backward with interleaved gate/up rows,
      tests/ops/test_moe_module.py:121-349 (gold fwd/bwd formulas),
      sonicmoe/moe.py:40-43,739-758 (expert math).
* `moe_fp8_emulated`  the FP8 frontier dataflow with every quantizer applied
      exactly where the reference applies it, GEMMs done as
      dequantise -> fp32 matmul: sonicmoe/quack_utils/sm100_funcs.py:207-455
      (up-proj + SwiGLU + z/y1 quant), :784-807 (down-proj), :824-885 (dgated),
      :894-976 (wgrad operand quant + wgrad), sonicmoe/functional/__init__.py
      :1429-1437 (dgrad), sonicmoe/functional/reduction_over_k_gather.py:99-196
      (combine, ascending lane order, fp32 accumulate, bf16 store).
* `TorchMoEBaseline`  the reference's pure-PyTorch backend
      (KernelBackendMoE.torch, sonicmoe/moe.py:739-758 + router :664-677 +
      bincount :696-697) restated without Paddle; this is the timed CPU baseline.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import quant as Q


# ----------------------------------------------------------------------------
# router
# ----------------------------------------------------------------------------
def router_topk_softmax(logits: torch.Tensor, K: int):
    """top-K on logits (descending), softmax over the K values in fp32.  Ties (frequent when the logits
    come out of a bf16 linear) go to the lower expert index - torch.topk leaves that unspecified, a stable
    descending sort pins it."""
    vals, idx = torch.sort(logits.float(), dim=-1, descending=True, stable=True)
    vals, idx = vals[:, :K], idx[:, :K]
    return F.softmax(vals, dim=-1, dtype=torch.float32), idx.to(torch.int32)


def router_backward(scores: torch.Tensor, idx: torch.Tensor, dscores: torch.Tensor, E: int):
    """dlogit[t, idx[t,k]] = s_k * (g_k - sum_j g_j s_j), zeros elsewhere."""
    dot = (dscores * scores).sum(dim=-1, keepdim=True)
    d = scores * (dscores - dot)
    out = torch.zeros(scores.shape[0], E, dtype=torch.float32)
    out.scatter_(1, idx.long(), d)
    return out


# ----------------------------------------------------------------------------
# expert math helpers (interleaved layout: even rows of w1[e] = gate, odd = up)
# ----------------------------------------------------------------------------
GELU_C0, GELU_C1 = 0.7978845608028654, 0.044715        # sqrt(2/pi); the tanh approximation of GELU


def swiglu(z: torch.Tensor) -> torch.Tensor:
    g, u = z[..., 0::2], z[..., 1::2]
    sig = 1.0 / (1.0 + torch.exp(-g))
    return (g * sig) * u


def glu(z: torch.Tensor, act: str = "swiglu") -> torch.Tensor:
    """act(gate) * up on interleaved columns: swiglu, reglu = relu(g)*u, geglu = gelu_tanh(g)*u
    (the reference maps the names to quack.activation.swiglu / reglu / geglu, quack_utils/gemm_gated.py:171-177)."""
    if act == "swiglu":
        return swiglu(z)
    g, u = z[..., 0::2], z[..., 1::2]
    if act == "reglu":
        return torch.relu(g) * u
    if act == "geglu":
        return (0.5 * g * (1.0 + torch.tanh(GELU_C0 * (g + GELU_C1 * g ** 3)))) * u
    raise ValueError(act)


def dglu(z: torch.Tensor, dy: torch.Tensor, act: str = "swiglu"):
    """-> (dz interleaved, y = act(g)*u) for upstream dy with respect to y."""
    if act == "swiglu":
        return dswiglu(z, dy)
    g, u = z[..., 0::2], z[..., 1::2]
    if act == "reglu":
        a, da = torch.relu(g), (g > 0).to(z.dtype)
    elif act == "geglu":
        t = torch.tanh(GELU_C0 * (g + GELU_C1 * g ** 3))
        a = 0.5 * g * (1.0 + t)
        da = 0.5 * (1.0 + t) + 0.5 * g * (1.0 - t * t) * GELU_C0 * (1.0 + 3.0 * GELU_C1 * g * g)
    else:
        raise ValueError(act)
    dz = torch.stack([da * u * dy, a * dy], dim=-1).reshape(z.shape)
    return dz, a * u


def dswiglu(z: torch.Tensor, dy: torch.Tensor):
    """quack dswiglu_precise expression order (_gated_epilogues.py:442-457):
    returns (dz interleaved, y)."""
    g, u = z[..., 0::2], z[..., 1::2]
    sig = 1.0 / (1.0 + torch.exp(-g))
    silu = g * sig
    sd = silu * dy
    dg = ((sig - silu * sig) * dy + sd) * u
    dz = torch.stack([dg, sd], dim=-1).reshape(z.shape)
    return dz, silu * u


def _segments(efo):
    efo = efo.tolist()
    return [(e, efo[e], efo[e + 1]) for e in range(len(efo) - 1) if efo[e + 1] > efo[e]]


def combine(y2: torch.Tensor, md: dict, N: int, weighted: bool) -> torch.Tensor:
    """o[t] = sum_j w_j * y2[s_rev[naept[t]+j]], ascending j, fp32 accumulate."""
    naept = md["naept"].long()
    s_rev = md["s_reverse_scatter_idx"].long()
    scores = md["topk_scores"]
    H = y2.shape[1]
    out = torch.zeros(N, H, dtype=torch.float32)
    kmax = int((naept[1:] - naept[:-1]).max()) if N > 0 else 0
    for j in range(kmax):
        has = (naept[:-1] + j) < naept[1:]
        tm = (naept[:-1] + j)[has]
        rows = y2[s_rev[tm]].float()
        if weighted:
            rows = rows * scores[tm].unsqueeze(1)
        out[has] = out[has] + rows
    return out


# ----------------------------------------------------------------------------
# fp32 gold
# ----------------------------------------------------------------------------
def moe_fp32(x, w1, w2, md: dict, dy=None, act: str = "swiglu"):
    """x [N,H], w1 [E,2I,H], w2 [E,H,I] (any float dtype, promoted to fp32),
    md = oracle.routing.topk_metadata(...).  Returns dict(o, and with dy: dx, dw1,
    dw2, ds (token-major, length TK))."""
    x, w1, w2 = x.float(), w1.float(), w2.float()
    N, H = x.shape
    E, I2, _ = w1.shape
    efo, xg = md["efo"], md["x_gather_idx"].long()
    s = md["topk_scores"][md["s_scatter_idx"].long()]
    TKp = xg.shape[0]
    z = torch.zeros(TKp, I2)
    y2 = torch.zeros(TKp, H)
    for e, a, b in _segments(efo):
        z[a:b] = x[xg[a:b]] @ w1[e].T
    y1 = glu(z, act)
    for e, a, b in _segments(efo):
        y2[a:b] = y1[a:b] @ w2[e].T
    out = dict(o=combine(y2, md, N, True), z=z, y1=y1, y2=y2)
    if dy is None:
        return out
    dy = dy.float()
    dout = dy[xg]
    D = torch.zeros(TKp, I2 // 2)
    for e, a, b in _segments(efo):
        D[a:b] = dout[a:b] @ w2[e]
    dz, y = dglu(z, s.unsqueeze(1) * D, act)
    ds_row = (y * D).sum(dim=1)
    y1s = s.unsqueeze(1) * y
    dw1 = torch.zeros_like(w1)
    dw2 = torch.zeros(E, I2 // 2, H)
    dx_exp = torch.zeros(TKp, H)
    for e, a, b in _segments(efo):
        dw2[e] = y1s[a:b].T @ dout[a:b]
        dw1[e] = dz[a:b].T @ x[xg[a:b]]
        dx_exp[a:b] = dz[a:b] @ w1[e]
    out.update(dx=combine(dx_exp, md, N, False), dw1=dw1, dw2=dw2.transpose(1, 2).contiguous(),
               dw2_IH=dw2, ds=ds_row[md["s_reverse_scatter_idx"].long()], dz=dz, y1s=y1s, D=D)
    return out


# ----------------------------------------------------------------------------
# FP8 frontier dataflow, emulated
# ----------------------------------------------------------------------------
def quantize_weights(w1, w2, iso32: bool = False):
    """Four row-wise 1x32 layouts (blockscaled_fp8_gemm.py:4363-4406):
    W1 (E,2I,H) scales along H; W1T (E,H,2I) along 2I; W2 (E,H,I) along I;
    W2T (E,I,H) along H.  Returns dict name -> (bytes, raw scales), flattened over E.
    `iso32`: one scale per 32x32 block and ONE payload per weight, its transpose being the byte transpose
    (blockscaled_fp8_gemm.py:3765-3856); expressed here in the same (bytes, 1x32 raw scales) form."""
    if iso32:
        def iq(w):
            E, N, K = w.shape
            q, s = Q.iso32_quant(w.reshape(E * N, K))                    # s: [E*N/32, K/32]
            q, s = q.reshape(E, N, K), s.reshape(E, N // 32, K // 32)
            rows = s.repeat_interleave(32, dim=1)                        # [E, N, K/32]
            cols = s.transpose(1, 2).repeat_interleave(32, dim=1)        # [E, K, N/32]
            return (q, rows.contiguous()), (q.transpose(1, 2).contiguous(), cols.contiguous())
        (a, at), (b, bt) = iq(w1), iq(w2)
        return dict(w1=a, w1t=at, w2=b, w2t=bt)

    def rq(w):
        E, N, K = w.shape
        q, s = Q.row_quant(w.reshape(E * N, K))
        return q.reshape(E, N, K), s.reshape(E, N, K // 32)
    return dict(w1=rq(w1), w1t=rq(w1.transpose(1, 2).contiguous()),
                w2=rq(w2), w2t=rq(w2.transpose(1, 2).contiguous()))


def _deq_w(qs):
    q, s = qs
    E, N, K = q.shape
    return Q.dequant_rows(q.reshape(E * N, K), s.reshape(E * N, K // 32)).reshape(E, N, K)


def moe_fp8_emulated(x, w1, w2, md: dict, dy=None, y1_bf16_rne: bool = True, act: str = "swiglu",
                     iso32_weight: bool = False):
    """x, dy bf16 [N,H]; w1 [E,2I,H], w2 [E,H,I] bf16.  All outputs of the FP8 path
    plus every quantised intermediate (bytes and scale bytes)."""
    N, H = x.shape
    E, I2, _ = w1.shape
    I = I2 // 2
    efo, xg = md["efo"], md["x_gather_idx"].long()
    TKp = xg.shape[0]
    s = md["topk_scores"][md["s_scatter_idx"].long()]
    wq = quantize_weights(w1, w2, iso32_weight)
    W1, W1T, W2, W2T = (_deq_w(wq[k]) for k in ("w1", "w1t", "w2", "w2t"))
    r = dict(wq=wq)

    # forward ---------------------------------------------------------------
    xq, xs = Q.row_quant(x)
    xd = Q.dequant_rows(xq, xs)
    z = torch.zeros(TKp, I2)
    for e, a, b in _segments(efo):
        z[a:b] = xd[xg[a:b]] @ W1[e].T
    y1 = glu(z, act)
    if y1_bf16_rne:
        y1 = Q.bf16_rne(y1)
    zq, zs = Q.row_quant(z, amax_floor=1e-4)
    y1q, y1s_ = Q.row_quant(y1)
    y1d = Q.dequant_rows(y1q, y1s_)
    y2 = torch.zeros(TKp, H)
    for e, a, b in _segments(efo):
        y2[a:b] = y1d[a:b] @ W2[e].T
    y2 = y2.to(torch.bfloat16)
    o = combine(y2, md, N, True).to(torch.bfloat16)
    r.update(x_fp8=xq, x_scales=xs, z_acc=z, z_fp8=zq, z_scales=zs, y1_fp8=y1q, y1_scales=y1s_,
             y2=y2, o=o)
    if dy is None:
        return r

    # backward --------------------------------------------------------------
    dq, dsc = Q.row_quant(dy)
    dd = Q.dequant_rows(dq, dsc)
    D = torch.zeros(TKp, I)
    for e, a, b in _segments(efo):
        D[a:b] = dd[xg[a:b]] @ W2T[e].T
    zd = Q.dequant_rows(zq, zs)
    dz, y = dglu(zd, s.unsqueeze(1) * D, act)
    ds_row = (y * D).sum(dim=1)
    y1s = (s.unsqueeze(1) * y).to(torch.bfloat16)
    dz = dz.to(torch.bfloat16)
    # wgrad / dgrad operands
    y1s_q, y1s_cs = Q.col_quant(y1s)
    dz_q, dz_bs = Q.iso32_quant(dz)
    dout_q, dout_cs = Q.col_quant(dy, md["x_gather_idx"])
    x_q, x_cs = Q.col_quant(x, md["x_gather_idx"])
    y1s_d = Q.dequant_cols(y1s_q, y1s_cs)
    dout_d = Q.dequant_cols(dout_q, dout_cs)
    x_d = Q.dequant_cols(x_q, x_cs)
    dz_rs = dz_bs.repeat_interleave(32, dim=0)            # row scales (TKp, 2I/32)
    dz_d = Q.dequant_rows(dz_q, dz_rs)
    dw1 = torch.zeros(E, I2, H)
    dw2 = torch.zeros(E, I, H)
    dx_exp = torch.zeros(TKp, H)
    for e, a, b in _segments(efo):
        dw2[e] = y1s_d[a:b].T @ dout_d[a:b]
        dw1[e] = dz_d[a:b].T @ x_d[a:b]
        dx_exp[a:b] = dz_d[a:b] @ W1T[e].T
    dx_exp = dx_exp.to(torch.bfloat16)
    dx = combine(dx_exp, md, N, False).to(torch.bfloat16)
    r.update(dout_fp8=dq, dout_scales=dsc, D=D, dz=dz, y1s=y1s, ds_row=ds_row,
             ds=ds_row[md["s_reverse_scatter_idx"].long()],
             y1s_col=(y1s_q, y1s_cs), dz_iso=(dz_q, dz_bs), dout_col=(dout_q, dout_cs), x_col=(x_q, x_cs),
             dw1=dw1, dw2_IH=dw2, dx_exp=dx_exp, dx=dx)
    return r


# ----------------------------------------------------------------------------
# the reference's pure-PyTorch backend (timed CPU baseline)
# ----------------------------------------------------------------------------
class TorchMoEBaseline(torch.nn.Module):
    """router Linear(H->E) -> top-k -> softmax over the K logits -> sort by
    expert -> per-expert F.linear / interleaved SwiGLU / F.linear -> gate multiply
    -> fp32 index_add (sonicmoe/moe.py:664-677,739-758)."""

    def __init__(self, E, K, H, I, std=0.02, dtype=torch.bfloat16, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.E, self.K, self.H, self.I = E, K, H, I
        self.router = torch.nn.Parameter((torch.randn(E, H, generator=g) * std).to(dtype))
        self.w1 = torch.nn.Parameter((torch.randn(E, 2 * I, H, generator=g) * std).to(dtype))
        self.w2 = torch.nn.Parameter((torch.randn(E, H, I, generator=g) * std).to(dtype))

    def experts_only(self, x, sel, gates):
        """The expert compute on pre-routed inputs (sel [T,K] expert ids, gates [T,K]): the region the reference's
        own benchmark times; the router linear / top-k stay outside."""
        return self._experts(x, sel.flatten().long(), gates.type_as(x))

    def forward(self, x):
        logits = F.linear(x, self.router)
        vals, sel = logits.topk(self.K, dim=-1)
        gates = F.softmax(vals.float(), dim=-1).type_as(x)
        return self._experts(x, sel.flatten(), gates), logits

    def _experts(self, x, sel, gates):
        T = x.shape[0]
        with torch.no_grad():
            _, order = sel.sort(stable=True)
            freq = sel.bincount(minlength=self.E)
        fan_in = order // self.K
        batch_gates = gates.flatten()[order]
        h = x[fan_in].split(freq.tolist(), dim=0)
        h = [F.linear(h[e], self.w1[e]) for e in range(self.E)]
        h = [t[..., 1::2] * F.silu(t[..., ::2]) for t in h]
        h = torch.cat([F.linear(h[e], self.w2[e]) for e in range(self.E)], dim=0)
        h = h * batch_gates.unsqueeze(-1)
        out = torch.zeros(T, self.H, dtype=torch.float32).index_add(0, fan_in, h.float())
        return out.to(x.dtype)
