"""Helpers shared by the layer-level parity tests (not a test module).

At the full benchmark sizes the CPU oracle cannot run a whole layer in seconds.  Two constructions carve out of a
full-size problem a small layer whose results must coincide with the corresponding pieces of the full one, for the
fp32 gold AND for the FP8-emulating oracle - i.e. including every quantisation group:

* `block_closure`: for a sample of tokens, every 32-row block (of the expert-sorted order) that holds one of their
  routed rows is taken whole.  Row-wise 1x32 groups live inside a row, the 32x32 blocks of dz and the 32-row column
  groups of the weight-gradient operands are exactly these blocks, and an expert's rows are ordered by token, so in
  the small layer every kept block re-appears with the same 32 rows in the same order.  out, dx and dscores of the
  sampled tokens are therefore those of the full layer.
* `single_expert`: one expert with all the tokens routed to it, in order: its dw1 / dw2 (sums over all its rows)
  are those of the full layer.
"""
import numpy as np
import torch

from oracle import routing as R

COS_MIN, RRMSE_MAX = 0.997, 0.076          # the tolerance the reference publishes for its FP8 path
REPORT = []                                # every gate() call of the session: written out by tests/conftest.py


def stats(got, ref):
    got, ref = got.detach().double().cpu().flatten(), ref.detach().double().cpu().flatten()
    cos = float((got * ref).sum() / (got.norm() * ref.norm()).clamp(min=1e-30))
    rr = float((got - ref).norm() / ref.norm().clamp(min=1e-30))
    return cos, rr


def gate(name, got, gold, emu, strict, report=None):
    """GPU result against the FP8-emulating oracle (cos >= 0.9995, RRMSE <= 3 %) and against the fp32 gold.
    strict: the published bound as it stands (cos >= 0.997, RRMSE <= 7.6 %); otherwise the bound is widened to what
    the emulation of the reference dataflow itself delivers on the same inputs (+3 % / -5e-4), for input
    distributions on which that emulation exceeds the published figure."""
    c_e, r_e = stats(got, emu)
    c_g, r_g = stats(got, gold)
    e_c, e_r = stats(emu, gold)
    REPORT.append((name, "strict" if strict else "emulation-relative", c_g, r_g, e_c, e_r, c_e, r_e))
    if report is not None:
        report.append((name, c_g, r_g, e_c, e_r, c_e, r_e))
    assert c_e >= 0.9995 and r_e <= 0.03, f"{name} vs FP8-emulating oracle: cos {c_e:.5f} rrmse {r_e:.5f}"
    cos_min, rr_max = (COS_MIN, RRMSE_MAX) if strict else (min(COS_MIN, e_c - 5e-4), max(RRMSE_MAX, 1.03 * e_r))
    assert c_g >= cos_min and r_g <= rr_max, (f"{name} vs fp32 gold: cos {c_g:.5f} rrmse {r_g:.5f} "
                                              f"(need {cos_min:.5f} / {rr_max:.5f}; emulation {e_c:.5f} / {e_r:.5f})")


def slot_positions(md, N, K):
    """[N*K] expert-sorted position of every (token, slot), -1 for masked slots."""
    pos = np.full(N * K, -1, dtype=np.int64)
    tk = md["real_TK"]
    pos[md["score_src_idx"][:tk].numpy().astype(np.int64)] = md["s_reverse_scatter_idx"][:tk].numpy().astype(np.int64)
    return pos


def block_closure(idx, scores, md, sample, E):
    """-> (tokens U [n] ascending, idx_mini [n,K] with experts relabelled to 0..E'-1 and dropped slots -1,
    scores_mini [n,K], experts used [E'], rows of U holding the sampled tokens)."""
    N, K = idx.shape
    pos = slot_positions(md, N, K).reshape(N, K)
    blocks = np.unique(pos[sample.numpy()][pos[sample.numpy()] >= 0] // 32)
    keep = (pos >= 0) & np.isin(pos // 32, blocks)
    U = np.nonzero(keep.any(axis=1))[0]
    idx_np = idx.numpy().astype(np.int64)
    used = np.unique(idx_np[keep])
    relabel = np.full(E, -1, dtype=np.int64)
    relabel[used] = np.arange(len(used))
    idx_mini = np.where(keep[U], relabel[np.clip(idx_np[U], 0, E - 1)], -1).astype(np.int32)
    where = np.searchsorted(U, sample.numpy())
    assert (U[where] == sample.numpy()).all()
    return (torch.from_numpy(U), torch.from_numpy(idx_mini), scores[torch.from_numpy(U)].float().contiguous(),
            torch.from_numpy(used), torch.from_numpy(where))


def single_expert(idx, scores, e):
    """-> (tokens routed to expert e, ascending; idx [n,1] zeros; scores [n,1])."""
    hit = (idx == e)
    tok = hit.any(dim=1).nonzero().flatten()
    sc = (scores * hit).sum(dim=1)[tok].float().unsqueeze(1).contiguous()
    return tok, torch.zeros(tok.numel(), 1, dtype=torch.int32), sc


def ds_by_slot(res_ds, md, n, K):
    """token-major ds of an oracle result -> [n, K] (zeros at masked slots)."""
    out = torch.zeros(n * K)
    tk = md["real_TK"]
    out[md["score_src_idx"][:tk].long()] = res_ds[:tk].float()
    return out.view(n, K)


def oracles_on(x, dy, w1, w2, idx, scores, E):
    from oracle import moe as OM
    md = R.topk_metadata(idx, scores, E, 128)
    return md, OM.moe_fp32(x, w1, w2, md, dy), OM.moe_fp8_emulated(x, w1, w2, md, dy)
