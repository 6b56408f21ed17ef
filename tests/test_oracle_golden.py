"""The oracle against the reference's own goldens (fixtures made by
tests/golden/make_golden.py from the reference's tests/ops/conftest.py gold
functions and the Python fallback of deepep_topk_to_sonic_metadata)."""
import os

import numpy as np
import pytest
import torch

from oracle import quant as Q
from oracle import routing as R

SEEDS = [42, 123, 777]
TAGS = ["unit", "small", "large", "wide"]


@pytest.fixture(scope="module")
def qgold(golden_dir):
    return np.load(os.path.join(golden_dir, "quant_gold.npz"))


@pytest.fixture(scope="module")
def rgold(golden_dir):
    return np.load(os.path.join(golden_dir, "routing_gold.npz"))


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


@pytest.mark.parametrize("seed", SEEDS)
@pytest.mark.parametrize("tag", TAGS)
def test_row_quant_matches_reference_gold(qgold, seed, tag):
    k = f"s{seed}_{tag}"
    x = _bf16(qgold[k + "_x"])
    q, s = Q.row_quant(x)
    assert np.array_equal(q.numpy(), qgold[k + "_row_q"])
    assert np.array_equal(s.numpy(), qgold[k + "_row_s"])
    deq = Q.dequant_rows(q, s).to(torch.bfloat16)
    assert np.array_equal(deq.view(torch.int16).numpy(), qgold[k + "_row_deq"])


@pytest.mark.parametrize("seed", SEEDS)
@pytest.mark.parametrize("tag", ["unit", "small", "large", "wide"])
def test_col_and_iso_quant_match_reference_gold(qgold, seed, tag):
    k = f"s{seed}_{tag}"
    if k + "_col_q" not in qgold:
        pytest.skip("rows not a multiple of 32")
    x = _bf16(qgold[k + "_x"])
    q, s = Q.col_quant(x)
    assert np.array_equal(q.numpy(), qgold[k + "_col_q"])
    assert np.array_equal(s.numpy(), qgold[k + "_col_s"])
    q, bs = Q.iso32_quant(x)
    assert np.array_equal(q.numpy(), qgold[k + "_iso_q"])
    assert np.array_equal(bs.repeat_interleave(32, dim=0).numpy(), qgold[k + "_iso_s"])


@pytest.mark.parametrize("rows,cols", [(128, 128), (256, 384), (200, 96), (384, 3072)])
def test_isa_layout_matches_reference_unpack(qgold, rows, cols):
    packed = torch.from_numpy(qgold[f"isa_{rows}_{cols}_packed"])
    raw = Q.unpack_isa(packed, rows, cols)
    assert np.array_equal(raw.numpy(), qgold[f"isa_{rows}_{cols}_raw"])
    repacked = Q.pack_isa(raw, rows, cols, fill=0)
    idx = Q.isa_index(rows, cols).reshape(-1)
    assert torch.equal(repacked[idx], packed[idx])


def test_e4m3_cast_pinned_by_bit_level_encoder():
    g = torch.Generator().manual_seed(0)
    v = torch.cat([torch.randn(20000, generator=g) * s for s in (1e-3, 0.05, 1.0, 30.0, 400.0)])
    v = torch.cat([v, torch.tensor([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 1000.0, -1e9, 2.0 ** -9, 2.0 ** -10,
                                    1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9, 2.0 ** -6, 0.0175, 17.0, 18.0, 19.0])])
    a = Q.f32_to_e4m3_bytes(v).numpy()
    b = Q.f32_to_e4m3_bytes_bitwise(v.numpy())
    # -0.0 keeps its sign in both
    assert np.array_equal(a, b)


def test_zero_group_and_floor_rules():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    x[1, 3] = 1.0
    q, s = Q.row_quant(x)
    assert s[0, 0] == 0 and s[0, 1] == 0 and s[1, 0] == 119 and q[0].sum() == 0   # 1.0 -> 2^-8 scale
    q, s = Q.row_quant(x, amax_floor=1e-4)
    # 1e-4 = 1.6384 * 2^-14 -> bexp 113, mantissa < 0.75 -> 113 - 8 = 105
    assert s[0, 0] == 105
    # carry threshold: amax = 1.75 * 2^k stays, just above carries
    x = torch.tensor([[1.75] + [0.0] * 31, [1.875] + [0.0] * 31], dtype=torch.bfloat16)
    _, s = Q.row_quant(x)
    assert s[0, 0] == 119 and s[1, 0] == 120


@pytest.mark.parametrize("case", ["c0", "c1", "c2", "c3", "c4", "c5"])
def test_routing_matches_reference_python_fallback(rgold, case):
    idx = torch.from_numpy(rgold[case + "_idx"])
    probs = torch.from_numpy(rgold[case + "_probs"])
    E = int(rgold[case + "_E"])
    md = R.topk_metadata(idx, probs, E, 128, lane_order="slot", pad_mode="virtual")
    assert md["real_TKp"] == int(rgold[case + "_TKp"])
    for k in ["efo", "x_gather_idx", "s_scatter_idx", "s_reverse_scatter_idx", "naept", "topk_scores"]:
        assert np.array_equal(md[k].numpy(), rgold[f"{case}_{k}"]), k
    # the CUDA-kernel flavour differs only in lane order inside a token and pad sentinel
    md2 = R.topk_metadata(idx, probs, E, 128)
    for k in ["efo", "x_gather_idx", "naept"]:
        assert torch.equal(md2[k], md[k])
    tk = md["real_TK"]
    assert torch.equal(md2["topk_scores"][md2["s_scatter_idx"].long()][md2["s_reverse_scatter_idx"].long()],
                       md2["topk_scores"][:tk])
