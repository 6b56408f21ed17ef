"""Host-side arithmetic of bench.py: the FLOPs it credits to each GEMM call of the step, the DRAM traffic it reads
from the committed ncu summary, and the fraction it reports (no GPU needed)."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_roofline_flops_traffic_and_fraction(bench):
    cfg = bench.CONFIGS["C2"]
    T, K, H, I = cfg["T"], cfg["K"], cfg["H"], cfg["I"]
    unit = float(T) * K * H * I
    pk = {"bf16": 1650.0, "bf16_sustained": 1400.0, "source": "test"}
    order = ["topk_metadata#0", "gemm_gated#2", "gemm_varlen_m#3", "gemm_dgated_fused#8", "gemm_varlen_m#9",
             "gemm_wgrad_pair#12"]
    us = {"topk_metadata#0": 25.0, "gemm_gated#2": 450.0, "gemm_varlen_m#3": 255.0, "gemm_dgated_fused#8": 330.0,
          "gemm_varlen_m#9": 440.0, "gemm_wgrad_pair#12": 690.0}
    r = bench._roofline("C2", 1, T, K, H, I, order, us, pk)
    # the slowest GEMM call is the paired weight-gradient launch: dw1 (4) + dw2 (2) units of T*K*H*I
    assert r["kernel"] == "gemm_wgrad_pair#12" and r["bound"] == "tensor"
    want = 6 * unit / 690e-6 / 1e12
    assert abs(r["achieved"] - want) < 0.1
    assert abs(r["frac"] - want / 3300.0) < 1e-3 and abs(r["frac_of_sustained_peak"] - want / 2800.0) < 1e-3
    table = bench.ncu_dram_bytes("C2")
    assert table is not None, "profiles/gemm_dram_traffic_c2.json is part of the repository"
    assert r["traffic"] == table["gemm_wgrad_mn#0"] + table["gemm_wgrad_mn#1"]
    # with the two weight gradients launched separately the second (dw1, 4 units) dominates
    order2 = order[:-1] + ["gemm_wgrad_mn#11", "gemm_wgrad_mn#13"]
    us2 = dict(us, **{"gemm_wgrad_mn#11": 260.0, "gemm_wgrad_mn#13": 480.0})
    del us2["gemm_wgrad_pair#12"]
    r2 = bench._roofline("C2", 1, T, K, H, I, order2, us2, pk)
    assert r2["kernel"] == "gemm_wgrad_mn#13"
    assert abs(r2["achieved"] - 4 * unit / 480e-6 / 1e12) < 0.1 and r2["traffic"] == table["gemm_wgrad_mn#1"]
    # several ranks: no single-GPU traffic figure applies
    assert bench._roofline("C2", 8, T, K, H, I, order, us, pk)["traffic"] is None


def test_configs_and_published_baseline(bench):
    c2 = bench.CONFIGS["C2"]
    assert (c2["T"], c2["H"], c2["I"], c2["E"], c2["K"]) == (8192, 3072, 1536, 8, 8)
    assert abs(bench.PUBLISHED_US["C2"] - 2659.8) < 1e-6
    for name in ("C3", "C4", "C5"):
        assert name in bench.CONFIGS
