"""Generate the committed golden fixtures from the reference's own CPU-loadable code.

Run once in a container that has the reference checkout (read-only):

    python tests/golden/make_golden.py /path/to/reference

It loads, by file path, the two pieces of the reference that import with only
torch + pytest (no Paddle, no GPU):

* tests/ops/conftest.py            gold_e8m0_row_quant / gold_e8m0_col_quant /
                                   gold_e8m0_iso32_quant / gold_dequant /
                                   unpack_isa_scales
* sonicmoe/ernie_compat/deepep_metadata.py
                                   the pure-PyTorch fallback of
                                   deepep_topk_to_sonic_metadata(..., device="cpu")

and stores seeded inputs together with the reference's outputs as small .npz
files next to this script.  The tests never read the reference; they read the
.npz files.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
SEEDS = [42, 123, 777]


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().copy()


def main(ref_root):
    gold = load(os.path.join(ref_root, "tests/ops/conftest.py"), "ref_ops_conftest")

    # ---- quantizers -------------------------------------------------------
    out = {}
    for seed in SEEDS:
        g = torch.Generator().manual_seed(seed)
        for tag, (M, K, scale) in {"unit": (128, 256, 1.0), "small": (64, 128, 1e-3),
                                   "large": (96, 160, 100.0), "wide": (32, 1024, 0.02)}.items():
            x = (torch.randn(M, K, generator=g) * scale).to(torch.bfloat16)
            key = f"s{seed}_{tag}"
            out[key + "_x"] = bf16_bits(x)
            q, s = gold.gold_e8m0_row_quant(x)
            out[key + "_row_q"] = q.view(torch.uint8).numpy()
            out[key + "_row_s"] = s.numpy()
            out[key + "_row_deq"] = bf16_bits(gold.gold_dequant(q, s))
            if M % 32 == 0:
                q, s = gold.gold_e8m0_col_quant(x)
                out[key + "_col_q"] = q.view(torch.uint8).numpy()
                out[key + "_col_s"] = s.numpy()
                q, s = gold.gold_e8m0_iso32_quant(x)
                out[key + "_iso_q"] = q.view(torch.uint8).numpy()
                out[key + "_iso_s"] = s.numpy()
    # ISA layout: random packed buffers, unpacked by the reference helper
    for (rows, cols) in [(128, 128), (256, 384), (200, 96), (384, 3072)]:
        g = torch.Generator().manual_seed(rows * 7 + cols)
        nbytes = -(-rows // 128) * (-(-cols // 128)) * 512
        packed = torch.randint(0, 256, (nbytes,), generator=g, dtype=torch.uint8)
        out[f"isa_{rows}_{cols}_packed"] = packed.numpy()
        out[f"isa_{rows}_{cols}_raw"] = gold.unpack_isa_scales(packed, rows, cols).numpy()
    np.savez_compressed(os.path.join(HERE, "quant_gold.npz"), **out)

    # ---- routing metadata (reference Python fallback, CPU) -----------------
    # The module's package-relative imports are not needed by the fallback;
    # give it an empty parent package so `from . import x` style failures are
    # confined to the optional CUDA extension probes it already guards.
    pkg = types.ModuleType("sonicmoe_ref_stub")
    sys.modules["sonicmoe_ref_stub"] = pkg
    md = load(os.path.join(ref_root, "sonicmoe/ernie_compat/deepep_metadata.py"), "ref_deepep_metadata")
    assert not md._HAS_TOPK_CUDA_KERNEL
    out = {}
    cases = {
        "c0": dict(N=64, K=2, E=8, p_mask=0.0, seed=0),
        "c1": dict(N=300, K=8, E=8, p_mask=0.0, seed=1),
        "c2": dict(N=257, K=8, E=32, p_mask=0.5, seed=2),
        "c3": dict(N=1000, K=4, E=128, p_mask=0.3, seed=3),
        "c4": dict(N=1, K=8, E=16, p_mask=0.0, seed=4),
        "c5": dict(N=128, K=6, E=6, p_mask=0.9, seed=5),
    }
    for name, c in cases.items():
        g = torch.Generator().manual_seed(c["seed"])
        N, K, E = c["N"], c["K"], c["E"]
        scores = torch.rand(N, E, generator=g)
        idx = scores.topk(K, dim=-1).indices.to(torch.int32)   # distinct experts per row
        mask = torch.rand(N, K, generator=g) < c["p_mask"]
        idx = torch.where(mask, torch.full_like(idx, -1), idx)
        probs = torch.rand(N, K, generator=g, dtype=torch.float32)
        tpe = torch.bincount(idx[idx >= 0].long(), minlength=E).tolist()
        res = md.deepep_topk_to_sonic_metadata(idx, probs, tpe, E, device="cpu", block=128)
        efo, xg, ssc, srev, naept, sc, TKp, npad, N_recv, _ = res
        out[name + "_idx"] = idx.numpy()
        out[name + "_probs"] = probs.numpy()
        out[name + "_E"] = np.int64(E)
        for k, v in dict(efo=efo, x_gather_idx=xg, s_scatter_idx=ssc, s_reverse_scatter_idx=srev,
                         naept=naept, topk_scores=sc).items():
            out[f"{name}_{k}"] = v.numpy()
        out[name + "_TKp"] = np.int64(TKp)
    np.savez_compressed(os.path.join(HERE, "routing_gold.npz"), **out)
    print("wrote quant_gold.npz, routing_gold.npz")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of PFCCLab/supersonic-moe>")
    main(sys.argv[1])
