"""The C-ABI library loads and exports every symbol include/smoe_b200.h declares (no compute calls: no GPU here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "smoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(smoe_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path_entry_points():
    syms = declared_symbols()
    for must in ("smoe_topk_metadata", "smoe_count_cumsum", "smoe_quant_rows", "smoe_quant_cols_t", "smoe_quant_iso32",
                 "smoe_gemm_gated", "smoe_gemm_varlen_m", "smoe_gemm_dgated", "smoe_gemm_wgrad", "smoe_combine"):
        assert must in syms


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol(built_library):
    from sonicmoe import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_host_side_argument_checks(built_library):
    """Shape / argument errors are reported by return code before anything touches a device."""
    from sonicmoe._lib import lib
    assert lib.smoe_quant_rows(None, 4, 48, None, None, None, None) == 1          # K % 32
    assert lib.smoe_gemm_varlen_m(None, None, None, None, None, None, 100, 128, 128, 1, None, None) == 1
    assert lib.smoe_gemm_gated(None, 1, None, None, None, None, None, None, None, None, None, 128, 128, 128, 1, None,
                               None) == 1                                           # N % 256
    assert lib.smoe_topk_metadata(None, None, 4, 17, 8, 128, 0, 0, 0, 0, None, None, None, None, None, None, None,
                                  None, None, None) == 1                            # top-k > 16
    assert lib.smoe_topk_metadata_workspace(64, 8) > 0
    assert lib.smoe_combine(None, None, None, None, None, 4, 12, None) == 1        # H % 8
