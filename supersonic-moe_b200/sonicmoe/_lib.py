"""ctypes binding of libsmoe_b200.so (the C ABI declared in include/smoe_b200.h).

There is no fallback: if the library is missing or a symbol cannot be resolved
the import of this module raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsmoe_b200.so")

_P, _I, _L = c_void_p, c_int, c_int64

# name -> (restype, argtypes); mirrors include/smoe_b200.h one to one
SIGNATURES = {
    "smoe_count_cumsum": (_I, [_P, _I, _L, _L, _P, _P, _P]),
    "smoe_topk_metadata_workspace": (_L, [_L, _L]),
    "smoe_topk_metadata": (_I, [_P, _P, _L, _L, _L, _L, _L, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "smoe_topk_metadata_static": (_I, [_P, _P, _L, _L, _L, _L, _L, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "smoe_topk_metadata_static_capacity": (_L, []),
    "smoe_ep_plan_dest": (_I, [_P, _L, _L, _L, _L, _P, _P, _P]),
    "smoe_ep_plan_send_idx": (_I, [_P, _P, _P, _L, _L, _L, _L, _P, _P, _P]),
    "smoe_ep_combine_pull": (_I, [_P, _P, _P, _L, _P, _P, _P, _P, _L, _L, _P]),
    "smoe_ep_tables_bytes": (_L, []),
    "smoe_ep_tables": (_I, [_P, _L, _L, _L, _L, _P, _P]),
    "smoe_ep_dispatch_pull_dev": (_I, [_P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P]),
    "smoe_ep_combine_pull_dev": (_I, [_P, _P, _L, _P, _P, _P, _P, _L, _L, _P]),
    "smoe_ep_dispatch_pull": (_I, [_P, _P, _P, _L, _L, _L, _L, _L, _L, _L, _L, _L, _P, _P, _P, _P, _P]),
    "smoe_quant_rows": (_I, [_P, _L, _L, _P, _P, _P, _P]),
    "smoe_quant_rows_gather": (_I, [_P, _P, _P, _L, _L, _P, _P, _P]),
    "smoe_quant_dual_gather": (_I, [_P, _P, _P, _L, _L, _P, _P, _P, _P, _P]),
    "smoe_quant_rows_scatter": (_I, [_P, _L, _L, _P, _P, _P, _P, _L, _P, _P, _P]),
    "smoe_gather_scales_isa": (_I, [_P, _P, _L, _L, _P, _P]),
    "smoe_gather_rows_fp8": (_I, [_P, _P, _P, _P, _L, _L, _P, _P, _P]),
    "smoe_scatter_rows_fp8": (_I, [_P, _P, _L, _L, _P, _P, _P, _P, _L, _P, _P, _P]),
    "smoe_quant_cols_t": (_I, [_P, _P, _P, _L, _L, _P, _P, _P]),
    "smoe_requant_cols_t": (_I, [_P, _P, _P, _P, _L, _L, _P, _P, _P]),
    "smoe_quant_iso32": (_I, [_P, _L, _L, _P, _P, _P, _P, _P]),
    "smoe_gemm_varlen_m": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "smoe_gemm_varlen_m_bt": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "smoe_transpose_u8": (_I, [_P, _L, _L, _L, _P, _P]),
    "smoe_gemm_gated": (_I, [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "smoe_gemm_dgated": (_I, [_P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _P, _P]),
    "smoe_gemm_dgated_partials": (_L, [_L]),
    "smoe_gemm_dgated_fused": (_I, [_P] * 14 + [_L, _L, _L, _L, _P, _P]),
    "smoe_gemm_dgated_fused_partials": (_L, [_L]),
    "smoe_gemm_dgated_fused_gather": (_I, [_P, _L, _P] + [_P] * 13 + [_L, _L, _L, _L, _P, _P]),
    "smoe_gemm_wgrad": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _P, _P]),
    "smoe_gemm_wgrad_mn": (_I, [_P, _P, _P, _P, _P, _P, _L, _L, _L, _L, _I, _I, _P, _P]),
    "smoe_gemm_wgrad_mn_pair": (_I, [_P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _L, _P, _L, _L, _L, _I, _I, _P, _P]),
    "smoe_glu_fwd": (_I, [_P, _L, _L, _I, _P, _P, _P, _P, _P]),
    "smoe_glu_bwd": (_I, [_P, _P, _P, _P, _L, _L, _I, _P, _P, _P, _P]),
    "smoe_combine": (_I, [_P, _P, _P, _P, _P, _L, _L, _P]),
    "smoe_gather_scores": (_I, [_P, _P, _L, _P, _P]),
    "smoe_ds_finalize": (_I, [_P, _L, _L, _P, _L, _P, _P, _P, _P, _P]),
    "smoe_status_post": (_I, [_P, _P, _P]),
    "smoe_topk_softmax": (_I, [_P, _L, _L, _L, _P, _P, _P]),
    "smoe_topk_softmax_bwd": (_I, [_P, _P, _P, _L, _L, _L, _P, _P]),
}

# exported for the library's own tests and timing experiments only (csrc/smoe_internal.h); not product ABI
INTERNAL_SIGNATURES = {
    "smoe_internal_gemm_knobs": (_I, [_I]),
    "smoe_internal_gemm_trace": (_I, [_P]),
}

ERRORS = {1: "SMOE_ERR_SHAPE", 2: "SMOE_ERR_ALIGN", 3: "SMOE_ERR_DRIVER", 4: "SMOE_ERR_TMAP", 5: "SMOE_ERR_LAUNCH",
          6: "SMOE_ERR_ARG"}


class SmoeError(RuntimeError):
    pass


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python supersonic-moe_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the MoE kernels)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in {**SIGNATURES, **INTERNAL_SIGNATURES}.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int, what: str):
    if rc != 0:
        raise SmoeError(f"{what} failed: {ERRORS.get(rc, rc)}")
