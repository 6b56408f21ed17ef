"""Quantizer entry points under the reference's names
(sonicmoe/quack_utils/__init__.py:30-60, blockscaled_fp8_gemm.py)."""
from __future__ import annotations

import torch

from .. import ops

SF_TILE_M, SF_TILE_K, SF_TILE_STORAGE, SF_VEC_SIZE = 128, 128, 512, 32


def quantize_and_pack_activation(x: torch.Tensor):
    """bf16 [M,K] -> (e4m3 [M,K], ISA-packed ue8m0 scales) (blockscaled_fp8_gemm.py:3214-3283)."""
    q, _, isa = ops.quant_rows(x.contiguous(), raw=False, isa=True)
    return q.view(torch.float8_e4m3fn), isa


def quantize_activation_blockscaled_fast(x: torch.Tensor):
    """bf16 [M,K] -> (e4m3 [M,K], raw ue8m0 scales [M,K/32]) (blockscaled_fp8_gemm.py:518-596)."""
    q, raw, _ = ops.quant_rows(x.contiguous(), raw=True, isa=False)
    return q.view(torch.float8_e4m3fn), raw


def pack_blockscaled_1x32_scales(raw: torch.Tensor, cols: int):
    """raw [rows, cols/32] u8 -> ISA layout (blockscaled_fp8_gemm.py:225-245)."""
    return ops.gather_scales_isa(raw.contiguous(), None, raw.shape[0], cols)


def colwise_quantize_and_pack(src: torch.Tensor, rows: int, gather_idx: torch.Tensor | None = None):
    """Column-wise 1x32 of src[gather_idx]; returns (e4m3 TRANSPOSED [dim, rows], ISA scales for (dim, rows))."""
    q_t, isa = ops.quant_cols_t(src.contiguous(), gather_idx, rows)
    return q_t.view(torch.float8_e4m3fn), isa


def dual_quantize_iso32(x: torch.Tensor):
    """32x32-block quantizer: (q [rows,cols], row ISA, q_t [cols,rows], col ISA) (blockscaled_fp8_gemm.py:2052-2198)."""
    q, ri, q_t, ci = ops.quant_iso32(x.contiguous())
    return q.view(torch.float8_e4m3fn), ri, q_t.view(torch.float8_e4m3fn), ci
