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


def quantize_activation_blockscaled_fast(x: torch.Tensor, group_size: int = 32, scale_dtype=None,
                                         pack_scale_words: bool = False):
    """bf16 [M,K] -> (e4m3 [M,K], ue8m0 scales) (blockscaled_fp8_gemm.py:518-596).  Scales: u8 [M,K/32] by default;
    `pack_scale_words`: int32 [M,K/128], four scale bytes per word (the compact form an FP8 dispatch transports);
    `scale_dtype=torch.int32`: int32 [M,K/32], one word per group."""
    if group_size != 32:
        raise NotImplementedError("1x32 groups only")
    want_i32 = str(scale_dtype) in ("torch.int32", "int32")
    if pack_scale_words and want_i32:
        raise ValueError("pack_scale_words and an explicit int32 scale_dtype are mutually exclusive")
    q, raw, _ = ops.quant_rows(x.contiguous(), raw=True, isa=False)
    if pack_scale_words:
        if raw.shape[1] % 4:
            raise ValueError(f"pack_scale_words requires the number of 1x32 groups to be divisible by 4, got "
                             f"{raw.shape[1]} for K={x.shape[1]}")
        raw = raw.view(torch.int32)
    elif want_i32:
        raw = raw.to(torch.int32)
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
