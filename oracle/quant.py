"""CPU restatement of the reference's MXFP8 1x32 ue8m0 block-scaled quantizers.

TEST INFRASTRUCTURE ONLY.  Nothing on the product path may import this module;
it is the checker the CUDA kernels are compared against.

Every function works on CPU torch tensors and is written as plain vectorised
integer / float arithmetic so that it can be read next to the reference:

* E8M0 rule (amax -> scale byte -> quant scale):
  sonicmoe/quack_utils/blockscaled_fp8_gemm.py:487-499 (general form),
  :3043-3056 (simplified form), sonicmoe/quack_utils/_gated_epilogues.py:977-1028
  (epilogue form with the 1e-4 amax floor used only for z).
* Row-wise kernels: blockscaled_fp8_gemm.py:446-515 (raw scales),
  :2992-3068 (ISA-packed scales).
* Column-wise kernel: blockscaled_fp8_gemm.py:1517-1592.
* 32x32 "iso32" kernel: blockscaled_fp8_gemm.py:2052-2148.
* ISA scale layout: blockscaled_fp8_gemm.py:104-107,225-245;
  tests/ops/conftest.py:231-259 (unpack).

The reference kernels are canonical where they differ from the reference's
torch gold (tests/ops/conftest.py:99-114): an all-zero group yields scale byte 0
in the kernels (the gold clamps amax to 1e-12 and yields 79), and the fp8 cast
saturates to +-448 (PTX cvt.rn.satfinite) instead of producing NaN.
"""
from __future__ import annotations

import math

import numpy as np
import torch

GROUP = 32
SF_TILE_M = 128
SF_TILE_K = 128
SF_TILE_STORAGE = 512
E4M3_MAX = 448.0


# ----------------------------------------------------------------------------
# scalar rule
# ----------------------------------------------------------------------------
def e8m0_from_amax(amax: torch.Tensor) -> torch.Tensor:
    """amax (f32, >= 0) -> ue8m0 byte as int32.

    bexp = bits>>23 & 0xFF; carry = mantissa > 0x600000; e = max(bexp-8+carry, 0),
    and 0 when bexp == 0 (blockscaled_fp8_gemm.py:487-493).
    """
    bits = amax.contiguous().view(torch.int32)
    bexp = (bits >> 23) & 0xFF
    carry = ((bits & 0x7FFFFF) > 0x600000).to(torch.int32)
    e = bexp - 8 + carry
    e = torch.where(bexp > 0, e, torch.zeros_like(e))
    return e.clamp(min=0)


def quant_scale_from_e8m0(e8m0: torch.Tensor) -> torch.Tensor:
    """2^(127 - e8m0) built as int_as_float(clamp(254 - e8m0, 1, 254) << 23)
    (blockscaled_fp8_gemm.py:496-498)."""
    q = (254 - e8m0).clamp(1, 254).to(torch.int32)
    return (q << 23).view(torch.float32)


def dequant_scale_from_e8m0(e8m0: torch.Tensor) -> torch.Tensor:
    """int_as_float(e8m0 << 23) = 2^(e8m0 - 127); byte 0 dequantises to 0.0
    (_gated_epilogues.py:2897-2900)."""
    return (e8m0.to(torch.int32) << 23).view(torch.float32)


def f32_to_e4m3_bytes(v: torch.Tensor) -> torch.Tensor:
    """cvt.rn.satfinite.e4m3x2.f32: round to nearest even, saturate to +-448.

    torch's CPU cast does not saturate (values above 464 become NaN), so clamp
    first.  NaN stays NaN (0x7F / 0xFF)."""
    v = v.float()
    c = torch.clamp(v, -E4M3_MAX, E4M3_MAX)
    c = torch.where(torch.isnan(v), v, c)
    return c.to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_bytes_to_f32(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float8_e4m3fn).float()


def f32_to_e4m3_bytes_bitwise(v: np.ndarray) -> np.ndarray:
    """Independent bit-level encoder (numpy, slow) used only to pin the torch
    cast above: RNE to 3 mantissa bits, min normal 2^-6, subnormal step 2^-9,
    saturate at 448."""
    v = np.asarray(v, dtype=np.float32)
    out = np.zeros(v.shape, dtype=np.uint8)
    sign = (np.signbit(v)).astype(np.uint8) << 7
    a = np.abs(v).astype(np.float64)
    nan = np.isnan(a)
    a = np.minimum(a, 448.0)
    # subnormal / normal split at 2^-6
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6)
    step = np.exp2(e - 3)
    q = np.rint(a / step)  # rint = ties to even
    val = q * step
    # re-normalise after rounding up to the next binade
    with np.errstate(divide="ignore"):
        e2 = np.floor(np.log2(np.where(val > 0, val, 1.0)))
    e2 = np.maximum(e2, -6)
    mant = val / np.exp2(e2)  # in [1,2) for normals, [0,1) for subnormals
    is_sub = val < 2.0 ** -6
    exp_field = np.where(is_sub, 0, e2 + 7).astype(np.int64)
    man_field = np.where(is_sub, np.rint(val / 2.0 ** -9), np.rint((mant - 1.0) * 8)).astype(np.int64)
    out = (exp_field << 3 | man_field).astype(np.uint8)
    out = np.where(nan, 0x7F, out).astype(np.uint8)
    return out | sign


# ----------------------------------------------------------------------------
# quantizers (inputs bf16 or f32; outputs uint8 bytes)
# ----------------------------------------------------------------------------
def _quant_groups(v: torch.Tensor, amax: torch.Tensor, amax_floor: float | None):
    """v: (..., G) f32 groups, amax: (...) -> bytes (..., G), e8m0 (...)."""
    if amax_floor is not None:
        amax = torch.clamp(amax, min=amax_floor)
    e = e8m0_from_amax(amax)
    qs = quant_scale_from_e8m0(e)
    q = f32_to_e4m3_bytes(v * qs.unsqueeze(-1))
    return q, e.to(torch.uint8)


def row_quant(x: torch.Tensor, amax_floor: float | None = None):
    """Row-wise 1x32: x (M,K) -> fp8 bytes (M,K) u8, raw scales (M,K/32) u8."""
    M, K = x.shape
    assert K % GROUP == 0
    v = x.float().reshape(M, K // GROUP, GROUP)
    q, e = _quant_groups(v, v.abs().amax(dim=-1), amax_floor)
    return q.reshape(M, K), e


def col_quant(x: torch.Tensor, gather_idx: torch.Tensor | None = None):
    """Column-wise 1x32 of src[gather_idx] (TK,dim): groups are 32 consecutive
    ROWS of one column.  Returns fp8 bytes (TK,dim) and raw scales (dim,TK/32)
    (blockscaled_fp8_gemm.py:1559-1583)."""
    if gather_idx is not None:
        x = x[gather_idx.long()]
    TK, dim = x.shape
    assert TK % GROUP == 0
    v = x.float().reshape(TK // GROUP, GROUP, dim).permute(0, 2, 1)  # (g, dim, 32)
    q, e = _quant_groups(v, v.abs().amax(dim=-1), None)
    q = q.permute(0, 2, 1).reshape(TK, dim)
    return q.contiguous(), e.transpose(0, 1).contiguous()


def iso32_quant(x: torch.Tensor):
    """One ue8m0 per 32x32 block, same rule.  Returns fp8 bytes (M,K) and the
    block scales (M/32, K/32) (blockscaled_fp8_gemm.py:2085-2106)."""
    M, K = x.shape
    assert M % GROUP == 0 and K % GROUP == 0
    v = x.float().reshape(M // GROUP, GROUP, K // GROUP, GROUP).permute(0, 2, 1, 3)
    v = v.reshape(M // GROUP, K // GROUP, GROUP * GROUP)
    q, e = _quant_groups(v, v.abs().amax(dim=-1), None)
    q = q.reshape(M // GROUP, K // GROUP, GROUP, GROUP).permute(0, 2, 1, 3).reshape(M, K)
    return q.contiguous(), e


def dequant_rows(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """fp8 bytes (M,K) with raw row scales (M,K/32) -> f32."""
    M, K = q.shape
    s = dequant_scale_from_e8m0(scales.to(torch.int32))
    return (e4m3_bytes_to_f32(q).reshape(M, K // GROUP, GROUP) * s.unsqueeze(-1)).reshape(M, K)


def dequant_cols(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """fp8 bytes (TK,dim) with raw column scales (dim,TK/32) -> f32 (TK,dim)."""
    TK, dim = q.shape
    s = dequant_scale_from_e8m0(scales.to(torch.int32)).transpose(0, 1)  # (TK/32, dim)
    return (e4m3_bytes_to_f32(q).reshape(TK // GROUP, GROUP, dim) * s.unsqueeze(1)).reshape(TK, dim)


# ----------------------------------------------------------------------------
# ISA scale layout
# ----------------------------------------------------------------------------
def isa_storage_bytes(rows: int, cols: int) -> int:
    return math.ceil(rows / SF_TILE_M) * math.ceil(cols / SF_TILE_K) * SF_TILE_STORAGE


def isa_index(rows: int, cols: int) -> torch.Tensor:
    """(rows, cols/32) -> byte index in the packed buffer:
    ((row//128)*ceil(cols/128) + g//4)*512 + (row%32)*16 + ((row%128)//32)*4 + g%4."""
    groups = math.ceil(cols / GROUP)
    k_tiles = math.ceil(cols / SF_TILE_K)
    r = torch.arange(rows, dtype=torch.int64).unsqueeze(1)
    g = torch.arange(groups, dtype=torch.int64).unsqueeze(0)
    rt = r % SF_TILE_M
    return ((r // SF_TILE_M) * k_tiles + g // 4) * SF_TILE_STORAGE + (rt % 32) * 16 + (rt // 32) * 4 + g % 4


def pack_isa(raw: torch.Tensor, rows: int, cols: int, fill: int = 127) -> torch.Tensor:
    """raw (rows, cols/32) u8 -> packed u8 of isa_storage_bytes(rows, cols);
    bytes no row/group maps to keep `fill` (127 = 1.0 in the reference's Triton
    paths, blockscaled_fp8_gemm.py:3244-3251)."""
    out = torch.full((isa_storage_bytes(rows, cols),), fill, dtype=torch.uint8)
    out[isa_index(rows, cols).reshape(-1)] = raw.reshape(-1)
    return out


def unpack_isa(packed: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    return packed.contiguous().view(torch.uint8).flatten()[isa_index(rows, cols).reshape(-1)].reshape(rows, -1)


def gather_scales_to_isa(raw: torch.Tensor, gather_idx: torch.Tensor, cols: int) -> torch.Tensor:
    """Row scales (T, cols/32) gathered to TK rows by gather_idx, ISA layout
    (sonicmoe/quack_utils/sm100_funcs.py:148-180)."""
    g = raw[gather_idx.long()]
    return pack_isa(g, g.shape[0], cols)


def bf16_rne(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> bf16 -> fp32 with round-to-nearest-even (_gated_epilogues.py:338-364)."""
    return v.float().to(torch.bfloat16).float()
