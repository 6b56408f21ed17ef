"""Addressing beyond 2^31: the largest benchmark config (T=65536, H=6144, K=8) has expert-sorted activations of
TKp x H = 3.2e9 elements, so every kernel must index rows with 64-bit arithmetic (the reference switches to int64
offsets above 2^31-1: blockscaled_fp8_gemm.py:571-574, :3258-3260, reduction_over_k_gather.py:372-375).

One [rows, 6144] problem with rows x 6144 > 2^31 goes through the row quantizer, the grouped GEMM (A and its scales
read, C written past the 2 Gi-element mark) and the combine (rows gathered from both ends); rows sampled from the
first and the last tiles are compared with the CPU oracle.  About 7 GB on the device."""
import pytest
import torch

from oracle import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROWS, K = 2816 * 128, 6144            # 360448 x 6144 = 2.21e9 elements > 2^31


@pytest.fixture(scope="module")
def big():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if torch.cuda.get_device_properties(0).total_memory < 24e9:
        pytest.skip("needs ~7 GB of device memory")
    from sonicmoe import ops
    assert ROWS * K > 2 ** 31
    g = torch.Generator(device=DEV).manual_seed(17)
    x = torch.empty(ROWS, K, dtype=torch.bfloat16, device=DEV)
    step = 32768
    for r in range(0, ROWS, step):      # drawn in slabs: no multi-GB fp32 temporary
        x[r:r + step] = torch.randn(min(step, ROWS - r), K, generator=g, device=DEV)
    q, raw, isa = ops.quant_rows(x, raw=True, isa=True)
    torch.cuda.synchronize()
    yield dict(ops=ops, x=x, q=q, raw=raw, isa=isa)
    torch.cuda.empty_cache()


def _sample_rows():
    return torch.cat([torch.arange(0, 40), torch.arange(ROWS // 2 - 20, ROWS // 2 + 20),
                      torch.arange((2 ** 31) // K - 8, (2 ** 31) // K + 8), torch.arange(ROWS - 40, ROWS)])


def test_row_quantizer_past_two_gi_elements(big):
    rows = _sample_rows()
    xs = big["x"][rows.to(DEV)].cpu()
    q_ref, s_ref = Q.row_quant(xs)
    assert torch.equal(big["q"][rows.to(DEV)].cpu(), q_ref)
    assert torch.equal(big["raw"][rows.to(DEV)].cpu(), s_ref)
    # ISA-packed scales of the sampled rows: byte(row, g) = ((row/128)*ceil(K/128) + g/4)*512 + (row%32)*16 +
    # ((row%128)/32)*4 + g%4
    gi = torch.arange(K // 32)
    at = ((rows.unsqueeze(1) // 128) * (K // 128) + gi // 4) * 512 + (rows.unsqueeze(1) % 32) * 16 + \
        ((rows.unsqueeze(1) % 128) // 32) * 4 + gi % 4
    assert torch.equal(big["isa"][at.to(DEV)].cpu(), s_ref)


def test_grouped_gemm_past_two_gi_elements(big):
    """C = A . B[e]^T over two experts splitting the rows unevenly; N = 256 keeps C small while A (2.2 GB) and its
    scales are addressed to the end."""
    ops = big["ops"]
    E, N = 2, 256
    g = torch.Generator().manual_seed(5)
    b = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
    bq, bs = Q.row_quant(b.view(E * N, K))
    b_q_d, _, b_sf_d = ops.quant_rows(b.view(E * N, K).to(DEV), raw=False, isa=True)
    assert torch.equal(b_q_d.cpu(), bq)
    split = 1000 * 128
    efo = torch.tensor([0, split, ROWS], dtype=torch.int32, device=DEV)
    c = ops.gemm_varlen_m(big["q"], big["isa"], b_q_d.view(E, N, K), b_sf_d, efo)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    rows = _sample_rows()
    a_d = Q.dequant_rows(big["q"][rows.to(DEV)].cpu(), big["raw"][rows.to(DEV)].cpu())
    b_d = Q.dequant_rows(bq, bs).view(E, N, K)
    ref = torch.stack([a_d[i] @ b_d[int(r >= split)].T for i, r in enumerate(rows.tolist())])
    got = c[rows.to(DEV)].float().cpu()
    cos = float((got * ref).sum() / (got.norm() * ref.norm()))
    rr = float((got - ref).norm() / ref.norm())
    assert cos > 0.99999 and rr < 0.005, (cos, rr)      # bf16 rounding of C only


def test_combine_gathers_rows_from_both_ends(big):
    """out[t] = sum_j w_j * y[row_j] with rows taken from the whole [ROWS, K] bf16 buffer (fp32 accumulate)."""
    ops = big["ops"]
    T, Kt = 512, 8
    g = torch.Generator().manual_seed(9)
    lanes = torch.randint(0, ROWS, (T, Kt), generator=g)
    lanes[0] = torch.arange(ROWS - Kt, ROWS)               # the very last rows
    lanes[1] = torch.arange(0, Kt)
    w = torch.rand(T * Kt, generator=g)
    s_rev = lanes.flatten().to(torch.int32)
    naept = (torch.arange(T + 1) * Kt).to(torch.int32)
    out = ops.combine(big["x"], s_rev.to(DEV), naept.to(DEV), w.to(DEV), T)
    torch.cuda.synchronize()
    y = big["x"][lanes.flatten().to(DEV)].float().cpu().view(T, Kt, K)
    ref = torch.zeros(T, K)
    for j in range(Kt):                                     # ascending lane order, fp32
        ref += w.view(T, Kt)[:, j:j + 1] * y[:, j]
    # fused multiply-add on the GPU vs multiply-then-add here: equal up to the last bf16 bit
    torch.testing.assert_close(out.cpu().float(), ref, rtol=8e-3, atol=1e-2)
