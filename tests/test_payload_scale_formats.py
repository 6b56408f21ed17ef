"""Host-side conversion of the 1x32 ue8m0 scale formats an FP8 dispatch payload may arrive in (reference:
sonicmoe/quack_utils/blockscaled_fp8_gemm.py:535-550, sonicmoe/interface.py:135-187) into one byte per group."""
import pytest
import torch

from sonicmoe.interface import scale_bytes


def test_every_scale_format_gives_the_same_bytes():
    N, H = 5, 256
    g = torch.Generator().manual_seed(0)
    raw = torch.randint(0, 256, (N, H // 32), generator=g, dtype=torch.uint8)
    assert torch.equal(scale_bytes(raw, H), raw)
    # four scale bytes per little-endian word: byte j of a row is group j
    words = raw.view(torch.int32)
    assert words.shape == (N, H // 128)
    assert torch.equal(scale_bytes(words, H), raw)
    # one word per group
    assert torch.equal(scale_bytes(raw.to(torch.int32), H), raw)
    if getattr(torch, "float8_e8m0fnu", None) is not None:
        assert torch.equal(scale_bytes(raw.view(torch.float8_e8m0fnu), H), raw)
    # a strided view is accepted and comes back contiguous
    wide = torch.zeros(N, 2 * (H // 32), dtype=torch.uint8)
    wide[:, ::2] = raw
    out = scale_bytes(wide[:, ::2], H)
    assert out.is_contiguous() and torch.equal(out, raw)


def test_a_format_that_matches_nothing_is_refused():
    N, H = 4, 256
    with pytest.raises(ValueError, match="none of the 1x32 ue8m0 formats"):
        scale_bytes(torch.zeros(N, H // 32, dtype=torch.float32), H)
    with pytest.raises(ValueError):
        scale_bytes(torch.zeros(N, H // 32 + 1, dtype=torch.uint8), H)
    with pytest.raises(ValueError):
        scale_bytes(torch.zeros(N, 3, dtype=torch.int32), H)
