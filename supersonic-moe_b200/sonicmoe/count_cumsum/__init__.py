"""count_cumsum(x, E, do_cumsum=True) - histogram of expert ids and its inclusive
cumsum, int32 (sonicmoe/count_cumsum/__init__.py:20-35)."""
import torch

from ..ops import count_cumsum as _count_cumsum


@torch.no_grad()
def count_cumsum(x: torch.Tensor, E: int, do_cumsum: bool = True):
    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in (torch.int32, torch.long)
    return _count_cumsum(x.contiguous(), E, do_cumsum)
