"""Host-side logic of the functional layer that needs no GPU: flags and configuration precedence, the pair-list to
table conversion of the general-routing entry point, result placement and the FP8 hand-off's error path."""
import pytest
import torch

import sonicmoe.functional as F
from sonicmoe.config import SonicMoEConfig, get_active_config


def test_fp8_flag_contexts_nest_and_restore():
    before = (F.is_fp8_active(), F.is_using_quack_gemm())
    with F.enable_fp8():
        assert F.is_fp8_active() and F.is_using_quack_gemm()
        with F.enable_fp8(False):
            assert not F.is_fp8_active()
        assert F.is_fp8_active()
        # an active configuration object wins over the context flag
        with SonicMoEConfig(use_fp8=False).activate():
            assert not F.is_fp8_active()
        assert F.is_fp8_active()
    assert (F.is_fp8_active(), F.is_using_quack_gemm()) == before
    assert get_active_config() is None


def test_memory_modes_precedence(monkeypatch):
    monkeypatch.delenv("SONIC_MOE_FP8_ISO32_WEIGHT", raising=False)
    monkeypatch.delenv("SONIC_MOE_STAGEWISE_MEMORY", raising=False)
    assert F._modes(None) == (False, False)
    monkeypatch.setenv("SONIC_MOE_FP8_ISO32_WEIGHT", "1")
    monkeypatch.setenv("SONIC_MOE_STAGEWISE_MEMORY", "true")
    assert F._modes(None) == (True, True)
    # an explicit field beats the environment; an explicit config beats the active one
    assert F._modes(SonicMoEConfig(iso32_weight=False)) == (False, True)
    with SonicMoEConfig(stagewise_memory=False).activate():
        assert F._modes(None) == (True, False)
        assert F._modes(SonicMoEConfig(iso32_weight=False, stagewise_memory=True)) == (False, True)
    with pytest.raises(NotImplementedError):
        SonicMoEConfig(swiglu_clamp_value=7.0)


def test_pair_list_becomes_padded_tables_and_scores_stay_differentiable():
    T = 6
    tok = torch.tensor([0, 0, 0, 2, 3, 3, 5])                    # sorted by token; tokens 1 and 4 have no pair
    exp = torch.tensor([4, 1, 7, 2, 0, 3, 6])
    sc = torch.tensor([.5, .25, .25, 1., .75, .25, .9], requires_grad=True)
    idx, scores = F._pairs_to_table(sc, tok, exp, T)
    assert idx.dtype == torch.int32 and idx.shape == (T, 3) and scores.shape == (T, 3)
    assert idx.tolist() == [[4, 1, 7], [-1, -1, -1], [2, -1, -1], [0, 3, -1], [-1, -1, -1], [6, -1, -1]]
    sv = scores.detach()
    assert torch.equal(sv[0], sc[:3].detach()) and float(sv[3, 1]) == 0.25 and float(sv[1].sum()) == 0.0
    (scores * torch.arange(18.).view(T, 3)).sum().backward()
    assert sc.grad.tolist() == [0., 1., 2., 6., 9., 10., 15.]
    # no pairs at all: one masked lane per token
    idx0, sc0 = F._pairs_to_table(torch.zeros(0), torch.zeros(0, dtype=torch.long), torch.zeros(0, dtype=torch.long), 3)
    assert idx0.tolist() == [[-1]] * 3 and sc0.shape == (3, 1)
    # more pairs for one token than the metadata kernel has lanes
    many = F._MAX_PAIRS_PER_TOKEN + 1
    with pytest.raises(NotImplementedError):
        F._pairs_to_table(torch.ones(many), torch.zeros(many, dtype=torch.long), torch.arange(many), 2)


def test_result_placement_is_consumed_once_innermost_first():
    a, b, c = torch.zeros(1), torch.zeros(2), torch.zeros(3)
    assert F._take_placement() == (None, None)
    with F.place_results(a, b):
        with F.place_results(c, None):
            out, dx = F._take_placement()
            assert out is c and dx is None
            assert F._take_placement() == (None, None)           # consumed
        out, dx = F._take_placement()
        assert out is a and dx is b
    assert F._take_placement() == (None, None)


def test_down_projection_refuses_a_z_it_was_not_handed():
    with pytest.raises(RuntimeError, match="no _UpProjection.forward produced"):
        F._handoff_take(torch.zeros(4, 4))
    z = torch.zeros(())
    F._handoff_put(z, {"y1": 1})
    assert F._handoff_take(z) == {"y1": 1}
    with pytest.raises(RuntimeError):
        F._handoff_take(z)                                         # taken once


def test_gated_output_payload_wants_four_tensors():
    sf = torch.zeros(8, dtype=torch.uint8)
    with pytest.raises(ValueError):
        F.attach_preallocated_gated_outputs(sf, (1, 2, 3))
    assert F.attach_preallocated_gated_outputs(sf, (1, 2, 3, 4)) is sf
    assert getattr(sf, F._GATED_OUTPUT_PAYLOAD_ATTR) == (1, 2, 3, 4)
