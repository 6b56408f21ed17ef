"""Host-side layout logic of SonicMoEMlpNode (no GPU): split-half <-> interleaved stacking and the in-place
main_grad flush (reference: sonicmoe/ernie_compat/mlp_node_v2.py:275-322, 378-396)."""
import torch

from sonicmoe.ernie_compat import flush_w1_main_grad_, stack_w1_interleaved, stack_w2


def test_w1_stacking_interleaves_gate_and_up_rows():
    E, H, I = 3, 8, 4
    g = torch.Generator().manual_seed(0)
    ws = [torch.randn(H, 2 * I, generator=g) for _ in range(E)]
    w1 = stack_w1_interleaved(ws, I)
    assert w1.shape == (E, 2 * I, H) and w1.is_contiguous()
    for e in range(E):
        for j in range(I):
            assert torch.equal(w1[e, 2 * j], ws[e][:, j])            # gate j
            assert torch.equal(w1[e, 2 * j + 1], ws[e][:, I + j])    # up j


def test_w2_stacking_transposes_each_expert():
    E, H, I = 2, 6, 5
    ws = [torch.randn(I, H) for _ in range(E)]
    w2 = stack_w2(ws)
    assert w2.shape == (E, H, I)
    for e in range(E):
        assert torch.equal(w2[e], ws[e].T)


def test_flush_turns_kernel_layout_storage_into_framework_layout_in_place():
    E, H, I = 2, 8, 4
    g = torch.Generator().manual_seed(1)
    dw1_native = torch.randn(E, 2 * I, H, generator=g)               # what the kernels accumulate
    mg1 = torch.zeros(E, H, 2 * I)
    mg1.view(E, 2 * I, H).copy_(dw1_native)
    ptr = mg1.data_ptr()
    per_expert = [mg1[e] for e in range(E)]                          # the aliases the experts hold
    flush_w1_main_grad_(mg1)
    assert mg1.data_ptr() == ptr
    for e in range(E):
        want = torch.cat([dw1_native[e, 0::2].T, dw1_native[e, 1::2].T], dim=1)     # [H, I gates | I ups]
        assert torch.equal(per_expert[e], want)
    # the gradient of stack_w1_interleaved w.r.t. the split-half weights is exactly that mapping
    ws = [torch.randn(H, 2 * I, generator=g, requires_grad=True) for _ in range(E)]
    stacked = torch.stack(ws)
    gate, up = stacked[:, :, :I], stacked[:, :, I:]
    w1 = torch.stack([gate, up], dim=3).reshape(E, H, 2 * I).permute(0, 2, 1)
    (w1 * dw1_native).sum().backward()
    for e in range(E):
        assert torch.equal(ws[e].grad, per_expert[e])


def test_gradient_buffers_outlive_weight_updates_and_steps():
    """The fp32 buffers whose slices are the experts' `main_grad` are allocated once: neither `step()` nor a weight
    update (which replaces the stacked weight copies) may replace them - an optimizer that captured `main_grad`
    would otherwise keep reading a dead tensor - while the stacked copies do follow the new weights."""
    from types import SimpleNamespace
    from sonicmoe.ernie_compat import SonicMoEMlpNode

    E, H, I = 2, 8, 4
    g = torch.Generator().manual_seed(2)
    experts = [SimpleNamespace(up_gate_proj=SimpleNamespace(weight=torch.randn(H, 2 * I, generator=g)),
                               down_proj=SimpleNamespace(weight=torch.randn(I, H, generator=g))) for _ in range(E)]
    node = SonicMoEMlpNode(experts, E, H, I)
    w1, w2 = node._stacked_weights()
    held1 = [e.up_gate_proj.weight.main_grad for e in experts]
    held2 = [e.down_proj.weight.main_grad for e in experts]
    assert w1.main_grad.data_ptr() == held1[0].data_ptr() and w2.main_grad.data_ptr() == held2[0].data_ptr()
    held1[1].fill_(3.0)

    experts[0].up_gate_proj.weight.add_(1.0)                     # version counter moves: a new stack, same buffers
    w1b, _ = node._stacked_weights()
    assert w1b is not w1 and torch.equal(w1b[0, 0], experts[0].up_gate_proj.weight[:, 0])
    node.step()
    experts[1].down_proj.weight.data.copy_(torch.zeros(I, H))    # invisible to the version counter; after step()
    w1c, w2c = node._stacked_weights()
    assert torch.equal(w2c[1], torch.zeros(H, I))
    for e in range(E):
        assert experts[e].up_gate_proj.weight.main_grad.data_ptr() == held1[e].data_ptr()
        assert experts[e].down_proj.weight.main_grad.data_ptr() == held2[e].data_ptr()
    assert w1c.main_grad.data_ptr() == held1[0].data_ptr() and float(held1[1].min()) == 3.0
