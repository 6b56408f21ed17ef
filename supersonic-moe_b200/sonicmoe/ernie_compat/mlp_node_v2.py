"""`SonicMoEMlpNode`: the expert FFN of one MoE layer behind the interface a DeepEP-style host framework calls
(mirrors sonicmoe/ernie_compat/mlp_node_v2.py:411-706 of the reference).

The host framework keeps one module per expert with split-half weights

    up_gate_proj.weight [H, 2I]   columns [0, I) = gate, [I, 2I) = up
    down_proj.weight    [I, H]

and reads per-expert fp32 `weight.main_grad` buffers in those layouts.  The kernels want stacked, interleaved
operands (`w1 [E, 2I, H]` with rows gate0, up0, gate1, up1, ...; `w2 [E, H, I]`).  The node

* stacks the expert weights into the kernel layout once per weight version (cache keyed by data pointer and
  version counter, mlp_node_v2.py:254-322),
* owns one fp32 buffer per weight whose slices ARE the experts' `main_grad` (mlp_node_v2.py:325-363); while
  micro-batches accumulate, the W1 buffer is addressed through its kernel-layout view `[E, 2I, H]`, and `step()`
  rewrites it in place to the framework layout `[E, H, 2I]` split-half (mlp_node_v2.py:378-396).  The W2 gradient
  needs no rewrite here: this build's dw2 GEMM already produces `[E, I, H]`, the framework's layout,
* runs `run_sonic_moe` on the dispatched rows; dx and the gradient of the dispatched probabilities flow through
  autograd (mlp_node_v2.py:559-653, `_differentiable_router_scores` :169-238).

Framework tensors are torch tensors here (the reference adapts Paddle tensors through its compatibility layer).
"""
from __future__ import annotations

from typing import Any, Sequence

import torch

from ..enums import ActivationType


def _cache_key(*tensors: torch.Tensor) -> tuple:
    return tuple((t.data_ptr(), t._version) for t in tensors)


def stack_w1_interleaved(weights: Sequence[torch.Tensor], I: int) -> torch.Tensor:
    """Per-expert `[H, 2I]` split-half -> `[E, 2I, H]` with gate / up rows interleaved."""
    stacked = torch.stack([w.detach() for w in weights])                    # [E, H, 2I]
    gate, up = stacked[:, :, :I], stacked[:, :, I:]
    E, H = stacked.shape[0], stacked.shape[1]
    return torch.stack([gate, up], dim=3).reshape(E, H, 2 * I).permute(0, 2, 1).contiguous()


def stack_w2(weights: Sequence[torch.Tensor]) -> torch.Tensor:
    """Per-expert `[I, H]` -> `[E, H, I]`."""
    return torch.stack([w.detach() for w in weights]).permute(0, 2, 1).contiguous()


def flush_w1_main_grad_(mg1: torch.Tensor) -> None:
    """In place: storage holding the kernel layout `[E, 2I, H]` (interleaved) becomes the framework layout
    `[E, H, 2I]` (all gates, then all ups).  `mg1` has the framework shape `[E, H, 2I]`."""
    E, H, two_I = mg1.shape
    I = two_I // 2
    native = mg1.view(E, two_I, H)
    rhs = native.view(E, I, 2, H).permute(0, 3, 2, 1).contiguous()          # [E, H, 2, I]
    mg1.view(E, H, 2, I).copy_(rhs)


class _MarkPending(torch.autograd.Function):
    """Identity on the node's output; its backward (the first to run) notes on the node that gradients in the
    kernels' layout are about to be accumulated, so that `step()` knows a flush is due."""

    @staticmethod
    def forward(ctx, out, node):
        ctx.node = node
        return out.view_as(out)

    @staticmethod
    def backward(ctx, g):
        ctx.node._pending_flush = True
        return g, None


class SonicMoEMlpNode:
    """Drop-in for the host framework's MlpNode on the top-k dispatch path.

    experts            per-expert modules with `up_gate_proj.weight [H, 2I]` and `down_proj.weight [I, H]`
    n_experts          local experts E
    hidden_size, intermediate_size
    activation_type    SwiGLU (fused GEMM epilogues), ReGLU or GEGLU (plain GEMMs + activation kernels)
    stream_id          kept for signature compatibility (work runs on the current stream)

    Training-loop contract (mlp_node_v2.py:655-679):

        for micro-batch: out = node(x, tokens_per_expert, indices, probs); out.backward(grad)
        node.step()            # main_grad now in the framework layout
        optimizer.step(); optimizer.zero_grad()
    """

    def __init__(self, experts: Sequence[Any], n_experts: int, hidden_size: int, intermediate_size: int,
                 activation_type: ActivationType | str = ActivationType.SWIGLU, stream_id: int = 0):
        self._experts = list(experts)
        if len(self._experts) != n_experts:
            raise ValueError(f"{len(self._experts)} expert modules for n_experts={n_experts}")
        self._E, self._H, self._I = n_experts, hidden_size, intermediate_size
        if isinstance(activation_type, str):
            activation_type = ActivationType(activation_type)
        from ..enums import activation_code
        activation_code(activation_type)          # SwiGLU, ReGLU, GEGLU; raises for anything else
        self._activation_type = activation_type
        self._stream_id = stream_id
        self._w_cache: dict = {}
        self._pending_flush = False
        self._warmed_for_step = False

    # ---- weights ---------------------------------------------------------------------------------------------
    def _stacked_weights(self):
        w1s = [e.up_gate_proj.weight for e in self._experts]
        w2s = [e.down_proj.weight for e in self._experts]
        key = ("w",) + _cache_key(*w1s, *w2s)
        hit = self._w_cache.get(key)
        if hit is None:
            for k in [k for k in self._w_cache if isinstance(k, tuple) and k[0] == "w"]:
                del self._w_cache[k]                                # weights moved on: drop the stale stack
            w1 = stack_w1_interleaved(w1s, self._I).requires_grad_(True)
            w2 = stack_w2(w2s).requires_grad_(True)
            hit = self._w_cache[key] = (w1, w2)
        w1, w2 = hit
        # gradients accumulate into the node's buffers, addressed in the kernels' layouts
        w1.main_grad = self._w1_native_view()
        w2.main_grad = self._w2_main_grad()
        return w1, w2

    def _w1_main_grad(self) -> torch.Tensor:
        """`[E, H, 2I]` fp32, slice e aliased to `experts[e].up_gate_proj.weight.main_grad`; allocated lazily."""
        mg = self._w_cache.get("w1_mg")
        if mg is None:
            dev = self._experts[0].up_gate_proj.weight.device
            mg = self._w_cache["w1_mg"] = torch.zeros(self._E, self._H, 2 * self._I, dtype=torch.float32, device=dev)
            for i, e in enumerate(self._experts):
                e.up_gate_proj.weight.main_grad = mg[i]
        return mg

    def _w2_main_grad(self) -> torch.Tensor:
        """`[E, I, H]` fp32, slice e aliased to `experts[e].down_proj.weight.main_grad`."""
        mg = self._w_cache.get("w2_mg")
        if mg is None:
            dev = self._experts[0].down_proj.weight.device
            mg = self._w_cache["w2_mg"] = torch.zeros(self._E, self._I, self._H, dtype=torch.float32, device=dev)
            for i, e in enumerate(self._experts):
                e.down_proj.weight.main_grad = mg[i]
        return mg

    def _w1_native_view(self) -> torch.Tensor:
        """Storage of the W1 buffer as the kernels address it, `[E, 2I, H]`.  Between `step()` and the optimizer's
        `zero_grad()` the storage holds the framework layout; a backward in that window would mix the two (the
        reference has the same contract)."""
        return self._w1_main_grad().view(self._E, 2 * self._I, self._H)

    def _flush_native_grads(self) -> None:
        if not self._pending_flush:
            return
        flush_w1_main_grad_(self._w1_main_grad())
        self._pending_flush = False

    def flush_grads(self) -> None:
        """Deferred layout flush without ending the step (reading `main_grad` between micro-batches is then only
        valid if no further backward follows before it is zeroed)."""
        self._flush_native_grads()

    # ---- public API ------------------------------------------------------------------------------------------
    def prequantize_weights(self) -> None:
        """FP8 copies of both weights in all four layouts, once per step (mlp_node_v2.py:527-543)."""
        if self._warmed_for_step:
            return
        from ..functional import precompute_weight_fp8
        w1, w2 = self._stacked_weights()
        precompute_weight_fp8(w1, w2)
        self._warmed_for_step = True

    def warmup(self, total_K_list=None, max_workers: int = 0) -> None:
        """Nothing to compile at run time: the kernels are built ahead of time into the shared library."""
        return None

    def forward(self, dispatched_hidden_states: torch.Tensor, tokens_per_expert, dispatched_indices=None,
                dispatched_probs=None) -> torch.Tensor:
        """dispatched_hidden_states [N_recv, H] bf16; tokens_per_expert list[int] | Tensor [E];
        dispatched_indices [N_recv, topk] int32 local expert ids, -1 = masked; dispatched_probs [N_recv, topk] f32.
        Returns [N_recv, H] bf16 in the input's row order."""
        if dispatched_indices is None:
            raise AssertionError("dispatched_indices is required (identity layout path removed)")
        if dispatched_probs is None:
            raise AssertionError("dispatched_probs required when dispatched_indices is given")
        from ..interface import run_sonic_moe
        self.prequantize_weights()
        w1, w2 = self._stacked_weights()
        out = run_sonic_moe(dispatched_hidden_states, dispatched_indices, dispatched_probs,
                            dispatched_indices.shape[1], self._E, w1, w2, fp8=True,
                            tokens_per_expert=tokens_per_expert, activation_type=self._activation_type)
        return _MarkPending.apply(out, self)

    __call__ = forward

    def step(self) -> None:
        """Commit the accumulated weight gradients: after this call every expert's `main_grad` is in the framework
        layout.  Call before `optimizer.step()`."""
        self._flush_native_grads()
        self._warmed_for_step = False
        # The optimizer is about to change the expert weights, often through `param.data.copy_(master)`, which does
        # not move the tensor version counter the caches look at: drop the stacked copies and their FP8 forms now
        # (they would be rebuilt after the update anyway; the fp32 gradient buffers stay).
        from ..functional import drop_weight_fp8
        for k in [k for k in self._w_cache if isinstance(k, tuple) and k[0] == "w"]:
            drop_weight_fp8(*self._w_cache.pop(k))

    def invalidate_caches(self) -> None:
        """Drop the stacked weights, the gradient buffers and the FP8 weight cache."""
        from ..functional import clear_weight_cache
        self._w_cache.clear()
        clear_weight_cache()
        self._warmed_for_step = False
        self._pending_flush = False
