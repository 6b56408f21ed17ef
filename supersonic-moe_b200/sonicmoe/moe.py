"""`MoE` module: router Linear + interleaved-SwiGLU experts
(sonicmoe/moe.py:96-114 `Experts`, :205-254 `MoE.__init__`, :580-662 forward and
switch aux loss).  Only the sm_100a MXFP8 backend exists here; the reference's
pure-PyTorch backend is restated under oracle/ for checking, not shipped."""
from __future__ import annotations

from contextlib import ExitStack

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import SonicMoEConfig
from .enums import ActivationType, KernelBackendMoE, is_glu
from .functional import enable_fp8, moe_TC_softmax_topk_layer


class Experts(nn.Module):
    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True,
                 std: float | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        self.std = std
        self.num_experts, self.in_features, self.out_features = num_experts, in_features, out_features
        self.reset_parameters()

    def extra_repr(self):
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()


class MoE(nn.Module):
    def __init__(self, num_experts: int, num_experts_per_tok: int, hidden_size: int, intermediate_size: int,
                 activation_function: ActivationType, add_bias: bool, std: float,
                 config: SonicMoEConfig | None = None) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.config = config
        self.router = nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)
        self.activation_function = activation_function
        self.c_fc = Experts(num_experts, hidden_size,
                            2 * intermediate_size if is_glu(activation_function) else intermediate_size,
                            add_bias=add_bias, std=std)
        self.c_proj = Experts(num_experts, intermediate_size, hidden_size, add_bias=add_bias, std=std)
        self.stream_id = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0

    def forward(self, hidden_states: torch.Tensor, kernel_backend_moe: KernelBackendMoE = KernelBackendMoE.sonicmoe,
                is_inference_mode: bool = False, fp8_protocol=None, use_fp8: bool = False,
                config: SonicMoEConfig | None = None):
        original_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        active_config = config or self.config
        if kernel_backend_moe != KernelBackendMoE.sonicmoe:
            raise NotImplementedError(
                f"kernel_backend_moe={kernel_backend_moe}: only KernelBackendMoE.sonicmoe (sm_100a MXFP8 kernels) is "
                "built; there is no PyTorch/CPU fallback")
        with ExitStack() as stack:
            if active_config is not None:
                stack.enter_context(active_config.activate())
            if use_fp8:
                stack.enter_context(enable_fp8())
            hidden_states, router_logits, expert_frequency = moe_TC_softmax_topk_layer(
                hidden_states, self.router.weight, self.c_fc.weight.permute(1, 2, 0), self.c_fc.bias,
                self.c_proj.weight.permute(1, 2, 0), self.c_proj.bias, self.top_k, self.stream_id,
                self.activation_function, is_inference_mode or not self.training, fp8_protocol)
        hidden_states = hidden_states.view(original_shape)
        if is_inference_mode:
            aux_loss = None
        else:
            aux_loss = self._compute_switch_loss(
                logits=router_logits, probs=F.softmax(router_logits, dim=-1, dtype=torch.float32),
                expert_frequency=expert_frequency)
        return hidden_states, aux_loss

    def _compute_switch_loss(self, logits, probs, expert_frequency):
        logits = logits.view(-1, logits.size(-1))
        probs = probs.view(-1, probs.size(-1))
        num_experts = logits.size(1)
        acc_probs = probs.sum(0)
        expert_frequency = expert_frequency.float()
        return num_experts * (F.normalize(acc_probs, p=1, dim=0) * F.normalize(expert_frequency, p=1, dim=0)).sum()
