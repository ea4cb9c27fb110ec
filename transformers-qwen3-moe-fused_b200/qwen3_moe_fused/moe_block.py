"""`MoeFusedLinear` and the sparse MoE block on the kernels of this package.

`MoeFusedLinear` mirrors the reference module
(qwen3_moe_fused/modular_qwen3_moe_fused.py:29-59): parameter `weight` of shape
(num_experts, out_features, in_features), Kaiming-uniform initialisation with bound
sqrt(15 / in_features), `forward(input, m_sizes)`.

`moe_block_forward` computes what `Qwen3MoeFusedSparseMoeBlock.forward` computes
(:79-118), using one kernel each for the router epilogue (softmax + top-k + renormalise +
cast), the expand+gather, and the un-permute + weighted combine.
"""
import math
from typing import Optional

import torch
from torch import nn

from .functional import moe_fused_linear
from .kernels.fused_mlp import gate_up_silu_forward
from .kernels.indexing import get_expert_counts_and_idx
from .kernels.routing import combine, gather_rows, softmax_topk_autograd
from .kernels.silu_mul import silu_mul


# The inference path can feed gate / up straight from the token tensor (TMA gather4 in the token load,
# `gate_up_silu_forward(..., row_index=...)`).  Measured at 16384 tokens x top-8 on B200 it is SLOWER than
# writing the expanded rows first (block forward 2.85 ms against 1.19 ms): a CTA needs 32 gather4 loads
# per 64-column stage, each with its own four row coordinates, and the loads of one warp issue one after
# the other, which takes longer than the stage's MMAs.  Off by default; the result is the same either way.
GATHER_IN_KERNEL = False


def moe_fused_kaiming_uniform_(weight: torch.Tensor) -> None:
    bound = math.sqrt(3 * 5 / weight.shape[-1])
    nn.init.uniform_(weight, -bound, bound)


class MoeFusedLinear(nn.Module):
    __constants__ = ["in_features", "out_features", "num_experts"]

    def __init__(self, in_features: int, out_features: int, num_experts: int,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.num_experts = num_experts
        self.weight = nn.Parameter(torch.empty((num_experts, out_features, in_features), device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        moe_fused_kaiming_uniform_(self.weight)

    def forward(self, input: torch.Tensor, m_sizes: torch.Tensor) -> torch.Tensor:
        return moe_fused_linear(input, self.weight, m_sizes)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, num_experts={self.num_experts}"


def route(router_logits: torch.Tensor, num_selected: int, norm_topk_prob: bool, dtype: torch.dtype):
    """(routing_weights (T,k) dtype, selected_experts (T,k) int64)."""
    return softmax_topk_autograd(router_logits.contiguous(), num_selected, norm_topk_prob, dtype)


def moe_block_forward(hidden_states: torch.Tensor, gate_weight: torch.Tensor, gate_proj: torch.Tensor,
                      up_proj: torch.Tensor, down_proj: torch.Tensor, num_selected: int,
                      norm_topk_prob: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """hidden_states (B, S, H); gate_weight (E, H); gate_proj/up_proj (E, I, H); down_proj (E, H, I).
    Returns (output (B, S, H), router_logits (B*S, E))."""
    B, S, H = hidden_states.shape
    T = B * S
    E = gate_weight.shape[0]
    k = num_selected
    x = hidden_states.reshape(T, H)
    router_logits = torch.nn.functional.linear(x, gate_weight)
    routing_weights, selected = route(router_logits, k, norm_topk_prob, x.dtype)
    m_sizes, sort_idx, inv_sort_idx = get_expert_counts_and_idx(selected.view(T * k), E)
    if not torch.is_grad_enabled() and GATHER_IN_KERNEL:
        # gate, up and SiLU-mul in one kernel whose token load gathers the rows straight from the (T, H)
        # tokens (same result bit for bit; the expanded, sorted copy is never written)
        h = gate_up_silu_forward(x.contiguous(), gate_proj, up_proj, m_sizes, row_index=sort_idx, index_div=k)
    elif not torch.is_grad_enabled():
        # inference: gate, up and SiLU-mul in one kernel (same result bit for bit)
        h = gate_up_silu_forward(gather_rows(x.contiguous(), sort_idx, inv_sort_idx, k), gate_proj, up_proj, m_sizes)
    else:
        xs = gather_rows(x.contiguous(), sort_idx, inv_sort_idx, k)
        gate_h = moe_fused_linear(xs, gate_proj, m_sizes)
        up_h = moe_fused_linear(xs, up_proj, m_sizes)
        h = silu_mul(gate_h, up_h)
    y = moe_fused_linear(h, down_proj, m_sizes)
    out = combine(y, sort_idx, inv_sort_idx, routing_weights)
    return out.view(B, S, H), router_logits


def fused_sparse_moe_block_forward(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """`forward` for the reference's `Qwen3MoeFusedSparseMoeBlock`
    (qwen3_moe_fused/modular_qwen3_moe_fused.py:79-118): same inputs, outputs and gradients, computed by
    `moe_block_forward` (router epilogue, expand + gather and un-permute + weighted sum as one kernel
    each; under `torch.no_grad()` gate, up and SiLU-mul as one tensor-core kernel).  `self` needs the
    attributes of that class: `gate` (a bias-free Linear), `gate_proj` / `up_proj` / `down_proj` (plain
    `MoeFusedLinear` modules), `num_selected`, `norm_topk_prob`."""
    for name in ("gate_proj", "up_proj", "down_proj"):
        if not _is_plain_fused_linear(getattr(self, name)):
            raise NotImplementedError(f"{name} is a {type(getattr(self, name)).__name__}: this forward takes plain MoeFusedLinear "
                                      "projections (LoRA or 4-bit projections go through fast_lora)")
    return moe_block_forward(hidden_states, self.gate.weight, self.gate_proj.weight, self.up_proj.weight,
                             self.down_proj.weight, self.num_selected, self.norm_topk_prob)


def _is_plain_fused_linear(module) -> bool:
    """True for a module that is exactly a weight-only fused linear: this package's `MoeFusedLinear` or the
    class of that name in the reference's modular file (not a subclass that changes `forward`)."""
    cls = type(module)
    return cls.__name__ == "MoeFusedLinear" and isinstance(getattr(module, "weight", None), torch.Tensor) and \
        not hasattr(module, "base_layer") and not hasattr(module, "quant_state")


def patch_Qwen3MoeFusedSparseMoeBlock_forward(block_class=None) -> None:
    """Installs `fused_sparse_moe_block_forward` on the sparse MoE block class, the way the reference's
    own patch function does for its fused-LoRA forward (qwen3_moe_fused/fast_lora.py:84-85).  Without an
    argument the class is `Qwen3MoeFusedSparseMoeBlock` of the reference's modular file, which is
    importable through this package when `QWEN3_MOE_FUSED_REFERENCE` points at a checkout."""
    if block_class is None:
        from .modular_qwen3_moe_fused import Qwen3MoeFusedSparseMoeBlock as block_class  # file of the reference checkout
    block_class.forward = fused_sparse_moe_block_forward
