"""`moe_fused_linear`: output[b, o] = sum_i weight[selected_experts[b], o, i] * input[b, i]
with rows pre-sorted by expert and `m_sizes[e]` rows per expert.

Drop-in for qwen3_moe_fused/functional.py:64-79 of the reference.
"""
import torch

from .grouped_gemm.interface import grouped_gemm


def moe_fused_linear(input: torch.Tensor, weight: torch.Tensor, m_sizes: torch.Tensor) -> torch.Tensor:
    """
    Args:
        input: `(batch_size, in_features)`, rows sorted by expert.
        weight: `(num_experts, out_features, in_features)`.
        m_sizes: `(num_experts,)` integer row counts per expert; sums to `batch_size`.

    Returns:
        `(batch_size, out_features)` in the dtype of `input`.
    """
    return grouped_gemm(input, weight, m_sizes)
