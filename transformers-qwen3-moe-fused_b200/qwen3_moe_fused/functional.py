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


# ------------------------------------------------------------------------------------------
# The operation's definition in plain torch, on unsorted rows with one expert id per row.
# The reference keeps these three next to `moe_fused_linear` (qwen3_moe_fused/functional.py:7-61)
# and its tests and benchmarks import them from this module as the thing the kernels are compared
# with (test_moe_fused_linear.py:47, test_moe_fused_linear_bwd.py:8-13,49-59), so they exist here
# under the same names, arguments and dtypes.  They run on whatever device their tensors are on and
# nothing in this package calls them: they are a yardstick, not a code path.
# ------------------------------------------------------------------------------------------
_NAIVE_ROWS_PER_STEP = 1024  # rows whose expert matrices are gathered at once (bounds the temporary)


def _moe_fused_linear_naive_fwd(input: torch.Tensor, weight: torch.Tensor, selected_experts: torch.Tensor) -> torch.Tensor:
    """output[b, o] = sum_i weight[selected_experts[b], o, i] * input[b, i]; (batch, out) in input's dtype."""
    batch = input.shape[0]
    output = input.new_empty((batch, weight.shape[1]))
    for a in range(0, batch, _NAIVE_ROWS_PER_STEP):
        rows = slice(a, min(a + _NAIVE_ROWS_PER_STEP, batch))
        per_row = weight[selected_experts[rows].long()]                       # (rows, out, in)
        output[rows] = torch.bmm(per_row, input[rows].unsqueeze(2)).squeeze(2)
    return output


def _moe_fused_linear_naive_bwd_input(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
                                      selected_experts: torch.Tensor) -> torch.Tensor:
    """grad_input[b, i] = sum_o weight[selected_experts[b], o, i] * grad_output[b, o]; shaped like input."""
    batch = input.shape[0]
    grad_input = torch.empty_like(input)
    for a in range(0, batch, _NAIVE_ROWS_PER_STEP):
        rows = slice(a, min(a + _NAIVE_ROWS_PER_STEP, batch))
        per_row = weight[selected_experts[rows].long()]
        grad_input[rows] = torch.bmm(grad_output[rows].unsqueeze(1), per_row).squeeze(1)
    return grad_input


def _moe_fused_linear_naive_bwd_weight(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
                                       selected_experts: torch.Tensor) -> torch.Tensor:
    """grad_weight[e, o, i] = sum over rows b with selected_experts[b] == e of grad_output[b, o] * input[b, i];
    shaped like weight, zeros for experts without rows."""
    batch = input.shape[0]
    grad_weight = torch.zeros_like(weight)
    for a in range(0, batch, _NAIVE_ROWS_PER_STEP):
        rows = slice(a, min(a + _NAIVE_ROWS_PER_STEP, batch))
        outer = grad_output[rows].unsqueeze(2) * input[rows].unsqueeze(1)     # (rows, out, in)
        grad_weight.index_add_(0, selected_experts[rows].long(), outer.to(grad_weight.dtype))
    return grad_weight
