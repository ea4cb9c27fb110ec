"""Autograd wrapper of the grouped GEMM.

Same behaviour as the reference's `GroupedGemm`
(qwen3_moe_fused/grouped_gemm/interface.py:8-31): dX only when the input needs a
gradient, dW only when the weight does; gradients in the dtype of their operand.
"""
import torch

from .backward_dw import grouped_gemm_backward_dw
from .forward import grouped_gemm_forward
from .forward_transposed import grouped_gemm_forward_transposed


class GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, m_sizes):
        ctx.save_for_backward(x, w, m_sizes)
        return grouped_gemm_forward(x, w, m_sizes)

    @staticmethod
    def backward(ctx, dy):
        x, w, m_sizes = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        dx = grouped_gemm_forward_transposed(dy, w, m_sizes, x.dtype) if ctx.needs_input_grad[0] else None
        dw = grouped_gemm_backward_dw(x, dy, m_sizes, w.dtype) if ctx.needs_input_grad[1] else None
        return dx, dw, None


grouped_gemm = GroupedGemm.apply
