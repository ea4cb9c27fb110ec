"""4-bit `MoeFusedLinear` forward.

The reference (`moe_fused_linear_4bit`, qwen3_moe_fused/quantize/layer.py:17-22) decodes
the whole weight and then calls `moe_fused_linear`; its TODO asks for the fused form.
Here both directions go through kernels that decode NF4 tiles inside the GEMM: the forward,
and the gradient of the input (the 4-bit weight itself is frozen and gets no gradient).
"""
import torch

from ..functional import moe_fused_linear
from ..grouped_gemm.forward_4bit import grouped_gemm_forward_4bit, grouped_gemm_forward_transposed_4bit
from .nf4 import dequantize_4bit


class _FusedLinear4bit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight_packed, quant_state, m_sizes):
        ctx.quant_state = quant_state
        ctx.save_for_backward(weight_packed, m_sizes)
        return grouped_gemm_forward_4bit(input, weight_packed, quant_state, m_sizes)

    @staticmethod
    def backward(ctx, grad_output):
        weight_packed, m_sizes = ctx.saved_tensors
        dx = None
        if ctx.needs_input_grad[0]:
            dx = grouped_gemm_forward_transposed_4bit(grad_output.contiguous(), weight_packed, ctx.quant_state, m_sizes)
        return dx, None, None, None


def moe_fused_linear_4bit(input: torch.Tensor, weight_packed: torch.Tensor, quant_state, m_sizes: torch.Tensor,
                          fused: bool | None = None) -> torch.Tensor:
    """`weight_packed`/`quant_state`: NF4 weight of logical shape (E, out, in).
    `fused=False` selects the reference's decode-then-GEMM form."""
    if fused is None:
        fused = True
    if fused:
        if torch.is_grad_enabled() and input.requires_grad:
            return _FusedLinear4bit.apply(input, weight_packed, quant_state, m_sizes)
        return grouped_gemm_forward_4bit(input, weight_packed, quant_state, m_sizes)
    weight = dequantize_4bit(weight_packed, quant_state, input.dtype)
    return moe_fused_linear(input, weight, m_sizes)
