"""4-bit `MoeFusedLinear` forward.

The reference (`moe_fused_linear_4bit`, qwen3_moe_fused/quantize/layer.py:17-22) decodes
the whole weight and then calls `moe_fused_linear`; its TODO asks for the fused form.
Here inference goes through the kernel that decodes NF4 tiles inside the GEMM, and the
decode-then-GEMM form is kept for the autograd path (dX needs the dense weight).
"""
import torch

from ..functional import moe_fused_linear
from ..grouped_gemm.forward_4bit import grouped_gemm_forward_4bit
from .nf4 import dequantize_4bit


def moe_fused_linear_4bit(input: torch.Tensor, weight_packed: torch.Tensor, quant_state, m_sizes: torch.Tensor,
                          fused: bool | None = None) -> torch.Tensor:
    """`weight_packed`/`quant_state`: NF4 weight of logical shape (E, out, in)."""
    if fused is None:
        fused = not (torch.is_grad_enabled() and input.requires_grad)
    if fused:
        return grouped_gemm_forward_4bit(input, weight_packed, quant_state, m_sizes)
    weight = dequantize_4bit(weight_packed, quant_state, input.dtype)
    return moe_fused_linear(input, weight, m_sizes)
