"""Expert MLP with base weights (dense or NF4) plus LoRA on gate / up / down, as one
autograd function with a hand-written backward.

Drop-in for `fast_lora` of the reference (qwen3_moe_fused/kernels/fast_lora.py:66-175):
same 17 positional arguments, gradients for x and the six LoRA matrices only.

    e = G'x   g = U'x   h = silu(e) * g   y = W'h       with  V' = V + s * B A

Differences in how the same quantities are computed:
  * an NF4 base weight is decoded inside the forward GEMM (the reference decodes the
    whole tensor first, :96); the backward decodes it once per projection for dX;
  * LoRA gradients are formed in rank-r space,
        dA = s * (dy B)^T x        dB = s * dy^T (x A^T),
    i.e. two thin grouped GEMMs per matrix, instead of a full (E, out, in) weight-gradient
    GEMM followed by two einsum projections (:139-149).
"""
import torch

from ..grouped_gemm.backward_dw import grouped_gemm_backward_dw
from ..grouped_gemm.forward import grouped_gemm_forward
from ..grouped_gemm.forward_4bit import grouped_gemm_forward_4bit, grouped_gemm_forward_transposed_4bit
from ..grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
from ..quantize.nf4 import dequantize_4bit
from .silu_mul import silu_mul_backward_inplace, silu_mul_forward


def _dense(weight, quant_state, dtype):
    if quant_state is None:
        return weight if weight.dtype == dtype else weight.to(dtype)
    return dequantize_4bit(weight, quant_state, dtype)


class FastLora(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, Gq, Gqs, Ag, Bg, Sg, Uq, Uqs, Au, Bu, Su, Wq, Wqs, Aw, Bw, Sw, m_sizes):
        dt = x.dtype
        x = x.contiguous()
        Ag, Bg, Au, Bu, Aw, Bw = (t.to(dt).contiguous() for t in (Ag, Bg, Au, Bu, Aw, Bw))
        if Gqs is None:
            Gq = Gq.to(dt)
        if Uqs is None:
            Uq = Uq.to(dt)
        if Wqs is None:
            Wq = Wq.to(dt)

        def base(_x, _wq, _wqs):
            if _wqs is None:
                return grouped_gemm_forward(_x, _wq, m_sizes, dt)
            return grouped_gemm_forward_4bit(_x, _wq, _wqs, m_sizes, dt)

        def mv_lora(_x, _wq, _wqs, _a, _b, _s):
            _y = base(_x, _wq, _wqs)
            _y += grouped_gemm_forward(grouped_gemm_forward(_x, _a, m_sizes, dt), _b, m_sizes, dt) * _s
            return _y

        e = mv_lora(x, Gq, Gqs, Ag, Bg, Sg)
        g = mv_lora(x, Uq, Uqs, Au, Bu, Su)
        h = silu_mul_forward(e, g)
        y = mv_lora(h, Wq, Wqs, Aw, Bw, Sw)

        ctx.custom_saved_tensors = (Gq, Gqs, Sg, Uq, Uqs, Su, Wq, Wqs, Sw, m_sizes)
        ctx.save_for_backward(x, Ag, Bg, Au, Bu, Aw, Bw, e, g)
        return y

    @staticmethod
    def backward(ctx, dy):
        Gq, Gqs, Sg, Uq, Uqs, Su, Wq, Wqs, Sw, m_sizes = ctx.custom_saved_tensors
        x, Ag, Bg, Au, Bu, Aw, Bw, e, g = ctx.saved_tensors
        dt = x.dtype
        dy = dy.contiguous().to(dt)

        def vm(_x, _w):  # rows times (E, k, n) weight read transposed
            return grouped_gemm_forward_transposed(_x, _w, m_sizes, dt)

        def vm_base(_x, _wq, _wqs):  # the same through a base weight that may be NF4 (decoded inside the kernel)
            if _wqs is None:
                return vm(_x, _wq)
            return grouped_gemm_forward_transposed_4bit(_x, _wq, _wqs, m_sizes, dt)

        def mv(_x, _w):
            return grouped_gemm_forward(_x, _w, m_sizes, dt)

        def vv(_y, _x):  # per-expert _y^T _x
            return grouped_gemm_backward_dw(_x, _y, m_sizes, dt)

        # down projection
        dyB = vm(dy, Bw)  # (rows, r)
        dh = vm_base(dy, Wq, Wqs)
        dh += vm(dyB, Aw) * Sw
        # dh, e, g become h, de, dg
        silu_mul_backward_inplace(dh, e, g)
        h, de, dg = dh, e, g
        del dh, e, g

        dAw = vv(dyB, h) * Sw
        dBw = vv(dy, mv(h, Aw)) * Sw

        dgB = vm(dg, Bu)
        dAu = vv(dgB, x) * Su
        dBu = vv(dg, mv(x, Au)) * Su

        deB = vm(de, Bg)
        dAg = vv(deB, x) * Sg
        dBg = vv(de, mv(x, Ag)) * Sg

        dx = None
        if ctx.needs_input_grad[0]:
            dx = vm_base(de, Gq, Gqs)
            dx += vm(deB, Ag) * Sg
            dx += vm_base(dg, Uq, Uqs)
            dx += vm(dgB, Au) * Su

        return (dx, None, None, dAg, dBg, None, None, None, dAu, dBu, None, None, None, dAw, dBw, None, None)


fast_lora = FastLora.apply
