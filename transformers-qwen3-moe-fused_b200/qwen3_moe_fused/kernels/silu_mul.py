"""h = silu(e) * g, its backward, and the in-place backward.

Drop-in for qwen3_moe_fused/kernels/silu_mul.py:114-174 of the reference, with the same
rounding points (SiLU in fp32 rounded to the storage dtype, products in the storage dtype).
"""
import torch

from .. import _lib


def _check(*ts: torch.Tensor) -> None:
    e = ts[0]
    assert e.is_cuda
    for t in ts:
        assert t.device == e.device
        assert t.is_contiguous()
        assert t.numel() == e.numel()
        assert t.dtype == e.dtype


def silu_mul_forward(e: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    _check(e, g)
    h = torch.empty_like(e)
    with torch.cuda.device(e.device):
        status = _lib.load().moe_silu_mul_fwd(
            _lib.ptr(e), _lib.ptr(g), _lib.ptr(h), e.numel(), _lib.float_code(e.dtype), _lib.stream_ptr(e.device)
        )
    _lib.check(status, "moe_silu_mul_fwd")
    return h


def silu_mul_backward(dh: torch.Tensor, e: torch.Tensor, g: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    _check(e, g, dh)
    de = torch.empty_like(e)
    dg = torch.empty_like(g)
    with torch.cuda.device(e.device):
        status = _lib.load().moe_silu_mul_bwd(
            _lib.ptr(dh), _lib.ptr(e), _lib.ptr(g), _lib.ptr(de), _lib.ptr(dg), e.numel(),
            _lib.float_code(e.dtype), _lib.stream_ptr(e.device),
        )
    _lib.check(status, "moe_silu_mul_bwd")
    return de, dg


def silu_mul_backward_inplace(dh: torch.Tensor, e: torch.Tensor, g: torch.Tensor) -> None:
    """dh, e, g are overwritten by h, de, dg."""
    _check(e, g, dh)
    with torch.cuda.device(e.device):
        status = _lib.load().moe_silu_mul_bwd_inplace(
            _lib.ptr(dh), _lib.ptr(e), _lib.ptr(g), e.numel(), _lib.float_code(e.dtype), _lib.stream_ptr(e.device)
        )
    _lib.check(status, "moe_silu_mul_bwd_inplace")


class SiluMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, e, g):
        ctx.save_for_backward(e, g)
        return silu_mul_forward(e, g)

    @staticmethod
    def backward(ctx, dh):
        e, g = ctx.saved_tensors
        return silu_mul_backward(dh.contiguous(), e, g)


silu_mul = SiluMul.apply
