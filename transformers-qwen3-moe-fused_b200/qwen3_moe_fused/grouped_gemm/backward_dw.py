"""w[e, n, k] = sum_{m in group e} y[m, n] * x[m, k]: the weight gradient.

Same contract as the reference's `grouped_gemm_backward_dw`
(qwen3_moe_fused/grouped_gemm/backward_dw.py:92-134).  Experts without rows receive
zeros from the kernel itself, so the output is allocated uninitialised.
"""
import torch

from .forward import _launch, is_int_tensor


def grouped_gemm_backward_dw(
    x: torch.Tensor, y: torch.Tensor, m_sizes: torch.Tensor, dtype: torch.dtype
) -> torch.Tensor:
    assert x.is_cuda
    assert y.device == x.device
    assert m_sizes.device == x.device
    assert is_int_tensor(m_sizes)
    assert x.is_contiguous()
    assert y.is_contiguous()
    assert m_sizes.is_contiguous()
    assert x.ndim == 2
    assert y.ndim == 2
    assert m_sizes.ndim == 1
    assert y.dtype == x.dtype
    M, K = x.shape
    _, N = y.shape
    assert y.shape[0] == M
    E = m_sizes.numel()

    w = torch.empty((E, N, K), device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        _launch("moe_grouped_gemm_dw", 2, x, y, m_sizes, w, M, N, K, E)
    return w
