"""y[m, n] = sum_k w[s[m], k, n] * x[m, k]: the input gradient of `grouped_gemm_forward`.

Same contract as the reference's `grouped_gemm_forward_transposed`
(qwen3_moe_fused/grouped_gemm/forward_transposed.py:107-151).  The weight is read in
place through an MN-major shared-memory descriptor; no transposed copy is made.
"""
from typing import Optional

import torch

from .forward import _launch, is_int_tensor


def grouped_gemm_forward_transposed(
    x: torch.Tensor, w: torch.Tensor, m_sizes: torch.Tensor, dtype: Optional[torch.dtype] = None
) -> torch.Tensor:
    assert x.is_cuda
    assert w.device == x.device
    assert m_sizes.device == x.device
    assert is_int_tensor(m_sizes)
    assert x.is_contiguous()
    assert w.is_contiguous()
    assert m_sizes.is_contiguous()
    assert x.ndim == 2
    assert w.ndim == 3
    assert m_sizes.ndim == 1
    assert w.dtype == x.dtype
    M, K = x.shape
    E, _, N = w.shape
    assert w.shape[1] == K
    assert m_sizes.numel() == E

    if dtype is None:
        dtype = x.dtype
    y = torch.empty((M, N), device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        _launch("moe_grouped_gemm_dx", 1, x, w, m_sizes, y, M, N, K, E)
    return y
