"""y[m, n] = sum_k w[s[m], n, k] * x[m, k] with rows grouped by expert.

Same contract as the reference's `grouped_gemm_forward`
(qwen3_moe_fused/grouped_gemm/forward.py:116-160): identical argument checks, output
allocated with torch, kernel enqueued on the current CUDA stream, `m_sizes` never read
on the host.
"""
from typing import Optional

import torch

from .. import _lib
from .._lib import is_int_tensor  # re-exported: the reference defines it here


def _launch(name: str, which: int, a, b, m_sizes, out, M: int, N: int, K: int, E: int) -> None:
    lib = _lib.load()
    m_sizes = _lib.as_index_tensor(m_sizes)
    fn = getattr(lib, name)
    # scratch for the per-expert tensor maps the tensor-core kernels derive from m_sizes
    ws_ptr, ws_bytes = _lib.workspace(a.device, lib.moe_grouped_gemm_workspace_bytes(which, M, N, K, E))
    status = fn(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype), _lib.ptr(out),
        M, N, K, E, _lib.float_code(a.dtype), _lib.float_code(out.dtype), ws_ptr, ws_bytes,
        _lib.stream_ptr(a.device),
    )
    _lib.check(status, name)


def grouped_gemm_forward(
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
    E, N, _ = w.shape
    assert w.shape[2] == K
    assert m_sizes.numel() == E

    if dtype is None:
        dtype = x.dtype
    y = torch.empty((M, N), device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        _launch("moe_grouped_gemm_fwd", 0, x, w, m_sizes, y, M, N, K, E)
    return y


@torch.no_grad()
def grouped_gemm_forward_gather(x: torch.Tensor, row_index: torch.Tensor, index_div: int, w: torch.Tensor,
                                m_sizes: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """`grouped_gemm_forward(x[row_index // index_div], w, m_sizes)` without materialising the gathered rows:
    x is the (T, K) token tensor, row_index (int32, M entries) names the token of every sorted row, and the
    kernel's token load gathers the rows (TMA gather4).  No counterpart in the reference, which gathers
    first (qwen3_moe_fused/modular_qwen3_moe_fused.py:95-103); same result bit for bit."""
    assert x.is_cuda and x.is_contiguous() and w.is_contiguous() and x.ndim == 2 and w.ndim == 3 and w.dtype == x.dtype
    assert row_index.dtype == torch.int32 and row_index.is_contiguous() and row_index.device == x.device
    assert is_int_tensor(m_sizes) and m_sizes.is_contiguous() and m_sizes.numel() == w.shape[0]
    M, K = row_index.numel(), x.shape[1]
    E, N, _ = w.shape
    assert w.shape[2] == K
    dtype = dtype or x.dtype
    lib = _lib.load()
    m_sizes = _lib.as_index_tensor(m_sizes)
    y = torch.empty((M, N), device=x.device, dtype=dtype)
    with torch.cuda.device(x.device):
        ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(0, M, N, K, E))
        status = lib.moe_grouped_gemm_fwd_gather(
            _lib.ptr(x), x.shape[0], _lib.ptr(row_index), index_div, _lib.ptr(w), _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype),
            _lib.ptr(y), M, N, K, E, _lib.float_code(x.dtype), _lib.float_code(dtype), ws_ptr, ws_bytes, _lib.stream_ptr(x.device))
    if status == _lib.ERR_UNSUPPORTED:  # shapes / dtypes outside the CTA-pair kernels: gather, then the general path
        from ..kernels.routing import _gather_rows

        return grouped_gemm_forward(_gather_rows(x, row_index, index_div), w, m_sizes, dtype)
    _lib.check(status, "moe_grouped_gemm_fwd_gather")
    return y
