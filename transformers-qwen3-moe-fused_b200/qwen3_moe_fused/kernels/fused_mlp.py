"""Gate projection + up projection + SiLU-mul of the expert MLP in one kernel (inference).

What the reference block computes with two `moe_fused_linear` calls and `F.silu(gate_h) * up_h`
(qwen3_moe_fused/modular_qwen3_moe_fused.py:105-108), with the same rounding points, so the
result equals the three-kernel composition bit for bit; the two projections are never written.
"""
from typing import Optional

import torch

from .. import _lib
from ..grouped_gemm.forward import grouped_gemm_forward
from .silu_mul import silu_mul_forward


@torch.no_grad()
def gate_up_silu_forward(x: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor, m_sizes: torch.Tensor,
                         row_index: Optional[torch.Tensor] = None, index_div: int = 1) -> torch.Tensor:
    """x (M, K) rows sorted by expert; gate_proj / up_proj (E, I, K); returns h (M, I).

    With `row_index` (int32, M entries) x is the (T, K) TOKEN tensor and sorted row r is
    x[row_index[r] // index_div]: the gather happens inside the kernel's token load (TMA gather4), so
    the expanded, sorted copy of the tokens is never written."""
    assert x.is_cuda and x.is_contiguous() and gate_proj.is_contiguous() and up_proj.is_contiguous()
    assert gate_proj.shape == up_proj.shape and gate_proj.dtype == x.dtype == up_proj.dtype
    E, I, kw = gate_proj.shape
    K = x.shape[1]
    assert kw == K and m_sizes.numel() == E
    m_sizes = _lib.as_index_tensor(m_sizes).contiguous()
    lib = _lib.load()
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_contiguous() and row_index.device == x.device
        M = row_index.numel()
        if x.dtype in (torch.bfloat16, torch.float16) and M > 0:
            h = torch.empty((M, I), device=x.device, dtype=x.dtype)
            ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(0, M, I, K, E))
            with torch.cuda.device(x.device):
                status = lib.moe_gate_up_silu_fwd_gather(
                    _lib.ptr(x), x.shape[0], _lib.ptr(row_index), index_div, _lib.ptr(gate_proj), _lib.ptr(up_proj),
                    _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype), _lib.ptr(h), M, I, K, E, _lib.float_code(x.dtype),
                    ws_ptr, ws_bytes, _lib.stream_ptr(x.device))
            if status != _lib.ERR_UNSUPPORTED:
                _lib.check(status, "moe_gate_up_silu_fwd_gather")
                return h
        # not covered by the gathering kernel: gather first
        from .routing import _gather_rows

        x = _gather_rows(x, row_index, index_div)
    M = x.shape[0]
    if x.dtype in (torch.bfloat16, torch.float16) and M > 0:
        h = torch.empty((M, I), device=x.device, dtype=x.dtype)
        ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(0, M, I, K, E))
        with torch.cuda.device(x.device):
            status = lib.moe_gate_up_silu_fwd(
                _lib.ptr(x), _lib.ptr(gate_proj), _lib.ptr(up_proj), _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype),
                _lib.ptr(h), M, I, K, E, _lib.float_code(x.dtype), ws_ptr, ws_bytes, _lib.stream_ptr(x.device))
        if status != _lib.ERR_UNSUPPORTED:
            _lib.check(status, "moe_gate_up_silu_fwd")
            return h
    # shapes / dtypes the fused kernel does not cover: the three kernels it stands for
    return silu_mul_forward(grouped_gemm_forward(x, gate_proj, m_sizes), grouped_gemm_forward(x, up_proj, m_sizes))
