"""Forward grouped GEMM with the NF4 weight decoded inside the kernel.

Same contract as the reference's `grouped_gemm_forward_4bit`
(qwen3_moe_fused/grouped_gemm/forward_4bit.py:135-208).  `w_quant_state` is any object
with the bitsandbytes `QuantState` attributes that function reads: `quant_type`,
`blocksize`, `code`, `absmax`, `shape`, `nested` and, when nested, `state2` / `offset`
(`qwen3_moe_fused.quantize.nf4.Nf4State` provides them without bitsandbytes).
"""
from typing import Optional

import torch

from .. import _lib
from .forward import is_int_tensor


def _unnest_absmax(state) -> torch.Tensor:
    """fp32 absmax per block.  A double-quantised ("nested") absmax is expanded by one kernel of
    this library (qwen3_moe_fused/grouped_gemm/forward_4bit.py:149-153 of the reference calls
    bitsandbytes for it): `state.absmax` holds one byte per block, `state.state2` the 256-level
    table `code`, its own fp32 `absmax` and `blocksize`, `state.offset` the mean that was
    subtracted.  Works on a bitsandbytes `QuantState` and on `quantize.nf4.Nf4State` alike."""
    absmax = state.absmax
    if not getattr(state, "nested", False):
        return absmax
    state2 = state.state2
    q = absmax.contiguous()
    assert q.is_cuda and q.dtype == torch.uint8
    code2 = state2.code.to(device=q.device, dtype=torch.float32).contiguous()
    absmax2 = state2.absmax.to(device=q.device, dtype=torch.float32).contiguous()
    assert code2.numel() == 256
    offset = state.offset
    if offset is not None:
        offset = torch.as_tensor(offset, dtype=torch.float32, device=q.device).reshape(1).contiguous()
    out = torch.empty(q.numel(), device=q.device, dtype=torch.float32)
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().moe_absmax_unnest(
            _lib.ptr(q), _lib.ptr(code2), _lib.ptr(absmax2), int(state2.blocksize), _lib.ptr(offset), _lib.ptr(out),
            q.numel(), _lib.stream_ptr(q.device)), "moe_absmax_unnest")
    return out


# Rows per expert (on average) from which decoding the whole weight once and running the dense
# kernel is faster than decoding tiles inside the GEMM: the fused kernel decodes a weight tile
# once per 256-token tile, so its decode work grows with the rows, while the one-off decode costs
# about 0.2 ms per 800 MB of 16-bit weight.  Measured crossover on B200 at (128, 1536, 2048):
# about 1400 rows per expert.
DECODE_ONCE_ROWS_PER_EXPERT = 1400


def grouped_gemm_forward_4bit(
    x: torch.Tensor,
    w_quant: torch.Tensor,
    w_quant_state,
    m_sizes: torch.Tensor,
    dtype: Optional[torch.dtype] = None,
    fused: Optional[bool] = None,
) -> torch.Tensor:
    """`fused`: True = decode inside the GEMM, False = decode the whole weight, then the dense
    kernel; None = by the number of rows per expert (see DECODE_ONCE_ROWS_PER_EXPERT)."""
    assert w_quant_state.quant_type == "nf4"
    blocksize = int(w_quant_state.blocksize)
    assert blocksize > 0 and blocksize & (blocksize - 1) == 0

    w_code = w_quant_state.code
    assert w_code.dtype == torch.float32
    w_absmax = _unnest_absmax(w_quant_state)
    assert w_absmax.dtype == torch.float32

    assert x.is_cuda
    assert w_quant.device == x.device
    assert w_code.device == x.device
    assert w_absmax.device == x.device
    assert m_sizes.device == x.device
    assert is_int_tensor(w_quant)
    assert is_int_tensor(m_sizes)
    assert x.is_contiguous()
    assert w_quant.is_contiguous()
    assert w_code.is_contiguous()
    assert w_absmax.is_contiguous()
    assert m_sizes.is_contiguous()
    assert x.ndim == 2
    assert len(w_quant_state.shape) == 3
    assert m_sizes.ndim == 1
    M, K = x.shape
    E, N, _ = w_quant_state.shape
    assert w_quant_state.shape[2] == K
    assert K % 2 == 0
    assert E * N * K % blocksize == 0
    assert w_quant.numel() * w_quant.element_size() == E * N * K // 2
    assert w_absmax.numel() == E * N * K // blocksize
    assert w_code.numel() == 16
    assert m_sizes.numel() == E

    if dtype is None:
        dtype = x.dtype
    if fused is None:
        fused = M < DECODE_ONCE_ROWS_PER_EXPERT * E or x.dtype == torch.float32
    if not fused:
        from ..quantize.nf4 import dequantize_4bit
        from .forward import grouped_gemm_forward

        return grouped_gemm_forward(x, dequantize_4bit(w_quant, w_quant_state, x.dtype), m_sizes, dtype)
    y = torch.empty((M, N), device=x.device, dtype=dtype)
    lib = _lib.load()
    m_sizes = _lib.as_index_tensor(m_sizes)
    ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(0, M, N, K, E))
    with torch.cuda.device(x.device):
        status = lib.moe_grouped_gemm_fwd_nf4(
            _lib.ptr(x), _lib.ptr(w_quant), _lib.ptr(w_code), _lib.ptr(w_absmax), blocksize,
            _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype), _lib.ptr(y), M, N, K, E,
            _lib.float_code(x.dtype), _lib.float_code(dtype), ws_ptr, ws_bytes, _lib.stream_ptr(x.device),
        )
    _lib.check(status, "moe_grouped_gemm_fwd_nf4")
    return y


def grouped_gemm_forward_transposed_4bit(
    x: torch.Tensor,
    w_quant: torch.Tensor,
    w_quant_state,
    m_sizes: torch.Tensor,
    dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """dX through an NF4 weight: y[m, i] = sum_o w[e(m), o, i] * x[m, o] with the NF4 tensor of
    logical shape (E, out, in) decoded inside the kernel; x (M, out), y (M, in).

    The reference has no such kernel (its backward decodes the whole weight first,
    qwen3_moe_fused/kernels/fast_lora.py:57-63,128); shapes the fused kernel does not cover
    take that route here too: decode, then `grouped_gemm_forward_transposed`."""
    assert w_quant_state.quant_type == "nf4"
    blocksize = int(w_quant_state.blocksize)
    w_code = w_quant_state.code
    w_absmax = _unnest_absmax(w_quant_state)
    assert x.is_cuda and x.is_contiguous() and x.ndim == 2
    assert w_quant.is_contiguous() and w_code.is_contiguous() and w_absmax.is_contiguous() and m_sizes.is_contiguous()
    assert is_int_tensor(w_quant) and is_int_tensor(m_sizes)
    M, K = x.shape
    E, k_w, N = w_quant_state.shape
    assert k_w == K and m_sizes.numel() == E
    assert w_quant.numel() * w_quant.element_size() == E * N * K // 2
    if dtype is None:
        dtype = x.dtype
    y = torch.empty((M, N), device=x.device, dtype=dtype)
    lib = _lib.load()
    m_sizes = _lib.as_index_tensor(m_sizes)
    ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(1, M, N, K, E))
    with torch.cuda.device(x.device):
        status = lib.moe_grouped_gemm_dx_nf4(
            _lib.ptr(x), _lib.ptr(w_quant), _lib.ptr(w_code), _lib.ptr(w_absmax), blocksize,
            _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype), _lib.ptr(y), M, N, K, E,
            _lib.float_code(x.dtype), _lib.float_code(dtype), ws_ptr, ws_bytes, _lib.stream_ptr(x.device),
        )
    if status == _lib.ERR_UNSUPPORTED:
        from ..quantize.nf4 import dequantize_4bit
        from .forward_transposed import grouped_gemm_forward_transposed

        return grouped_gemm_forward_transposed(x, dequantize_4bit(w_quant, w_quant_state, x.dtype), m_sizes, dtype)
    _lib.check(status, "moe_grouped_gemm_dx_nf4")
    return y
