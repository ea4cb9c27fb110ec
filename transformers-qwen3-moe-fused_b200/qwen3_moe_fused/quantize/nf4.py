"""NF4 (4-bit NormalFloat) weights in the bitsandbytes layout, without bitsandbytes.

Layout, as the reference's fused kernel reads it
(qwen3_moe_fused/grouped_gemm/forward_4bit.py:99-104, 142-153, 173-176):
  * the weight tensor is flattened; every `blocksize` consecutive values share one fp32
    `absmax`; value = code[index] * absmax
  * two 4-bit indices per byte, element 2j in the high nibble and 2j+1 in the low nibble
  * `code` is a 16-entry fp32 table handed to the kernels at run time.

`Nf4State` carries the attributes of a bitsandbytes `QuantState` that the reference's
call sites touch, so either object can be passed to `grouped_gemm_forward_4bit`,
`dequantize_4bit` here, and `fast_lora`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _lib


def nf4_code(device=None) -> torch.Tensor:
    """The 16 NF4 levels: equal-probability quantiles of N(0,1) on each side of an exact
    zero (8 positive steps, 7 negative), scaled to [-1, 1].  Built from the published
    construction with the 0.9677083 tail offset."""
    offset = 0.9677083

    def ppf(p: torch.Tensor) -> torch.Tensor:
        return math.sqrt(2.0) * torch.erfinv(2.0 * p - 1.0)

    pos = ppf(torch.linspace(offset, 0.5, 9, dtype=torch.float64)[:-1])
    neg = -ppf(torch.linspace(offset, 0.5, 8, dtype=torch.float64)[:-1])
    vals = torch.cat([pos, torch.zeros(1, dtype=torch.float64), neg]).sort().values
    vals = vals / vals.abs().max()
    return vals.to(torch.float32).to(device) if device is not None else vals.to(torch.float32)


@dataclass
class Nf4State:
    absmax: torch.Tensor  # (numel / blocksize,) fp32
    code: torch.Tensor  # (16,) fp32
    blocksize: int
    shape: torch.Size
    dtype: torch.dtype  # dtype the weight is decoded to
    quant_type: str = "nf4"
    nested: bool = False
    state2: Optional[object] = None
    offset: Optional[torch.Tensor] = None


@dataclass
class AbsmaxState:
    """Second-level state of a double-quantised absmax (the attributes of a bitsandbytes
    `QuantState.state2` that the decode reads)."""
    absmax: torch.Tensor  # (n_blocks / blocksize,) fp32
    code: torch.Tensor  # (256,) fp32 levels in [-1, 1], ascending
    blocksize: int


@torch.no_grad()
def nest_absmax(state: Nf4State, blocksize2: int = 256) -> Nf4State:
    """Double quantisation of `state.absmax`: subtract the mean, then 8-bit blockwise absmax
    quantisation to the nearest of 256 evenly spaced levels.  (bitsandbytes uses a non-uniform
    256-level table; the decode takes the table as data, so either works.)"""
    absmax = state.absmax.float()
    assert absmax.numel() % blocksize2 == 0
    offset = absmax.mean()
    centred = (absmax - offset).reshape(-1, blocksize2)
    absmax2 = centred.abs().amax(dim=1).clamp_min(torch.finfo(torch.float32).tiny)
    code = torch.linspace(-1.0, 1.0, 256, device=absmax.device, dtype=torch.float32)
    q = torch.round((centred / absmax2.unsqueeze(1) + 1.0) * 127.5).clamp(0, 255).to(torch.uint8)
    return Nf4State(absmax=q.reshape(-1).contiguous(), code=state.code, blocksize=state.blocksize, shape=state.shape,
                    dtype=state.dtype, nested=True, state2=AbsmaxState(absmax2.contiguous(), code, blocksize2),
                    offset=offset.reshape(1))


@torch.no_grad()
def quantize_nf4(weight: torch.Tensor, blocksize: int = 64) -> tuple[torch.Tensor, Nf4State]:
    """Blockwise absmax NF4 quantisation: each value maps to the nearest table level of
    value / absmax.  Returns (packed uint8 of numel/2 bytes shaped (numel/2, 1), state)."""
    assert weight.numel() % blocksize == 0 and blocksize % 2 == 0
    code = nf4_code(weight.device)
    flat = weight.reshape(-1, blocksize).float()
    absmax = flat.abs().amax(dim=1)
    scaled = flat / absmax.clamp_min(torch.finfo(torch.float32).tiny).unsqueeze(1)
    # nearest level via the 15 midpoints between consecutive levels
    mids = (code[1:] + code[:-1]) / 2
    idx = torch.bucketize(scaled.reshape(-1), mids).to(torch.uint8)
    packed = (idx[0::2] << 4) | idx[1::2]
    state = Nf4State(absmax=absmax.contiguous(), code=code, blocksize=blocksize, shape=weight.shape, dtype=weight.dtype)
    return packed.reshape(-1, 1).contiguous(), state


def dequantize_4bit(packed: torch.Tensor, state, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Decodes an NF4 tensor on the device (stand-in for bitsandbytes' `dequantize_4bit`
    at qwen3_moe_fused/quantize/layer.py:21 and qwen3_moe_fused/kernels/fast_lora.py:62)."""
    from ..grouped_gemm.forward_4bit import _unnest_absmax

    assert state.quant_type == "nf4"
    assert packed.is_cuda and packed.is_contiguous()
    dtype = out_dtype or state.dtype
    absmax = _unnest_absmax(state).contiguous()
    n = 1
    for d in state.shape:
        n *= int(d)
    out = torch.empty(tuple(state.shape), device=packed.device, dtype=dtype)
    with torch.cuda.device(packed.device):
        status = _lib.load().moe_nf4_dequant(
            _lib.ptr(packed), _lib.ptr(state.code), _lib.ptr(absmax), int(state.blocksize), _lib.ptr(out), n,
            _lib.float_code(dtype), _lib.stream_ptr(packed.device),
        )
    _lib.check(status, "moe_nf4_dequant")
    return out
