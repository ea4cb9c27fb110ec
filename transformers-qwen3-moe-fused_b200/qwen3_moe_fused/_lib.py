"""ctypes binding of libmoe_b200.so (declared in include/moe_b200.h).

The library is the only implementation of the kernels: if it is missing, loading it
raises.  There is no fallback to torch or to the CPU.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

F32, BF16, F16, I32, I64 = 0, 1, 2, 3, 4
ERR_UNSUPPORTED = -5  # MOE_ERR_UNSUPPORTED: the selected kernel family does not cover the request
PATH_AUTO, PATH_SIMT, PATH_TC, PATH_TC_SINGLE = 0, 1, 2, 3

_FLOAT_CODES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}
_INT_CODES = {torch.int32: I32, torch.int64: I64}

_LIB_PATH = Path(__file__).resolve().parent / "libmoe_b200.so"

# name -> (restype, argtypes); mirrors include/moe_b200.h one to one
_P, _I, _L, _Z = c_void_p, c_int, c_int64, c_size_t
SIGNATURES = {
    "moe_b200_version": (_I, []),
    "moe_status_string": (c_char_p, [_I]),
    "moe_set_gemm_path": (_I, [_I]),
    "moe_get_gemm_path": (_I, []),
    "moe_sort_workspace_bytes": (_Z, [_L, _I]),
    "moe_sort_by_expert": (_I, [_P, _I, _L, _I, _P, _P, _P, _P, _Z, _P]),
    "moe_sort_static_capacity_bytes": (_Z, []),
    "moe_sort_by_expert_static": (_I, [_P, _I, _L, _I, _P, _P, _P, _P]),
    "moe_batch_begins_ends": (_I, [_P, _I, _L, _I, _P, _P]),
    "moe_grouped_gemm_workspace_bytes": (_Z, [_I, _L, _I, _I, _I]),
    "moe_grouped_gemm_fwd": (_I, [_P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_dx": (_I, [_P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_dw": (_I, [_P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_gate_up_silu_fwd": (_I, [_P, _P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_gate_up_silu_fwd_gather": (_I, [_P, _L, _P, _I, _P, _P, _P, _I, _P, _L, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_fwd_gather": (_I, [_P, _L, _P, _I, _P, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_fwd_nf4": (_I, [_P, _P, _P, _P, _I, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_dx_nf4": (_I, [_P, _P, _P, _P, _I, _P, _I, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_nf4_dequant": (_I, [_P, _P, _P, _I, _P, _L, _I, _P]),
    "moe_absmax_unnest": (_I, [_P, _P, _P, _I, _P, _P, _L, _P]),
    "moe_silu_mul_fwd": (_I, [_P, _P, _P, _L, _I, _P]),
    "moe_silu_mul_bwd": (_I, [_P, _P, _P, _P, _P, _L, _I, _P]),
    "moe_silu_mul_bwd_inplace": (_I, [_P, _P, _P, _L, _I, _P]),
    "moe_router_softmax_topk": (_I, [_P, _I, _L, _I, _I, _I, _P, _I, _P, _P]),
    "moe_gather_rows": (_I, [_P, _P, _I, _P, _L, _I, _I, _P]),
    "moe_expand_rows": (_I, [_P, _P, _I, _P, _L, _I, _I, _P]),
    "moe_combine": (_I, [_P, _P, _P, _P, _L, _I, _I, _I, _P]),
    "moe_ep_plan": (_I, [_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "moe_ep_push_rows": (_I, [_P, _L, _L, _P, _I, _I, _P, _P, _I, _P, _I, _I, _P, _P]),
    "moe_ep_token_positions": (_I, [_P, _I, _L, _I, _I, _I, _P, _P, _P]),
    "moe_ep_push_tokens": (_I, [_P, _L, _L, _P, _P, _I, _I, _P, _I, _I, _P, _P]),
    "moe_ep_push_index": (_I, [_P, _P, _I, _P, _I, _L, _P, _I, _I, _P, _P, _P, _P]),
    "moe_ep_expand_rows": (_I, [_P, _L, _L, _P, _P, _L, _P, _P]),
    "moe_grouped_gemm_fwd_scattered": (_I, [_P, _P, _P, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_grouped_gemm_dx_scattered": (_I, [_P, _P, _P, _I, _P, _I, _P, _P, _L, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "moe_debug_read_error": (_I, [_P, _I]),
    "moe_debug_read_late_values": (_I, [_P]),
    "moe_debug_last_detail": (c_char_p, []),
}

_lib = None


class MoeB200Error(RuntimeError):
    pass


def lib_path() -> Path:
    return Path(os.environ.get("MOE_B200_LIB", _LIB_PATH))


def load() -> ctypes.CDLL:
    """Loads the shared library once and declares every prototype."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not path.exists():
            raise MoeB200Error(
                f"{path} not found: build it with `python build.py` in the package root "
                "(there is no fallback implementation)"
            )
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().moe_status_string(status).decode()
        detail = load().moe_debug_last_detail().decode()
        raise MoeB200Error(f"{what} failed with status {status}: {msg}" + (f" [{detail}]" if detail else ""))


def float_code(dtype: torch.dtype) -> int:
    try:
        return _FLOAT_CODES[dtype]
    except KeyError:
        raise MoeB200Error(f"unsupported floating dtype {dtype}") from None


def int_code(dtype: torch.dtype) -> int:
    try:
        return _INT_CODES[dtype]
    except KeyError:
        raise MoeB200Error(f"unsupported integer dtype {dtype}") from None


def as_index_tensor(t: torch.Tensor) -> torch.Tensor:
    """int32/int64 tensors pass through; other integer dtypes are widened on the device."""
    if t.dtype in _INT_CODES:
        return t
    return t.to(torch.int32)


def ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    return t.data_ptr() if t.numel() > 0 else None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_WORKSPACES: dict = {}


def workspace(device: torch.device, nbytes: int) -> tuple[int | None, int]:
    """(128-byte aligned device address, nbytes) of scratch memory for a launch on the current stream of
    `device`.  One buffer per (device, stream) is kept and grown on demand instead of allocating per
    call: launches on one stream run in order, so the next launch may overwrite the scratch of the
    previous one; launches on different streams get different buffers."""
    if nbytes <= 0:
        return None, 0
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr(device))
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes + 128:
        buf = torch.empty(max(nbytes + 128, 1 << 16), device=device, dtype=torch.uint8)
        _WORKSPACES[key] = buf
    return (buf.data_ptr() + 127) & ~127, nbytes


def is_int_tensor(x: torch.Tensor) -> bool:
    return x.dtype in {torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64}


def set_gemm_path(path: int) -> int:
    return load().moe_set_gemm_path(path)


def read_late_values() -> int:
    v = ctypes.c_int(0)
    check(load().moe_debug_read_late_values(ctypes.addressof(v)), "moe_debug_read_late_values")
    return v.value


def read_error_flag(clear: bool = True) -> int:
    flag = ctypes.c_int(0)
    check(load().moe_debug_read_error(ctypes.addressof(flag), int(clear)), "moe_debug_read_error")
    return flag.value
