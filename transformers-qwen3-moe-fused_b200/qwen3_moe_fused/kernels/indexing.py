"""Expert histogram and stable sort-by-expert on the device.

Drop-in for qwen3_moe_fused/kernels/indexing.py of the reference: same function names,
argument order, return order and int32 outputs.  The reference builds an E x M compare
matrix; here one histogram -> scan -> stable-scatter pass over the ids produces
bit-identical results.
"""
import torch

from .. import _lib


def _prepare(s: torch.Tensor) -> torch.Tensor:
    assert s.is_cuda
    assert s.ndim == 1
    assert _lib.is_int_tensor(s)
    return _lib.as_index_tensor(s.contiguous())


def _sort(s: torch.Tensor, E: int, want_idx: bool):
    s = _prepare(s)
    M = s.numel()
    lib = _lib.load()
    counts = torch.empty(E, device=s.device, dtype=torch.int32)
    idx = inv_idx = None
    if want_idx:
        idx = torch.empty(M, device=s.device, dtype=torch.int32)
        inv_idx = torch.empty(M, device=s.device, dtype=torch.int32)
    ws_bytes = lib.moe_sort_workspace_bytes(M, E)
    ws = torch.empty(ws_bytes, device=s.device, dtype=torch.uint8)
    with torch.cuda.device(s.device):
        status = lib.moe_sort_by_expert(
            _lib.ptr(s), _lib.int_code(s.dtype), M, E, counts.data_ptr(),
            inv_idx.data_ptr() if want_idx else None, idx.data_ptr() if want_idx else None,
            ws.data_ptr(), ws_bytes, _lib.stream_ptr(s.device),
        )
    _lib.check(status, "moe_sort_by_expert")
    return counts, inv_idx, idx


@torch.no_grad()
def get_batch_begins_ends(s: torch.Tensor, E: int) -> torch.Tensor:
    """(E, 2) int32: rows with id < e and rows with id <= e (s is assumed sorted).
    Reference: qwen3_moe_fused/kernels/indexing.py:7-14."""
    s = _prepare(s)
    out = torch.empty((E, 2), device=s.device, dtype=torch.int32)
    with torch.cuda.device(s.device):
        status = _lib.load().moe_batch_begins_ends(
            _lib.ptr(s), _lib.int_code(s.dtype), s.numel(), E, out.data_ptr(), _lib.stream_ptr(s.device)
        )
    _lib.check(status, "moe_batch_begins_ends")
    return out


@torch.no_grad()
def get_expert_counts(s: torch.Tensor, E: int) -> torch.Tensor:
    """(E,) int32 rows per expert.  Reference: qwen3_moe_fused/kernels/indexing.py:18-23."""
    return _sort(s, E, want_idx=False)[0]


@torch.no_grad()
def sort_experts(s: torch.Tensor, E: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(s_sorted, inv_idx, idx), all int32.  Reference: qwen3_moe_fused/kernels/indexing.py:27-45."""
    counts, inv_idx, idx = _sort(s, E, want_idx=True)
    # ids in sorted order are read back through the gather index: no second sort
    s_sorted = s.to(torch.int32)[inv_idx.long()] if s.numel() else s.to(torch.int32)
    return s_sorted, inv_idx, idx


@torch.no_grad()
def get_expert_counts_and_idx(s: torch.Tensor, E: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(counts, inv_idx, idx), all int32; `x[inv_idx]` sorts rows by expert and `y[idx]`
    undoes it.  Reference: qwen3_moe_fused/kernels/indexing.py:48-65."""
    return _sort(s, E, want_idx=True)
