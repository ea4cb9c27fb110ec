"""The C-ABI library: loads without a GPU, exports what include/moe_b200.h declares, and
rejects bad arguments before touching the device.  No kernel is launched here."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "moe_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(moe_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as entry

    entry.build()
    from qwen3_moe_fused import _lib

    return _lib.load()


def test_header_and_binding_agree(lib):
    from qwen3_moe_fused import _lib

    names = declared_functions()
    assert len(names) >= 20
    assert sorted(_lib.SIGNATURES) == names
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_version_and_status_strings(lib):
    assert lib.moe_b200_version() >= 1
    assert lib.moe_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.moe_status_string(code) not in (b"ok", b"unknown status")


def test_argument_errors_return_before_any_launch(lib):
    # dtype code 9 does not exist; negative sizes; NULL outputs
    assert lib.moe_sort_by_expert(None, 9, 4, 2, None, None, None, None, 0, None) == -1
    assert lib.moe_sort_by_expert(None, 3, -1, 2, None, None, None, None, 0, None) == -2
    assert lib.moe_sort_by_expert(None, 3, 4, 2, None, None, None, None, 0, None) == -3
    assert lib.moe_grouped_gemm_fwd(None, None, None, 3, None, 4, 4, 4, 2, 9, 1, None, 0, None) == -1
    assert lib.moe_grouped_gemm_fwd(None, None, None, 3, None, -4, 4, 4, 2, 1, 1, None, 0, None) == -2
    assert lib.moe_grouped_gemm_dw(None, None, None, 3, None, 4, 4, 4, 0, 1, 1, None, 0, None) == -2
    assert lib.moe_router_softmax_topk(None, 0, 4, 128, 64, 1, None, 0, None, None) == -2  # k > 32
    assert lib.moe_nf4_dequant(None, None, None, 48, None, 64, 1, None) == -2  # blocksize not 2^n
    assert lib.moe_silu_mul_fwd(None, None, None, -1, 1, None) == -2
    # expert-parallel and fused entry points
    assert lib.moe_ep_plan(None, 3, 0, 128, 0, 42, None, None, None, None, None, None, None, None, None) == -2  # 128 % 3
    assert lib.moe_ep_plan(None, 4, 0, 128, 0, 32, None, None, None, None, None, None, None, None, None) == -3
    assert lib.moe_ep_push_rows(None, 8, 64, None, 9, 4, None, None, 0, None, 1, 0, None, None) == -1
    assert lib.moe_ep_push_rows(None, 8, 64, None, 3, 4, None, None, 7, None, 1, 0, None, None) == -2  # first_expert >= E
    assert lib.moe_ep_push_rows(None, 8, 64, None, 3, 4, None, None, 0, None, 1, 0, None, None) == -3
    assert lib.moe_gate_up_silu_fwd(None, None, None, None, 3, None, 4, 4, 4, 2, 9, None, 0, None) == -1
    assert lib.moe_grouped_gemm_dx_nf4(None, None, None, None, 48, None, 3, None, 4, 4, 4, 2, 1, 1, None, 0, None) == -3
    assert lib.moe_grouped_gemm_fwd_scattered(None, None, None, 3, None, 2, None, None, -1, 4, 4, 2, 1, 1, None, 0, None) == -2
    assert lib.moe_expand_rows(None, None, 0, None, 4, 4, 1, None) == -2  # k <= 0


def test_sort_workspace_query(lib):
    assert lib.moe_sort_workspace_bytes(0, 128) == 128 * 4
    assert lib.moe_sort_workspace_bytes(2048, 128) == 2 * 128 * 4
    assert lib.moe_sort_workspace_bytes(2049, 128) == 3 * 128 * 4
    assert lib.moe_grouped_gemm_workspace_bytes(0, 65536, 1536, 2048, 128) == 3 * 128 * 128 + 128


def test_gemm_path_switch(lib):
    prev = lib.moe_set_gemm_path(1)
    assert lib.moe_get_gemm_path() == 1
    lib.moe_set_gemm_path(prev)
    assert lib.moe_get_gemm_path() == prev


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from qwen3_moe_fused import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("MOE_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.MoeB200Error):
        _lib.load()
    monkeypatch.delenv("MOE_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    assert _lib.load() is not None


def test_wrappers_reject_cpu_tensors():
    import torch

    from qwen3_moe_fused.functional import moe_fused_linear
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx

    with pytest.raises(AssertionError):
        moe_fused_linear(torch.zeros(4, 8), torch.zeros(2, 8, 8), torch.tensor([2, 2]))
    with pytest.raises(AssertionError):
        get_expert_counts_and_idx(torch.zeros(4, dtype=torch.int64), 2)
