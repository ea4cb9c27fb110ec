"""`moe_sort_by_expert_static`: the sort entry point for callers that cannot give the library
scratch memory (they may not call cudaMalloc where they call the sort, or have no allocator).
Its scratch is a fixed array inside the library, so this test calls it straight through the
C ABI, twice in a row (the second call finds the first call's leftovers in the array), and
requires the same counts and permutations as the workspace-taking entry point, bit for bit.
Collected last on purpose: a failure here cannot hide any other test's result."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, _lib, fn_static: bool, s: torch.Tensor, E: int):
    M = s.numel()
    dev = s.device
    counts = torch.empty(E, device=dev, dtype=torch.int32)
    inv_idx = torch.empty(M, device=dev, dtype=torch.int32)
    idx = torch.empty(M, device=dev, dtype=torch.int32)
    stream = _lib.stream_ptr(dev)
    if fn_static:
        st = lib.moe_sort_by_expert_static(s.data_ptr(), _lib.int_code(s.dtype), M, E, counts.data_ptr(),
                                           inv_idx.data_ptr(), idx.data_ptr(), stream)
    else:
        nbytes = lib.moe_sort_workspace_bytes(M, E)
        ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        st = lib.moe_sort_by_expert(s.data_ptr(), _lib.int_code(s.dtype), M, E, counts.data_ptr(), inv_idx.data_ptr(),
                                    idx.data_ptr(), ws.data_ptr(), nbytes, stream)
    _lib.check(st, "sort")
    torch.cuda.synchronize()
    return counts.cpu().numpy(), inv_idx.cpu().numpy(), idx.cpu().numpy()


def test_static_scratch_sort_matches_workspace_sort(cuda):
    from qwen3_moe_fused import _lib

    lib = _lib.load()
    assert lib.moe_sort_static_capacity_bytes() == 256 * 1024
    rng = np.random.default_rng(0)
    # two different problems back to back: the second runs on a dirty scratch array, and is
    # smaller than the first so stale histogram rows lie beyond what it uses
    for M, E, dtype in ((131072, 128, torch.int64), (5000, 11, torch.int32)):
        s = torch.from_numpy(rng.integers(0, E, M)).to(cuda, dtype)
        ref = _run(lib, _lib, False, s, E)
        for _ in range(2):
            got = _run(lib, _lib, True, s, E)
            for a, b in zip(got, ref):
                np.testing.assert_array_equal(a, b)


def test_static_scratch_rejects_oversized_problems(cuda):
    from qwen3_moe_fused import _lib

    lib = _lib.load()
    M, E = 1 << 22, 512  # needs (2048 + 1) * 512 * 4 bytes = 4 MB of scratch
    assert lib.moe_sort_workspace_bytes(M, E) > lib.moe_sort_static_capacity_bytes()
    s = torch.zeros(M, device=cuda, dtype=torch.int32)
    counts = torch.full((E,), -7, device=cuda, dtype=torch.int32)
    idx = torch.empty(M, device=cuda, dtype=torch.int32)
    st = lib.moe_sort_by_expert_static(s.data_ptr(), _lib.I32, M, E, counts.data_ptr(), idx.data_ptr(), idx.data_ptr(),
                                       _lib.stream_ptr(cuda))
    assert st == -4  # MOE_ERR_WORKSPACE, and nothing ran:
    torch.cuda.synchronize()
    assert bool((counts == -7).all())
    assert b"workspace" in lib.moe_status_string(st)
