"""Sort-by-expert kernels through the C ABI vs the oracle: bit-exact."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _run(s_np, E, dtype, cuda):
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx

    s = torch.from_numpy(s_np).to(cuda, dtype)
    counts, inv_idx, idx = get_expert_counts_and_idx(s, E)
    assert counts.dtype == inv_idx.dtype == idx.dtype == torch.int32
    return counts.cpu().numpy(), inv_idx.cpu().numpy(), idx.cpu().numpy()


@pytest.mark.parametrize("name", ["c1", "ragged", "empty_groups", "single", "wide"])
def test_golden_vectors(golden, cuda, name):
    g = golden(f"indexing_{name}")
    counts, inv_idx, idx = _run(g["s"], int(g["E"]), torch.int64, cuda)
    np.testing.assert_array_equal(counts, g["counts"])
    np.testing.assert_array_equal(inv_idx, g["inv_idx"])
    np.testing.assert_array_equal(idx, g["idx"])


@pytest.mark.parametrize("M,E", [(0, 4), (1, 1), (31, 3), (2048, 128), (2049, 128), (65536, 128), (131072, 128),
                                 (100003, 257), (5000, 1024), (7, 4096)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_random_vs_oracle(cuda, M, E, dtype):
    rng = np.random.default_rng(M * 31 + E)
    s = rng.integers(0, E, M).astype(np.int64)
    counts, inv_idx, idx = _run(s, E, dtype, cuda)
    rc, rinv, ridx = O.get_expert_counts_and_idx_fast(s, E)
    np.testing.assert_array_equal(counts, rc)
    np.testing.assert_array_equal(inv_idx, rinv)
    np.testing.assert_array_equal(idx, ridx)


def test_skewed_and_all_one_expert(cuda):
    rng = np.random.default_rng(5)
    E = 128
    p = (np.arange(E) + 1.0) ** -1.2
    s = rng.choice(E, 65536, p=p / p.sum())
    for arr in (s, np.full(10000, 17), np.sort(s), np.sort(s)[::-1].copy()):
        counts, inv_idx, idx = _run(arr.astype(np.int64), E, torch.int64, cuda)
        rc, rinv, ridx = O.get_expert_counts_and_idx_fast(arr, E)
        np.testing.assert_array_equal(counts, rc)
        np.testing.assert_array_equal(inv_idx, rinv)
        np.testing.assert_array_equal(idx, ridx)


def test_other_int_dtypes_and_siblings(cuda):
    from qwen3_moe_fused.kernels.indexing import get_batch_begins_ends, get_expert_counts, sort_experts

    rng = np.random.default_rng(6)
    E = 11
    s = rng.integers(0, E, 999)
    for dt in (torch.uint8, torch.int16):
        counts = get_expert_counts(torch.from_numpy(s).to(cuda, dt), E)
        np.testing.assert_array_equal(counts.cpu().numpy(), O.get_expert_counts(s, E))
    s_sorted, inv_idx, idx = sort_experts(torch.from_numpy(s).to(cuda), E)
    rs, rinv, ridx = O.sort_experts(s, E)
    np.testing.assert_array_equal(s_sorted.cpu().numpy(), rs)
    np.testing.assert_array_equal(inv_idx.cpu().numpy(), rinv)
    np.testing.assert_array_equal(idx.cpu().numpy(), ridx)
    be = get_batch_begins_ends(torch.from_numpy(np.sort(s)).to(cuda), E)
    np.testing.assert_array_equal(be.cpu().numpy(), O.get_batch_begins_ends(np.sort(s), E))


def test_permutation_properties_at_full_size(cuda):
    # size-independent checks at the block workload (131072 rows): inverse permutations,
    # sortedness, stability
    rng = np.random.default_rng(7)
    E, M = 128, 131072
    s = torch.from_numpy(rng.integers(0, E, M)).to(cuda)
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx

    counts, inv_idx, idx = get_expert_counts_and_idx(s, E)
    assert int(counts.sum()) == M
    ar = torch.arange(M, device=cuda, dtype=torch.int32)
    assert torch.equal(inv_idx[idx.long()], ar) and torch.equal(idx[inv_idx.long()], ar)
    ss = s[inv_idx.long()]
    assert bool((ss[1:] >= ss[:-1]).all())
    same = ss[1:] == ss[:-1]
    assert bool((inv_idx[1:][same] > inv_idx[:-1][same]).all())
