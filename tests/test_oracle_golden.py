"""The oracle against fixtures produced by the reference's own code (CPU only)."""
import numpy as np
import pytest

from oracle import moe_oracle as O


@pytest.mark.parametrize("name", ["c1", "ragged", "empty_groups", "single", "wide"])
def test_indexing_matches_reference(golden, name):
    g = golden(f"indexing_{name}")
    s, E = g["s"], int(g["E"])
    for fn in (O.get_expert_counts_and_idx, O.get_expert_counts_and_idx_fast):
        counts, inv_idx, idx = fn(s, E)
        assert counts.dtype == np.int32 and inv_idx.dtype == np.int32 and idx.dtype == np.int32
        np.testing.assert_array_equal(counts, g["counts"])
        np.testing.assert_array_equal(inv_idx, g["inv_idx"])
        np.testing.assert_array_equal(idx, g["idx"])
    s_sorted, inv2, idx2 = O.sort_experts(s, E)
    np.testing.assert_array_equal(s_sorted, g["s_sorted"])
    np.testing.assert_array_equal(inv2, g["inv_idx"])
    np.testing.assert_array_equal(O.get_expert_counts(s, E), g["counts"])
    np.testing.assert_array_equal(O.get_batch_begins_ends(np.sort(s), E), g["begins_ends"])


@pytest.mark.parametrize("name", ["c1", "odd", "empty"])
def test_linear_matches_reference(golden, name):
    g = golden(f"linear_{name}")
    x, w, s, dy = g["x"], g["w"], g["s"], g["dy"]
    E = w.shape[0]
    # literal row loops
    np.testing.assert_allclose(O.moe_fused_linear_fwd_rowloop(x, w, s), g["y"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.moe_fused_linear_bwd_input_rowloop(dy, w, s), g["dx"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.moe_fused_linear_bwd_weight_rowloop(dy, x, E, s), g["dw"], rtol=1e-4, atol=1e-4)
    # grouped form on sorted rows, un-sorted again
    m_sizes, inv_idx, idx = O.get_expert_counts_and_idx_fast(s, E)
    xs, dys = x[inv_idx], dy[inv_idx]
    np.testing.assert_allclose(O.grouped_gemm_fwd(xs, w, m_sizes)[idx], g["y"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.grouped_gemm_dx(dys, w, m_sizes)[idx], g["dx"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(O.grouped_gemm_dw(xs, dys, m_sizes), g["dw"], rtol=1e-4, atol=1e-4)


def test_block_matches_reference(golden):
    g = golden("block_tiny")
    hidden = g["hidden"].reshape(-1, g["hidden"].shape[-1])
    out, logits = O.moe_block_forward(hidden, g["gate"], g["gate_proj"], g["up_proj"], g["down_proj"], int(g["k"]))
    np.testing.assert_allclose(logits, g["logits"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(out, g["out"].reshape(out.shape), rtol=1e-4, atol=1e-5)


def test_plain_silu_mul_matches_torch():
    # plain path of the block: F.silu(gate) * up (modular_qwen3_moe_fused.py:108)
    import torch

    rng = np.random.default_rng(0)
    e = rng.standard_normal(4096).astype(np.float32) * 3
    g = rng.standard_normal(4096).astype(np.float32)
    ref = (torch.nn.functional.silu(torch.from_numpy(e)) * torch.from_numpy(g)).numpy()
    np.testing.assert_allclose(O.silu_mul_fwd(e, g), ref, rtol=1e-6, atol=1e-6)
    # backward against autograd
    et = torch.from_numpy(e).requires_grad_()
    gt = torch.from_numpy(g).requires_grad_()
    dh = rng.standard_normal(4096).astype(np.float32)
    (torch.nn.functional.silu(et) * gt).backward(torch.from_numpy(dh))
    h, de, dg = O.silu_mul_bwd(dh, e, g)
    np.testing.assert_allclose(de, et.grad.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dg, gt.grad.numpy(), rtol=1e-5, atol=1e-6)


def test_bf16_rounding_matches_torch():
    import torch

    rng = np.random.default_rng(1)
    x = (rng.standard_normal(100000) * 10 ** rng.uniform(-6, 6, 100000)).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(O.round_bf16(x), ref)


def test_router_matches_torch_when_untied():
    import torch

    rng = np.random.default_rng(2)
    logits = rng.standard_normal((512, 128)).astype(np.float32)
    w, idx = O.router_softmax_topk(logits, 8, True)
    p = torch.softmax(torch.from_numpy(logits), dim=1, dtype=torch.float32)
    tw, ti = torch.topk(p, 8, dim=-1)
    tw = tw / tw.sum(dim=-1, keepdim=True)
    np.testing.assert_array_equal(idx, ti.numpy())
    np.testing.assert_allclose(w, tw.numpy(), rtol=1e-5)


def test_router_tie_rule():
    logits = np.zeros((1, 8), np.float32)
    logits[0, [5, 2]] = 1.0
    _, idx = O.router_softmax_topk(logits, 4, True)
    np.testing.assert_array_equal(idx[0], [2, 5, 0, 1])


def test_nf4_table_and_roundtrip():
    code = O.nf4_code()
    assert code.shape == (16,) and code[0] == -1.0 and code[7] == 0.0 and code[15] == 1.0
    assert np.all(np.diff(code) > 0)
    # all 16 levels of the NF4 data type as published with it (QLoRA, appendix E), to 1e-6; the
    # device-side table of the package is built from the same construction
    published = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
                 -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
                 0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0]
    np.testing.assert_allclose(code, published, atol=1e-6)
    from qwen3_moe_fused.quantize.nf4 import nf4_code as package_code

    np.testing.assert_allclose(package_code().numpy(), published, atol=1e-6)
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((4, 8, 64)) * 0.02).astype(np.float32)
    packed, absmax = O.nf4_quantize(w, 64)
    assert packed.size == w.size // 2 and absmax.size == w.size // 64
    deq = O.nf4_dequantize(packed, absmax, code, 64, w.shape)
    # every decoded value is a table level times its block's absmax and is the nearest one
    assert np.abs(deq - w).max() <= 0.16 * np.abs(w).max()
    packed2, absmax2 = O.nf4_quantize(deq, 64)
    np.testing.assert_array_equal(packed2, packed)
    # high nibble holds the even element
    first = packed[0]
    lv = code[[first >> 4, first & 15]] * absmax[0]
    np.testing.assert_allclose(deq.reshape(-1)[:2], lv, rtol=1e-6)
