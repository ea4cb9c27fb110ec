"""CUDA-core grouped GEMMs (forward, dX, dW) through the C ABI vs the oracle, including the
reference's golden vectors and its odd tiny-model shapes."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import DT, assert_close, random_m_sizes, rounded, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def simt_path():
    from qwen3_moe_fused import _lib

    prev = _lib.set_gemm_path(_lib.PATH_SIMT)
    yield
    _lib.set_gemm_path(prev)


def run_all(cuda, x, w, dy, m_sizes, dtype, out_dtype=None):
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed

    od = DT[out_dtype or dtype]
    tx, tw, tdy = to_dev(x, dtype, cuda), to_dev(w, dtype, cuda), to_dev(dy, dtype, cuda)
    tm = torch.from_numpy(np.asarray(m_sizes)).to(cuda)
    y = grouped_gemm_forward(tx, tw, tm, od)
    dx = grouped_gemm_forward_transposed(tdy, tw, tm, od)
    dw = grouped_gemm_backward_dw(tx, tdy, tm, od)
    return to_np(y), to_np(dx), to_np(dw)


@pytest.mark.parametrize("name", ["c1", "odd", "empty"])
def test_golden_vectors_fp32(golden, cuda, name):
    g = golden(f"linear_{name}")
    x, w, s, dy = g["x"], g["w"], g["s"], g["dy"]
    E = w.shape[0]
    m_sizes, inv_idx, idx = O.get_expert_counts_and_idx_fast(s, E)
    y, dx, dw = run_all(cuda, x[inv_idx], w, dy[inv_idx], m_sizes, "f32")
    np.testing.assert_allclose(y[idx], g["y"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dx[idx], g["dx"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dw, g["dw"], rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("M,K,N,E,empty", [(1024, 2048, 768, 128, 0.0), (300, 3, 4, 11, 0.2), (65, 64, 128, 8, 0.0),
                                           (513, 100, 70, 5, 0.4), (1, 16, 16, 4, 0.0)])
def test_random_vs_oracle(cuda, dtype, M, K, N, E, empty):
    rng = np.random.default_rng(M + K + N + E)
    x = rounded(rng.standard_normal((M, K)), dtype)
    w = rounded(rng.standard_normal((E, N, K)) / np.sqrt(K), dtype)
    dy = rounded(rng.standard_normal((M, N)), dtype)
    m_sizes = random_m_sizes(rng, M, E, empty)
    y, dx, dw = run_all(cuda, x, w, dy, m_sizes, dtype)
    assert_close(y, O.grouped_gemm_fwd(x, w, m_sizes, dtype), dtype, "fwd")
    assert_close(dx, O.grouped_gemm_dx(dy, w, m_sizes, dtype), dtype, "dx")
    assert_close(dw, O.grouped_gemm_dw(x, dy, m_sizes, dtype), dtype, "dw")
    assert np.all(dw[np.asarray(m_sizes) == 0] == 0)


def test_int64_m_sizes_and_fp32_output(cuda):
    rng = np.random.default_rng(9)
    M, K, N, E = 200, 32, 48, 6
    x = rounded(rng.standard_normal((M, K)), "bf16")
    w = rounded(rng.standard_normal((E, N, K)), "bf16")
    dy = rounded(rng.standard_normal((M, N)), "bf16")
    m_sizes = random_m_sizes(rng, M, E).astype(np.int64)
    y, dx, dw = run_all(cuda, x, w, dy, m_sizes, "bf16", "f32")
    assert_close(y, O.grouped_gemm_fwd(x, w, m_sizes), "f32", "fwd", scale=5)
    assert_close(dw, O.grouped_gemm_dw(x, dy, m_sizes), "f32", "dw", scale=5)


def test_autograd_matches_reference_semantics(cuda):
    from qwen3_moe_fused.functional import moe_fused_linear

    rng = np.random.default_rng(10)
    M, K, N, E = 256, 64, 128, 8
    x = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(cuda)
    w = torch.from_numpy((rng.standard_normal((E, N, K)) / 8).astype(np.float32)).to(cuda)
    m_sizes = torch.from_numpy(random_m_sizes(rng, M, E)).to(cuda)
    dy = torch.randn(M, N, device=cuda)
    for req_x, req_w in ((True, True), (True, False), (False, True)):
        xx = x.clone().requires_grad_(req_x)
        ww = w.clone().requires_grad_(req_w)
        y = moe_fused_linear(xx, ww, m_sizes)
        y.backward(dy)
        assert (xx.grad is not None) == req_x and (ww.grad is not None) == req_w
        if req_x:
            assert_close(to_np(xx.grad), O.grouped_gemm_dx(to_np(dy), to_np(w), m_sizes.cpu().numpy()), "f32", "dx")
        if req_w:
            assert_close(to_np(ww.grad), O.grouped_gemm_dw(to_np(x), to_np(dy), m_sizes.cpu().numpy()), "f32", "dw")
