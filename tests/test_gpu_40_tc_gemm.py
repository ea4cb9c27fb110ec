"""tcgen05 grouped GEMMs (forward, dX, dW) through the C ABI vs the oracle.
Tolerance: max |got - ref| / max |ref| <= 1e-2 for bf16/fp16 inputs with fp32 accumulation
(the oracle accumulates the same rounded inputs in fp32 and rounds once)."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import DT, assert_close, random_m_sizes, rounded, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=["pair", "single"])
def tc_path(request):
    """Every test runs twice: CTA-pair kernels (where the shape qualifies) and single-CTA kernels."""
    from qwen3_moe_fused import _lib

    prev = _lib.set_gemm_path(_lib.PATH_TC if request.param == "pair" else _lib.PATH_TC_SINGLE)
    yield request.param
    torch.cuda.synchronize()
    _lib.set_gemm_path(prev)
    assert _lib.read_error_flag() == 0, "a bounded wait inside a tensor-core kernel gave up"


def tensors(cuda, rng, M, K, N, E, dtype, empty=0.0, m_sizes=None):
    x = rounded(rng.standard_normal((M, K)), dtype)
    w = rounded(rng.standard_normal((E, N, K)) / np.sqrt(K), dtype)
    dy = rounded(rng.standard_normal((M, N)), dtype)
    if m_sizes is None:
        m_sizes = random_m_sizes(rng, M, E, empty)
    return x, w, dy, np.asarray(m_sizes)


SHAPES = [
    # M, K(in), N(out), E, empty fraction
    (256, 64, 128, 8, 0.0),        # shape of the small fp32 case (here in bf16)
    (1024, 2048, 768, 128, 0.0),   # the reference's kernel test shape
    (1000, 192, 320, 7, 0.3),      # ragged, K and N not multiples of the tile
    (4096, 768, 2048, 16, 0.0),    # down_proj shape, few experts
    (129, 72, 200, 3, 0.0),        # K % 64 != 0, N % 64 != 0
    (5000, 256, 256, 128, 0.5),    # many empty experts
]


@pytest.mark.parametrize("M,K,N,E,empty", SHAPES)
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_forward(cuda, M, K, N, E, empty, dtype):
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward

    rng = np.random.default_rng(M + K + N + E)
    x, w, dy, m_sizes = tensors(cuda, rng, M, K, N, E, dtype, empty)
    y = grouped_gemm_forward(to_dev(x, dtype, cuda), to_dev(w, dtype, cuda), torch.from_numpy(m_sizes).to(cuda))
    assert_close(to_np(y), O.grouped_gemm_fwd(x, w, m_sizes, dtype), dtype, "fwd")


@pytest.mark.parametrize("M,K,N,E,empty", SHAPES)
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_dx(cuda, M, K, N, E, empty, dtype):
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed

    rng = np.random.default_rng(M + K + N + E + 1)
    x, w, dy, m_sizes = tensors(cuda, rng, M, K, N, E, dtype, empty)
    dx = grouped_gemm_forward_transposed(to_dev(dy, dtype, cuda), to_dev(w, dtype, cuda), torch.from_numpy(m_sizes).to(cuda))
    assert_close(to_np(dx), O.grouped_gemm_dx(dy, w, m_sizes, dtype), dtype, "dx")


@pytest.mark.parametrize("M,K,N,E,empty", SHAPES)
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_dw(cuda, M, K, N, E, empty, dtype):
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw

    rng = np.random.default_rng(M + K + N + E + 2)
    x, w, dy, m_sizes = tensors(cuda, rng, M, K, N, E, dtype, empty)
    dw = grouped_gemm_backward_dw(to_dev(x, dtype, cuda), to_dev(dy, dtype, cuda), torch.from_numpy(m_sizes).to(cuda), DT[dtype])
    ref = O.grouped_gemm_dw(x, dy, m_sizes, dtype)
    assert_close(to_np(dw), ref, dtype, "dw")
    assert np.all(to_np(dw)[m_sizes == 0] == 0)


THIN = [
    # LoRA-thin shapes (rank 8..64 as output width or as contraction length): M, K, N, E, empty
    (1000, 2048, 16, 8, 0.2),    # x @ A^T, rank 16
    (1000, 16, 1536, 8, 0.2),    # (x A^T) @ B^T, rank 16
    (777, 64, 24, 5, 0.0),       # rank 24 -> 32-column accumulator
    (513, 8, 128, 3, 0.0),       # rank 8
    (2048, 768, 64, 16, 0.3),    # rank 64
]


@pytest.mark.parametrize("M,K,N,E,empty", THIN)
def test_lora_thin_shapes(cuda, M, K, N, E, empty):
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed

    rng = np.random.default_rng(M + K + N)
    x, w, dy, m_sizes = tensors(cuda, rng, M, K, N, E, "bf16", empty)
    tm = torch.from_numpy(m_sizes).to(cuda)
    tx, tw, tdy = to_dev(x, "bf16", cuda), to_dev(w, "bf16", cuda), to_dev(dy, "bf16", cuda)
    assert_close(to_np(grouped_gemm_forward(tx, tw, tm)), O.grouped_gemm_fwd(x, w, m_sizes, "bf16"), "bf16", "thin fwd")
    assert_close(to_np(grouped_gemm_forward_transposed(tdy, tw, tm)), O.grouped_gemm_dx(dy, w, m_sizes, "bf16"), "bf16", "thin dx")
    dw = to_np(grouped_gemm_backward_dw(tx, tdy, tm, torch.bfloat16))
    assert_close(dw, O.grouped_gemm_dw(x, dy, m_sizes, "bf16"), "bf16", "thin dw")
    assert np.all(dw[m_sizes == 0] == 0)


def test_group_boundaries_every_residue(cuda):
    # group sizes sweep every residue mod 128 and mod 64 so that every tail length of an M
    # tile (forward/dX) and of a reduction block (dW) is exercised
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward

    rng = np.random.default_rng(11)
    sizes = np.array([0, 1, 127, 128, 129, 63, 64, 65, 255, 2, 191, 0, 300, 17], dtype=np.int32)
    M, K, N, E = int(sizes.sum()), 128, 128, len(sizes)
    x, w, dy, _ = tensors(cuda, rng, M, K, N, E, "bf16", m_sizes=sizes)
    tm = torch.from_numpy(sizes).to(cuda)
    y = grouped_gemm_forward(to_dev(x, "bf16", cuda), to_dev(w, "bf16", cuda), tm)
    assert_close(to_np(y), O.grouped_gemm_fwd(x, w, sizes, "bf16"), "bf16", "fwd")
    dw = grouped_gemm_backward_dw(to_dev(x, "bf16", cuda), to_dev(dy, "bf16", cuda), tm, torch.bfloat16)
    assert_close(to_np(dw), O.grouped_gemm_dw(x, dy, sizes, "bf16"), "bf16", "dw")


def test_fp32_output_and_int64_sizes(cuda):
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward

    rng = np.random.default_rng(12)
    x, w, dy, m_sizes = tensors(cuda, rng, 700, 128, 192, 9, "bf16")
    y = grouped_gemm_forward(to_dev(x, "bf16", cuda), to_dev(w, "bf16", cuda),
                             torch.from_numpy(m_sizes.astype(np.int64)).to(cuda), torch.float32)
    assert y.dtype == torch.float32
    assert_close(to_np(y), O.grouped_gemm_fwd(x, w, m_sizes), "f32", "fwd fp32 out", scale=20)


def test_tc_agrees_with_simt_at_scale(cuda, tc_path):
    # 65536 rows (the gate_up workload's row count) at a reduced width: the CUDA-core kernel
    # is the on-device anchor where the CPU oracle would take too long
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed

    torch.manual_seed(0)
    M, K, N, E = 65536, 256, 384, 128
    p = (torch.arange(E, dtype=torch.float64) + 1) ** -1.2
    ids = torch.multinomial(p / p.sum(), M, replacement=True)
    m_sizes = torch.bincount(ids, minlength=E).to(torch.int32).to(cuda)
    x = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    w = (torch.randn(E, N, K, device=cuda) * 0.05).to(torch.bfloat16)
    dy = torch.randn(M, N, device=cuda, dtype=torch.bfloat16)
    outs = {}
    tc = _lib.PATH_TC if tc_path == "pair" else _lib.PATH_TC_SINGLE
    for path in (tc, _lib.PATH_SIMT):
        _lib.set_gemm_path(path)
        outs[path] = (grouped_gemm_forward(x, w, m_sizes), grouped_gemm_forward_transposed(dy, w, m_sizes),
                      grouped_gemm_backward_dw(x, dy, m_sizes, torch.bfloat16))
    _lib.set_gemm_path(tc)
    for a, b, what in zip(outs[tc], outs[_lib.PATH_SIMT], ("fwd", "dx", "dw")):
        assert_close(to_np(a), to_np(b), "bf16", what)


def test_linearity_at_full_gate_up_shape(cuda):
    # full-size forward (65536 x 2048 -> 1536, 128 experts): f(x1 + x2) = f(x1) + f(x2) up to
    # rounding, and one randomly chosen row per expert against a direct product
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward

    torch.manual_seed(1)
    M, K, N, E = 65536, 2048, 1536, 128
    m_sizes = torch.full((E,), M // E, dtype=torch.int32, device=cuda)
    w = (torch.randn(E, N, K, device=cuda) * 0.02).to(torch.bfloat16)
    x1 = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    x2 = torch.randn(M, K, device=cuda, dtype=torch.bfloat16)
    y1 = grouped_gemm_forward(x1, w, m_sizes, torch.float32)
    y2 = grouped_gemm_forward(x2, w, m_sizes, torch.float32)
    y12 = grouped_gemm_forward((x1.float() + x2.float()).to(torch.bfloat16), w, m_sizes, torch.float32)
    err = (y12 - (y1 + y2)).abs().max() / y12.abs().max()
    assert float(err) < 2e-2
    rows = torch.arange(E, device=cuda) * (M // E) + torch.randint(0, M // E, (E,), device=cuda)
    ref = torch.einsum("enk,ek->en", w.float(), x1[rows].float())
    assert float((y1[rows] - ref).abs().max() / ref.abs().max()) < 1e-2


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,K,I,E,empty", [
    (3000, 256, 384, 8, 0.2),
    (8192, 2048, 768, 16, 0.0),     # the model's gate / up shape
    (700, 72, 192, 3, 0.0),         # features not a multiple of 128: the last pair tile is half empty
    (50, 64, 64, 4, 0.5),
])
def test_gate_up_silu_fused_equals_three_kernels(cuda, dtype, M, K, I, E, empty):
    """gate GEMM + up GEMM + SiLU-mul in one kernel: bit-identical to the separate kernels."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.kernels.fused_mlp import gate_up_silu_forward
    from qwen3_moe_fused.kernels.silu_mul import silu_mul_forward

    rng = np.random.default_rng(M + K + I)
    x = to_dev(rounded(rng.standard_normal((M, K)), dtype), dtype, cuda)
    wg = to_dev(rounded(rng.standard_normal((E, I, K)) / np.sqrt(K) * 2, dtype), dtype, cuda)
    wu = to_dev(rounded(rng.standard_normal((E, I, K)) / np.sqrt(K), dtype), dtype, cuda)
    m = torch.from_numpy(random_m_sizes(rng, M, E, empty)).to(cuda)
    prev = _lib.set_gemm_path(_lib.PATH_AUTO)
    try:
        h = gate_up_silu_forward(x, wg, wu, m)
        ref = silu_mul_forward(grouped_gemm_forward(x, wg, m), grouped_gemm_forward(x, wu, m))
        torch.cuda.synchronize()
    finally:
        _lib.set_gemm_path(prev)
    assert _lib.read_error_flag() == 0
    assert torch.equal(h, ref)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("T,k,K,I,E,empty", [
    (1000, 4, 256, 384, 8, 0.2),
    (4096, 8, 2048, 768, 64, 0.0),   # about 512 rows per expert: tiles with tails
    (300, 2, 72, 192, 5, 0.0),       # K % 64 != 0
    (64, 8, 128, 256, 16, 0.5),      # groups of a few rows
])
def test_token_rows_gathered_inside_the_kernel(cuda, dtype, T, k, K, I, E, empty):
    """Forward and fused gate/up forward fed from the (T, K) token tensor through the sort's gather index
    (TMA gather4 in the token load): bit-identical to gathering the rows first."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward, grouped_gemm_forward_gather
    from qwen3_moe_fused.kernels.fused_mlp import gate_up_silu_forward
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import _gather_rows

    rng = np.random.default_rng(T + K + I)
    p = rng.random(E) + 0.05
    p[rng.random(E) < empty] = 0.0
    p[0] += 0.01
    sel = torch.from_numpy(rng.choice(E, size=T * k, p=p / p.sum())).to(cuda)
    m_sizes, sort_idx, _ = get_expert_counts_and_idx(sel, E)
    tokens = to_dev(rounded(rng.standard_normal((T, K)), dtype), dtype, cuda)
    wg = to_dev(rounded(rng.standard_normal((E, I, K)) / np.sqrt(K) * 2, dtype), dtype, cuda)
    wu = to_dev(rounded(rng.standard_normal((E, I, K)) / np.sqrt(K), dtype), dtype, cuda)
    xs = _gather_rows(tokens, sort_idx, k)
    prev = _lib.set_gemm_path(_lib.PATH_AUTO)
    try:
        h_ref = gate_up_silu_forward(xs, wg, wu, m_sizes)
        h = gate_up_silu_forward(tokens, wg, wu, m_sizes, row_index=sort_idx, index_div=k)
        y_ref = grouped_gemm_forward(xs, wg, m_sizes)
        y = grouped_gemm_forward_gather(tokens, sort_idx, k, wg, m_sizes)
        # index_div = 1: an index of rows rather than of (token, slot) pairs
        y1 = grouped_gemm_forward_gather(tokens, (sort_idx // k).to(torch.int32).contiguous(), 1, wg, m_sizes)
        torch.cuda.synchronize()
    finally:
        _lib.set_gemm_path(prev)
    assert _lib.read_error_flag() == 0
    assert torch.equal(h, h_ref)
    assert torch.equal(y, y_ref) and torch.equal(y1, y_ref)
