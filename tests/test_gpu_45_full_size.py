"""The benchmark's own workloads at full size, through the C ABI, against the numpy oracle.

gate_up: 8192 tokens x top-8 (softmax of N(0,1) logits) = 65536 rows, 2048 -> 1536, 128
experts, built exactly as bench.py builds it (same routing function, same seed).
down: 65536 rows of SiLU(gate) * up, 768 -> 2048, expert ids Zipf(1.2) with three experts
emptied and the ids permuted.  Forward, dX and dW are compared on EVERY row and EVERY
expert (one float32 numpy GEMM per expert on the CPU).
NF4 + LoRA rank 16 at 512 / 4096 / 32768 tokens x top-8: sampled experts (the CPU decode
of all 128 experts would take minutes), every row of those experts.

Tolerance: max |got - ref| / max |ref| <= 1e-2, over the whole tensor and also inside every
expert's block on its own (so that one expert's error cannot hide behind another's scale).
Routing indices and permutations are compared bit for bit.
"""
import numpy as np
import pytest
import torch

import bench
from oracle import moe_oracle as O
from tests.helpers import to_np

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _blocks_err(got: torch.Tensor, ref: np.ndarray, bounds):
    """(global, worst per-block) max|got-ref| / max|ref| with blocks [a, b) along axis 0.
    `got` stays on the device until its block is compared, which bounds host memory."""
    worst_abs, ref_max, worst_rel, worst_block = 0.0, 0.0, 0.0, -1
    for i, (a, b) in enumerate(bounds):
        if b <= a:
            continue
        g = got[a:b].float().cpu().numpy()
        r = ref[a:b]
        d = float(np.abs(g - r).max())
        m = float(np.abs(r).max())
        worst_abs = max(worst_abs, d)
        ref_max = max(ref_max, m)
        if m > 0 and d / m > worst_rel:
            worst_rel, worst_block = d / m, i
    return worst_abs / max(ref_max, 1e-30), worst_rel, worst_block


def _group_bounds(m_sizes):
    ends = np.cumsum(np.asarray(m_sizes, np.int64))
    return list(zip((ends - m_sizes).tolist(), ends.tolist()))


def _check_three_gemms(cuda, x_d, w_d, dy_d, m_sizes_d, what):
    """fwd, dX, dW of one workload vs the oracle; returns the error table for the assert message."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed

    m_sizes = m_sizes_d.cpu().numpy()
    E = len(m_sizes)
    x, w, dy = to_np(x_d), to_np(w_d), to_np(dy_d)
    rows = _group_bounds(m_sizes)
    experts = [(e, e + 1) for e in range(E)]
    errs = {}

    y = grouped_gemm_forward(x_d, w_d, m_sizes_d)
    errs["fwd"] = _blocks_err(y, O.grouped_gemm_fwd(x, w, m_sizes, "bf16"), rows)
    del y
    dx = grouped_gemm_forward_transposed(dy_d, w_d, m_sizes_d)
    errs["dx"] = _blocks_err(dx, O.grouped_gemm_dx(dy, w, m_sizes, "bf16"), rows)
    del dx
    dw = grouped_gemm_backward_dw(x_d, dy_d, m_sizes_d, torch.bfloat16)
    errs["dw"] = _blocks_err(dw, O.grouped_gemm_dw(x, dy, m_sizes, "bf16"), experts)
    empty = np.flatnonzero(m_sizes == 0)
    if len(empty):
        assert float(dw[torch.from_numpy(empty).to(cuda)].abs().max()) == 0.0, f"{what}: empty experts must get zero dW"
    del dw
    torch.cuda.synchronize()
    assert _lib.read_error_flag() == 0, "a bounded wait inside a kernel gave up"
    for name, (glob, per_block, block) in errs.items():
        assert glob <= TOL and per_block <= TOL, (
            f"{what} {name}: global {glob:.3e}, worst expert {block} ({int(m_sizes[block])} rows) {per_block:.3e}; all: {errs}")
    return errs


def test_gate_up_workload_all_rows(cuda):
    """BASELINE config 2 as bench.py builds it: routing, permutation and gather bit-exact, then
    forward / dX / dW on all 65536 rows and all 128 experts."""
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import _gather_rows, softmax_topk

    cfg = bench.WORKLOADS["gate_up"]
    T, K, N, E, k = cfg["tokens"], cfg["K"], cfg["N"], cfg["E"], cfg["k"]
    logits, _ = bench.make_routing(cfg, seed=0)
    gen = torch.Generator().manual_seed(1234)
    bf = torch.bfloat16
    hidden = torch.randn(T, K, generator=gen).to(bf)
    dy = torch.randn(T * k, N, generator=gen).to(bf)
    w = (torch.randn(E, N, K, generator=torch.Generator().manual_seed(99)) * 0.02).to(bf)

    _, sel = softmax_topk(logits.to(cuda), k, True, bf)
    m_sizes, sort_idx, inv_sort_idx = get_expert_counts_and_idx(sel.view(-1), E)
    _, ref_sel = O.router_softmax_topk(logits.numpy(), k, True, "bf16")
    assert np.array_equal(sel.cpu().numpy(), ref_sel), "router indices differ from the oracle"
    rc, rsort, rinv = O.get_expert_counts_and_idx_fast(ref_sel.reshape(-1), E)
    assert np.array_equal(m_sizes.cpu().numpy(), rc)
    assert np.array_equal(sort_idx.cpu().numpy(), rsort) and np.array_equal(inv_sort_idx.cpu().numpy(), rinv)
    # the case the tile schedule has to get right: experts just above two full 256-token tiles
    assert ((rc > 512) & (rc <= 576)).sum() >= 4

    x_d = _gather_rows(hidden.to(cuda), sort_idx, k)
    assert torch.equal(x_d.cpu(), hidden[torch.from_numpy(rsort.astype(np.int64)) // k]), "gather differs from the oracle"
    _check_three_gemms(cuda, x_d, w.to(cuda), dy.to(cuda), m_sizes, "gate_up")


def test_down_workload_all_rows(cuda):
    """BASELINE config 3: SiLU(gate) * up rows, 768 -> 2048, Zipf(1.2) ids, experts 5 / 64 / 127
    of the unpermuted ids emptied; the largest expert holds more than a quarter of the rows."""
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.silu_mul import silu_mul_forward

    cfg = bench.WORKLOADS["down"]
    T, K, N, E, k = cfg["tokens"], cfg["K"], cfg["N"], cfg["E"], cfg["k"]
    M = T * k
    _, ids = bench.make_routing(cfg, seed=0)
    gen = torch.Generator().manual_seed(4321)
    bf = torch.bfloat16
    gate = torch.randn(M, K, generator=gen).to(bf)
    up = torch.randn(M, K, generator=gen).to(bf)
    dy = torch.randn(M, N, generator=gen).to(bf)
    w = (torch.randn(E, N, K, generator=gen) * 0.02).to(bf)

    m_sizes, sort_idx, inv_sort_idx = get_expert_counts_and_idx(ids.to(cuda), E)
    rc, rsort, rinv = O.get_expert_counts_and_idx_fast(ids.numpy(), E)
    assert np.array_equal(m_sizes.cpu().numpy(), rc)
    assert np.array_equal(sort_idx.cpu().numpy(), rsort) and np.array_equal(inv_sort_idx.cpu().numpy(), rinv)
    assert (rc == 0).sum() >= 3 and rc.max() > M // 4

    h_d = silu_mul_forward(gate.to(cuda), up.to(cuda))
    ref_h = O.silu_mul_fwd(gate.float().numpy(), up.float().numpy(), "bf16")
    ulp = np.abs(to_np(h_d) - ref_h) <= np.abs(ref_h) * 2.0 ** -7  # one bf16 step
    assert ulp.all(), "SiLU-mul differs from the oracle by more than one storage step"
    # rows in expert order (the activation is per row, so sorting before or after it is the same)
    x_d = h_d[sort_idx.long()].contiguous()
    dy_d = dy.to(cuda)[sort_idx.long()].contiguous()
    _check_three_gemms(cuda, x_d, w.to(cuda), dy_d, m_sizes, "down")


@pytest.mark.parametrize("tokens", [512, 4096, 32768])
def test_nf4_lora_workload_sampled_experts(cuda, tokens):
    """BASELINE config 4: NF4 base (blocksize 64, fp32 absmax) of shape (128, 1536, 2048) plus LoRA
    rank 16, uniform routing, forward and the LoRA gradients (and dX).  The 128 experts hold four
    distinct weight slices (expert e has slice e % 4), so that the oracle quantises and decodes four
    slices; every row of experts 0, 17, 63 and 127 is compared."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.functional import moe_fused_linear
    from qwen3_moe_fused.quantize.linear4bit import moe_fused_linear_4bit
    from qwen3_moe_fused.quantize.nf4 import Nf4State

    E, N, K, R, bs, distinct = 128, 1536, 2048, 16, 64, 4
    M = tokens * 8
    per = M // E
    scaling = 2.0
    rng = np.random.default_rng(tokens)
    code = O.nf4_code()
    w4 = (rng.standard_normal((distinct, N, K)) * 0.02).astype(np.float32)
    packed4, absmax4 = O.nf4_quantize(w4, bs, code)
    wdeq4 = O.nf4_dequantize(packed4, absmax4, code, bs, w4.shape, "bf16")
    packed = torch.from_numpy(np.tile(packed4.reshape(distinct, -1), (E // distinct, 1)).reshape(-1, 1)).to(cuda)
    absmax = torch.from_numpy(np.tile(absmax4.reshape(distinct, -1), (E // distinct, 1)).reshape(-1)).to(cuda)
    state = Nf4State(absmax=absmax, code=torch.from_numpy(code).to(cuda), blocksize=bs, shape=torch.Size((E, N, K)),
                     dtype=torch.bfloat16)
    bf = torch.bfloat16
    gen = torch.Generator().manual_seed(tokens)
    x = torch.randn(M, K, generator=gen).to(bf)
    dy = torch.randn(M, N, generator=gen).to(bf)
    A = (torch.randn(E, R, K, generator=gen) / K ** 0.5).to(bf)
    B = (torch.randn(E, N, R, generator=gen) * 0.01).to(bf)
    m_sizes = torch.full((E,), per, dtype=torch.int32, device=cuda)

    x_d = x.to(cuda).requires_grad_()
    A_d, B_d = A.to(cuda).requires_grad_(), B.to(cuda).requires_grad_()
    # lora.py:134 of the reference: result + lora_B(lora_A(x)) * scaling
    y = moe_fused_linear_4bit(x_d, packed, state, m_sizes) + moe_fused_linear(moe_fused_linear(x_d, A_d, m_sizes), B_d, m_sizes) * scaling
    y.backward(dy.to(cuda))
    torch.cuda.synchronize()
    assert _lib.read_error_flag() == 0

    f32 = lambda t: t.float().numpy()
    for e in (0, 17, 63, 127):
        a, b = e * per, (e + 1) * per
        xe, dye, Ae, Be, We = f32(x[a:b]), f32(dy[a:b]), f32(A[e]), f32(B[e]), wdeq4[e % distinct]
        u = O.round_bf16(xe @ Ae.T)
        v = O.round_bf16(u @ Be.T)
        ref_y = O.round_bf16(O.round_bf16(xe @ We.T) + O.round_bf16(v * scaling))
        dv = O.round_bf16(dye * scaling)
        du = O.round_bf16(dv @ Be)
        refs = {
            "y": (y[a:b], ref_y),
            "dB": (B_d.grad[e], dv.T @ u),
            "dA": (A_d.grad[e], du.T @ xe),
            "dx": (x_d.grad[a:b], dye @ We + du @ Ae),
        }
        for name, (got, ref) in refs.items():
            err = O.rel_err(to_np(got), ref)
            assert err <= TOL, f"tokens={tokens} expert {e} {name}: rel err {err:.3e}"


def test_gate_up_silu_block_shape(cuda):
    """The fused gate + up + SiLU-mul kernel at the block's shape (131072 rows of 16384 tokens x
    top-8, 2048 -> 768, 128 experts, softmax routing): bit-identical to the three separate kernels,
    and four experts (largest, smallest, two just above 1024 rows) against the oracle."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.kernels.fused_mlp import gate_up_silu_forward
    from qwen3_moe_fused.kernels.indexing import get_expert_counts_and_idx
    from qwen3_moe_fused.kernels.routing import softmax_topk
    from qwen3_moe_fused.kernels.silu_mul import silu_mul_forward

    T, K, I, E, k = 16384, 2048, 768, 128, 8
    gen = torch.Generator().manual_seed(7)
    bf = torch.bfloat16
    logits = torch.randn(T, E, generator=gen)
    _, sel = softmax_topk(logits.to(cuda), k, True, bf)
    m_sizes, _, _ = get_expert_counts_and_idx(sel.view(-1), E)
    x = torch.randn(T * k, K, generator=gen).to(bf)
    wg = (torch.randn(E, I, K, generator=gen) * 0.02).to(bf)
    wu = (torch.randn(E, I, K, generator=gen) * 0.02).to(bf)
    x_d, wg_d, wu_d = x.to(cuda), wg.to(cuda), wu.to(cuda)
    h = gate_up_silu_forward(x_d, wg_d, wu_d, m_sizes)
    three = silu_mul_forward(grouped_gemm_forward(x_d, wg_d, m_sizes), grouped_gemm_forward(x_d, wu_d, m_sizes))
    torch.cuda.synchronize()
    assert _lib.read_error_flag() == 0
    assert torch.equal(h, three)

    ms = m_sizes.cpu().numpy()
    bounds = _group_bounds(ms)
    above = [e for e in np.argsort(ms) if ms[e] > 1024][:2]
    for e in {int(np.argmax(ms)), int(np.argmin(ms)), *map(int, above)}:
        a, b = bounds[e]
        xe = x[a:b].float().numpy()
        ref = O.silu_mul_fwd(O.round_bf16(xe @ wg[e].float().numpy().T), O.round_bf16(xe @ wu[e].float().numpy().T), "bf16")
        err = O.rel_err(to_np(h[a:b]), ref)
        assert err <= TOL, f"expert {e} ({ms[e]} rows): rel err {err:.3e}"


def test_moe_fused_linear_module(cuda):
    """`MoeFusedLinear` (modular_qwen3_moe_fused.py:29-59 of the reference): parameter shape,
    initialisation bound, forward and the gradients of both its input and its weight."""
    from qwen3_moe_fused.moe_block import MoeFusedLinear

    torch.manual_seed(3)
    E, K, N, M = 16, 256, 384, 2000
    layer = MoeFusedLinear(K, N, E, device=cuda, dtype=torch.bfloat16)
    assert layer.weight.shape == (E, N, K)
    assert float(layer.weight.detach().float().abs().max()) <= (15 / K) ** 0.5 * (1 + 2.0 ** -8)
    assert "num_experts=16" in repr(layer)
    ms = np.random.default_rng(3).multinomial(M, np.ones(E) / E).astype(np.int32)
    ms[3] += ms[4]; ms[4] = 0
    m_sizes = torch.from_numpy(ms).to(cuda)
    x = torch.randn(M, K, device=cuda).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(M, N, device=cuda).to(torch.bfloat16)
    y = layer(x, m_sizes)
    y.backward(dy)
    xn, wn, dyn = to_np(x), to_np(layer.weight), to_np(dy)
    assert O.rel_err(to_np(y), O.grouped_gemm_fwd(xn, wn, ms, "bf16")) <= TOL
    assert O.rel_err(to_np(x.grad), O.grouped_gemm_dx(dyn, wn, ms, "bf16")) <= TOL
    assert O.rel_err(to_np(layer.weight.grad), O.grouped_gemm_dw(xn, dyn, ms, "bf16")) <= TOL
    assert float(layer.weight.grad[4].abs().max()) == 0.0
