"""SiLU-mul, router, gather, combine and NF4 decode kernels vs the oracle."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import DT, TOL, assert_close, rounded, to_dev, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("n", [0, 1, 7, 8, 1000, 65536 * 3 + 5])
def test_silu_mul_forward_backward(cuda, dtype, n):
    from qwen3_moe_fused.kernels.silu_mul import silu_mul_backward, silu_mul_backward_inplace, silu_mul_forward

    rng = np.random.default_rng(n + 1)
    e = rounded(rng.standard_normal(n) * 3, dtype)
    g = rounded(rng.standard_normal(n), dtype)
    dh = rounded(rng.standard_normal(n), dtype)
    te, tg, tdh = (to_dev(a, dtype, cuda) for a in (e, g, dh))
    h = silu_mul_forward(te, tg)
    de, dg = silu_mul_backward(tdh, te, tg)
    rh, rde, rdg = O.silu_mul_bwd(dh, e, g, dtype)
    if n == 0:
        assert h.numel() == 0
        return
    # one storage-dtype ulp of slack: the device exp is not bit-identical to numpy's
    ulp = {"bf16": 2 ** -7, "f16": 2 ** -10, "f32": 1e-5}[dtype]
    for got, ref, what in ((h, O.silu_mul_fwd(e, g, dtype), "h"), (de, rde, "de"), (dg, rdg, "dg")):
        got = to_np(got)
        assert np.all(np.abs(got - ref) <= ulp * np.maximum(np.abs(ref), 1e-3) * 2 + 1e-30), what
        if dtype != "f32":  # 16-bit storage: the rounding hides the last-ulp difference of exp almost always
            assert (got != ref).mean() < 0.02, f"{what}: too many elements differ from the oracle's rounding"
    # in-place form writes (h, de, dg) over (dh, e, g)
    e2, g2, dh2 = te.clone(), tg.clone(), tdh.clone()
    silu_mul_backward_inplace(dh2, e2, g2)
    assert torch.equal(dh2, h) and torch.equal(e2, de) and torch.equal(g2, dg)


def test_silu_mul_autograd_and_unaligned(cuda):
    from qwen3_moe_fused.kernels.silu_mul import silu_mul, silu_mul_forward

    base = torch.randn(4099, device=cuda, dtype=torch.bfloat16)
    e, g = base[1:4098].clone()[1:], base[2:4099].clone()[1:]  # storage offset -> not 16-byte aligned
    assert e.data_ptr() % 16 != 0
    ref = O.silu_mul_fwd(to_np(e), to_np(g), "bf16")
    got = to_np(silu_mul_forward(e, g))
    assert np.abs(got - ref).max() <= 2 ** -6 * np.abs(ref).max()
    e32 = torch.randn(1000, device=cuda, requires_grad=True)
    g32 = torch.randn(1000, device=cuda, requires_grad=True)
    silu_mul(e32, g32).sum().backward()
    ee = e32.detach().clone().requires_grad_()
    gg = g32.detach().clone().requires_grad_()
    (torch.nn.functional.silu(ee) * gg).sum().backward()
    assert torch.allclose(e32.grad, ee.grad, rtol=1e-4, atol=1e-5) and torch.allclose(g32.grad, gg.grad, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("T,E,k", [(8192, 128, 8), (1000, 11, 3), (77, 60, 4), (5, 1024, 32), (16, 8, 8),
                                   (140000, 128, 8),   # above the size where the eight-lanes-per-token form takes over
                                   (300, 256, 16), (64, 64, 8)])
@pytest.mark.parametrize("norm", [True, False])
def test_router_fp32_logits(cuda, T, E, k, norm):
    from qwen3_moe_fused.kernels.routing import softmax_topk

    rng = np.random.default_rng(T + E)
    logits = rng.standard_normal((T, E)).astype(np.float32)
    w, idx = softmax_topk(torch.from_numpy(logits).to(cuda), k, norm, torch.bfloat16)
    rw, ridx = O.router_softmax_topk(logits, k, norm, "bf16")
    # rows where two probabilities within the top k+1 are closer than fp32 rounding noise may
    # legitimately order differently between exp implementations; everything else is exact
    p = np.sort(np.exp(logits - logits.max(1, keepdims=True)) / np.exp(logits - logits.max(1, keepdims=True)).sum(1, keepdims=True), axis=1)[:, ::-1]
    gap = np.abs(np.diff(p[:, : min(k + 1, E)], axis=1)).min(axis=1) / p[:, 0]
    clear = gap > 1e-5
    assert clear.mean() > 0.98
    np.testing.assert_array_equal(idx.cpu().numpy()[clear], ridx[clear])
    assert np.abs(to_np(w)[clear] - rw[clear]).max() <= 2 ** -7 * rw.max()


def test_router_ties_pick_lowest_expert(cuda):
    from qwen3_moe_fused.kernels.routing import softmax_topk

    logits = torch.zeros((3, 128), device=cuda, dtype=torch.bfloat16)
    logits[0, [100, 7, 64]] = 2.0
    logits[1, :] = 1.0
    logits[2, [127, 126, 0]] = 3.0
    w, idx = softmax_topk(logits, 8, True, torch.bfloat16)
    rw, ridx = O.router_softmax_topk(to_np(logits), 8, True, "bf16")
    np.testing.assert_array_equal(idx.cpu().numpy(), ridx)
    assert idx[1].tolist() == list(range(8))
    assert np.abs(to_np(w) - rw).max() <= 2 ** -7


@pytest.mark.parametrize("T", [2000, 135000])  # one size for each form of the kernel
def test_router_many_ties(cuda, T):
    """Logits from a set of five values: every row has many exact ties, and distinct logits have
    clearly distinct probabilities, so the (value descending, expert ascending) rule is checked exactly."""
    from qwen3_moe_fused.kernels.routing import softmax_topk

    rng = np.random.default_rng(T)
    logits = (rng.integers(0, 5, (T, 128)) * 0.5).astype(np.float32)
    w, idx = softmax_topk(torch.from_numpy(logits).to(cuda).to(torch.bfloat16), 8, True, torch.bfloat16)
    rw, ridx = O.router_softmax_topk(logits, 8, True, "bf16")
    np.testing.assert_array_equal(idx.cpu().numpy(), ridx)
    assert np.abs(to_np(w) - rw).max() <= 2 ** -7


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("T,k,H", [(64, 8, 2048), (33, 3, 16), (5, 2, 7)])
def test_gather_and_combine(cuda, dtype, T, k, H):
    from qwen3_moe_fused.kernels.routing import _combine, _expand_rows, _gather_rows

    rng = np.random.default_rng(T * k + H)
    E = 9
    hidden = rounded(rng.standard_normal((T, H)), dtype)
    sel = rng.integers(0, E, T * k)
    _, sort_idx, inv_sort_idx = O.get_expert_counts_and_idx_fast(sel, E)
    weights = rounded(rng.random((T, k)), dtype)
    got = _gather_rows(to_dev(hidden, dtype, cuda), torch.from_numpy(sort_idx).to(cuda), k)
    np.testing.assert_array_equal(to_np(got), O.gather_rows(hidden, sort_idx, k))
    # the token-major form writes the same rows through the inverse index
    got2 = _expand_rows(to_dev(hidden, dtype, cuda), torch.from_numpy(inv_sort_idx).to(cuda), k)
    assert torch.equal(got2, got)
    y = rounded(rng.standard_normal((T * k, H)), dtype)
    out = _combine(to_dev(y, dtype, cuda), torch.from_numpy(inv_sort_idx).to(cuda), to_dev(weights, dtype, cuda))
    assert_close(to_np(out), O.combine(y, inv_sort_idx, weights, dtype), dtype, "combine")


def test_gather_combine_autograd(cuda):
    from qwen3_moe_fused.kernels.routing import combine, gather_rows

    T, k, H, E = 20, 3, 24, 5
    rng = np.random.default_rng(0)
    sel = rng.integers(0, E, T * k)
    _, sort_idx, inv_sort_idx = O.get_expert_counts_and_idx_fast(sel, E)
    si = torch.from_numpy(sort_idx).to(cuda)
    ii = torch.from_numpy(inv_sort_idx).to(cuda)
    hidden = torch.randn(T, H, device=cuda, requires_grad=True)
    w = torch.rand(T, k, device=cuda, requires_grad=True)
    out = combine(gather_rows(hidden, si, ii, k) * 2.0, si, ii, w)
    out.square().sum().backward()
    h2 = hidden.detach().clone().requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    exp = h2.unsqueeze(1).expand(T, k, H).reshape(T * k, H)[si.long()] * 2.0
    ref = torch.einsum("tkh,tk->th", exp[ii.long()].view(T, k, H), w2)
    ref.square().sum().backward()
    assert torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(hidden.grad, h2.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(w.grad, w2.grad, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape,bs", [((4, 24, 64), 64), ((3, 6, 32), 16), ((128, 96, 256), 256), ((2, 5, 6), 4)])
def test_nf4_dequant_bit_exact(cuda, dtype, shape, bs):
    from qwen3_moe_fused.quantize.nf4 import Nf4State, dequantize_4bit, nf4_code, quantize_nf4

    rng = np.random.default_rng(sum(shape))
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    code = O.nf4_code()
    np.testing.assert_allclose(nf4_code().numpy(), code, atol=1e-7)
    packed, absmax = O.nf4_quantize(w, bs, code)
    state = Nf4State(absmax=torch.from_numpy(absmax).to(cuda), code=torch.from_numpy(code).to(cuda), blocksize=bs,
                     shape=torch.Size(shape), dtype=DT[dtype])
    got = dequantize_4bit(torch.from_numpy(packed).to(cuda), state)
    ref = O.nf4_dequantize(packed, absmax, code, bs, shape, dtype)
    np.testing.assert_array_equal(to_np(got), ref)
    # device quantiser agrees with the oracle's
    p2, st2 = quantize_nf4(torch.from_numpy(w).to(cuda), bs)
    np.testing.assert_array_equal(p2.cpu().numpy().reshape(-1), packed)
    np.testing.assert_allclose(st2.absmax.cpu().numpy(), absmax, rtol=0, atol=0)
