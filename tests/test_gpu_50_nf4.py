"""NF4-fused forward (CUDA-core and tcgen05 forms) vs the oracle's decode + GEMM."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import DT, assert_close, random_m_sizes, rounded, to_dev, to_np

pytestmark = pytest.mark.gpu


def make(cuda, rng, M, K, N, E, bs, dtype, empty=0.0):
    from qwen3_moe_fused.quantize.nf4 import Nf4State

    code = O.nf4_code()
    w = (rng.standard_normal((E, N, K)) / np.sqrt(K)).astype(np.float32)
    packed, absmax = O.nf4_quantize(w, bs, code)
    w_deq = O.nf4_dequantize(packed, absmax, code, bs, w.shape, dtype)  # rounded to the activation dtype
    x = rounded(rng.standard_normal((M, K)), dtype)
    m_sizes = random_m_sizes(rng, M, E, empty)
    state = Nf4State(absmax=torch.from_numpy(absmax).to(cuda), code=torch.from_numpy(code).to(cuda), blocksize=bs,
                     shape=torch.Size(w.shape), dtype=DT[dtype])
    return x, torch.from_numpy(packed).to(cuda), state, m_sizes, O.grouped_gemm_fwd(x, w_deq, m_sizes, dtype)


@pytest.mark.parametrize("path", ["simt", "tc"])
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,K,N,E,bs,empty", [
    (1024, 2048, 768, 128, 256, 0.0),   # the reference's kernel test shape and block size
    (512, 256, 320, 8, 64, 0.2),
    (300, 128, 64, 5, 128, 0.0),
    (4096, 2048, 1536, 4, 64, 0.0),     # gate_up width, block size 64
])
def test_fused_forward(cuda, path, dtype, M, K, N, E, bs, empty):
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_4bit

    rng = np.random.default_rng(M + K + N + E + bs)
    x, packed, state, m_sizes, ref = make(cuda, rng, M, K, N, E, bs, dtype, empty)
    prev = _lib.set_gemm_path(_lib.PATH_SIMT if path == "simt" else _lib.PATH_TC)
    try:
        y = grouped_gemm_forward_4bit(to_dev(x, dtype, cuda), packed, state, torch.from_numpy(m_sizes).to(cuda), fused=True)
        torch.cuda.synchronize()
    finally:
        _lib.set_gemm_path(prev)
    assert _lib.read_error_flag() == 0
    assert_close(to_np(y), ref, dtype, f"nf4 fwd {path}")


def test_small_blocksize_and_odd_shapes_use_cuda_cores(cuda):
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_4bit

    rng = np.random.default_rng(3)
    x, packed, state, m_sizes, ref = make(cuda, rng, 77, 6, 10, 4, 4, "f32", 0.0)
    y = grouped_gemm_forward_4bit(to_dev(x, "f32", cuda), packed, state, torch.from_numpy(m_sizes).to(cuda))
    assert_close(to_np(y), ref, "f32", "nf4 fwd tiny", scale=5)


def test_fused_equals_decode_then_gemm(cuda):
    from qwen3_moe_fused.quantize.linear4bit import moe_fused_linear_4bit

    rng = np.random.default_rng(4)
    x, packed, state, m_sizes, ref = make(cuda, rng, 2048, 512, 512, 16, 64, "bf16", 0.1)
    tx = to_dev(x, "bf16", cuda)
    tm = torch.from_numpy(m_sizes).to(cuda)
    a = moe_fused_linear_4bit(tx, packed, state, tm, fused=True)
    b = moe_fused_linear_4bit(tx, packed, state, tm, fused=False)
    assert_close(to_np(a), to_np(b), "bf16", "fused vs unfused")
    assert_close(to_np(a), ref, "bf16", "fused vs oracle")


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("M,K,N,E,bs,empty", [
    (1024, 2048, 768, 16, 64, 0.0),     # gate-projection shape (E, out=768, in=2048)
    (512, 256, 320, 8, 64, 0.2),
    (4096, 2048, 1536, 4, 64, 0.0),
    (700, 512, 192, 3, 128, 0.0),       # block size 128: two 64-feature halves share an absmax
    (300, 128, 64, 5, 64, 0.0),         # input width below the pair kernel: decode + dX route
])
def test_fused_dx(cuda, dtype, M, K, N, E, bs, empty):
    """dX through the NF4 weight: the weight is the (E, out=N_w, in=K_w) tensor of `make`, dy has
    N_w columns and the result K_w columns."""
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_transposed_4bit

    rng = np.random.default_rng(M + K + N + E + bs + 1)
    from qwen3_moe_fused.quantize.nf4 import Nf4State

    code = O.nf4_code()
    w = (rng.standard_normal((E, N, K)) / np.sqrt(N)).astype(np.float32)
    packed, absmax = O.nf4_quantize(w, bs, code)
    w_deq = O.nf4_dequantize(packed, absmax, code, bs, w.shape, dtype)
    dy = rounded(rng.standard_normal((M, N)), dtype)
    m_sizes = random_m_sizes(rng, M, E, empty)
    state = Nf4State(absmax=torch.from_numpy(absmax).to(cuda), code=torch.from_numpy(code).to(cuda), blocksize=bs,
                     shape=torch.Size(w.shape), dtype=DT[dtype])
    ref = O.grouped_gemm_dx(dy, w_deq, m_sizes, dtype)
    dx = grouped_gemm_forward_transposed_4bit(to_dev(dy, dtype, cuda), torch.from_numpy(packed).to(cuda), state,
                                              torch.from_numpy(m_sizes).to(cuda))
    torch.cuda.synchronize()
    assert _lib.read_error_flag() == 0
    assert dx.shape == (M, K)
    assert_close(to_np(dx), ref, dtype, "nf4 dx")


def test_linear4bit_backward_is_fused_dx(cuda):
    from qwen3_moe_fused.quantize.linear4bit import moe_fused_linear_4bit

    rng = np.random.default_rng(5)
    x, packed, state, m_sizes, _ = make(cuda, rng, 1024, 512, 512, 8, 64, "bf16", 0.1)
    tm = torch.from_numpy(m_sizes).to(cuda)
    xa = to_dev(x, "bf16", cuda).requires_grad_()
    xb = xa.detach().clone().requires_grad_()
    dy = torch.randn(1024, 512, device=cuda).to(torch.bfloat16)
    moe_fused_linear_4bit(xa, packed, state, tm, fused=True).backward(dy)
    moe_fused_linear_4bit(xb, packed, state, tm, fused=False).backward(dy)
    assert_close(to_np(xa.grad), to_np(xb.grad), "bf16", "fused dX vs decode + dX")


@pytest.mark.parametrize("n,bs2", [(4096, 256), (1000 * 256, 256), (513 * 64, 64)])
def test_nested_absmax_decoded_on_the_device(cuda, n, bs2):
    """Double-quantised absmax -> fp32 absmax in one kernel, bit for bit what the oracle computes."""
    from qwen3_moe_fused.grouped_gemm.forward_4bit import _unnest_absmax
    from qwen3_moe_fused.quantize.nf4 import AbsmaxState, Nf4State

    rng = np.random.default_rng(n)
    q = rng.integers(0, 256, n).astype(np.uint8)
    code2 = np.sort(rng.uniform(-1, 1, 256)).astype(np.float32)
    absmax2 = rng.uniform(0.01, 0.2, n // bs2).astype(np.float32)
    offset = np.float32(0.0371)
    state = Nf4State(absmax=torch.from_numpy(q).to(cuda), code=torch.from_numpy(O.nf4_code()).to(cuda), blocksize=64,
                     shape=torch.Size((n * 64,)), dtype=torch.bfloat16, nested=True,
                     state2=AbsmaxState(torch.from_numpy(absmax2).to(cuda), torch.from_numpy(code2).to(cuda), bs2),
                     offset=torch.tensor([offset], device=cuda))
    got = _unnest_absmax(state).cpu().numpy()
    assert np.array_equal(got, O.absmax_unnest(q, code2, absmax2, bs2, offset))


def test_fused_forward_with_nested_absmax(cuda):
    """A weight whose absmax is itself quantised (double quantisation): the fused forward decodes the
    absmax on the device first and matches decode + GEMM of the oracle on the same quantised data."""
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_4bit
    from qwen3_moe_fused.quantize.nf4 import nest_absmax, quantize_nf4

    rng = np.random.default_rng(21)
    M, K, N, E, bs = 1024, 512, 512, 8, 64
    w = torch.from_numpy((rng.standard_normal((E, N, K)) / np.sqrt(K)).astype(np.float32)).to(cuda).to(torch.bfloat16)
    packed, state = quantize_nf4(w, bs)
    nested = nest_absmax(state, 256)
    assert nested.nested and nested.absmax.dtype == torch.uint8
    absmax = O.absmax_unnest(nested.absmax.cpu().numpy(), nested.state2.code.cpu().numpy(), nested.state2.absmax.cpu().numpy(),
                             256, float(nested.offset))
    # the nested absmax is close to the plain one (8-bit second level), and the kernel uses exactly the oracle's values
    assert np.abs(absmax - state.absmax.cpu().numpy()).max() <= 0.01 * state.absmax.abs().max().item()
    w_deq = O.nf4_dequantize(packed.cpu().numpy(), absmax, O.nf4_code(), bs, (E, N, K), "bf16")
    x = rounded(rng.standard_normal((M, K)), "bf16")
    m_sizes = random_m_sizes(rng, M, E, 0.1)
    y = grouped_gemm_forward_4bit(to_dev(x, "bf16", cuda), packed, nested, torch.from_numpy(m_sizes).to(cuda), fused=True)
    assert_close(to_np(y), O.grouped_gemm_fwd(x, w_deq, m_sizes, "bf16"), "bf16", "nested nf4 fwd")
