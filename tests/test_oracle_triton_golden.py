"""The oracle against fixtures made by executing the reference's Triton kernels under Triton's CPU
interpreter (tests/golden/make_golden_triton.py): SiLU-mul's rounding points, the three grouped GEMMs on
ragged groups with empty experts, and the 4-bit decode inside the forward kernel (nibble order, absmax
indexing, rounding of the decoded weight).  float16 / float32 (the interpreter has no bfloat16)."""
import numpy as np
import pytest

from oracle import moe_oracle as O

F16_STEP = 2.0 ** -10  # relative spacing of float16


def _within_one_step(got, want, step):
    """Equal up to one storage step of the larger magnitude (an fp32 sum in another order can flip a rounding)."""
    tol = np.maximum(np.abs(got), np.abs(want)) * step + 1e-7
    return np.abs(got - want) <= tol


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_silu_mul_rounding_points_match_the_triton_kernels(golden, dtype):
    g = golden(f"triton_silu_mul_{dtype}")
    e, gate, dh = g["e"], g["g"], g["dh"]
    h = O.silu_mul_fwd(e, gate, dtype)
    h2, de, dg = O.silu_mul_bwd(dh, e, gate, dtype)
    if dtype == "f16":
        # 16-bit storage: every rounding point of silu_mul.py:34-39,62-73 has to sit where the oracle puts it.
        # The sigmoid itself is fp32 in both, evaluated by different routines: allow one storage step.
        for got, want, name in ((h, g["h"], "h"), (h2, g["h"], "h (backward)"), (de, g["de"], "de"), (dg, g["dg"], "dg")):
            ok = _within_one_step(got, want, F16_STEP)
            assert ok.all(), f"{name}: {(~ok).sum()} of {ok.size} differ by more than one float16 step"
            assert (got == want).mean() > 0.97, f"{name}: only {(got == want).mean():.3f} bit-identical"
    else:
        for got, want in ((h, g["h"]), (h2, g["h"]), (de, g["de"]), (dg, g["dg"])):
            np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-7)
    # the in-place kernel (silu_mul.py:97-111) writes the same three results over its inputs
    np.testing.assert_array_equal(g["inplace_h"], g["h"])
    np.testing.assert_array_equal(g["inplace_de"], g["de"])
    np.testing.assert_array_equal(g["inplace_dg"], g["dg"])


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_grouped_gemms_match_the_triton_kernels(golden, dtype):
    g = golden(f"triton_grouped_gemm_{dtype}")
    x, w, dy, m_sizes = g["x"], g["w"], g["dy"], g["m_sizes"]
    assert (m_sizes == 0).any() and m_sizes.sum() == x.shape[0]
    y, dx, dw = O.grouped_gemm_fwd(x, w, m_sizes, dtype), O.grouped_gemm_dx(dy, w, m_sizes, dtype), O.grouped_gemm_dw(x, dy, m_sizes, dtype)
    if dtype == "f16":
        for got, want, name in ((y, g["y"], "y"), (dx, g["dx"], "dx"), (dw, g["dw"], "dw")):
            assert _within_one_step(got, want, F16_STEP).all(), name
            assert (got == want).mean() > 0.97, f"{name}: only {(got == want).mean():.3f} bit-identical"
    else:
        # the kernels' tl.dot on fp32 inputs is evaluated by the interpreter in fp32; sums in another order
        np.testing.assert_allclose(y, g["y"], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(dx, g["dx"], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(dw, g["dw"], rtol=1e-5, atol=1e-5)
    empty = np.flatnonzero(m_sizes == 0)
    assert not g["dw"][empty].any() and not dw[empty].any(), "experts without rows get a zero weight gradient"


def test_4bit_decode_matches_the_triton_kernel(golden):
    g = golden("triton_forward_4bit_f16")
    E, N, K = (int(v) for v in g["shape"])
    w = O.nf4_dequantize(g["packed"], g["absmax"], g["code"], int(g["blocksize"]), (E, N, K), "f16")
    y = O.grouped_gemm_fwd(g["x"], w, g["m_sizes"], "f16")
    assert _within_one_step(y, g["y"], F16_STEP).all()
    assert (y == g["y"]).mean() > 0.97
    # the check has teeth: the other nibble order, or absmax indexed per row instead of per flat block, is far off
    swapped = ((g["packed"] >> 4) | (g["packed"] << 4)).astype(np.uint8)
    w_swapped = O.nf4_dequantize(swapped, g["absmax"], g["code"], int(g["blocksize"]), (E, N, K), "f16")
    assert O.rel_err(O.grouped_gemm_fwd(g["x"], w_swapped, g["m_sizes"], "f16"), g["y"]) > 0.2
    rolled = np.roll(g["absmax"], 1)
    w_rolled = O.nf4_dequantize(g["packed"], rolled, g["code"], int(g["blocksize"]), (E, N, K), "f16")
    assert O.rel_err(O.grouped_gemm_fwd(g["x"], w_rolled, g["m_sizes"], "f16"), g["y"]) > 0.05
