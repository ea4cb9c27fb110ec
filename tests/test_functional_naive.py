"""The definitional torch functions kept beside `moe_fused_linear` (the reference's tests import them
from `qwen3_moe_fused.functional`) against fixtures made by the reference's own functions (CPU)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "transformers-qwen3-moe-fused_b200"))


@pytest.mark.parametrize("name", ["c1", "odd", "empty"])
def test_naive_functions_match_reference_fixtures(golden, name):
    from qwen3_moe_fused import functional as F

    g = golden(f"linear_{name}")
    x, w, dy = (torch.from_numpy(g[k]) for k in ("x", "w", "dy"))
    s = torch.from_numpy(g["s"])
    y = F._moe_fused_linear_naive_fwd(x, w, s)
    dx = F._moe_fused_linear_naive_bwd_input(dy, x, w, s)
    dw = F._moe_fused_linear_naive_bwd_weight(dy, x, w, s)
    assert y.dtype == x.dtype and dx.shape == x.shape and dw.shape == w.shape
    np.testing.assert_allclose(y.numpy(), g["y"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dx.numpy(), g["dx"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(dw.numpy(), g["dw"], rtol=1e-4, atol=1e-4)


def test_naive_functions_in_steps_and_against_autograd(monkeypatch):
    """More rows than one step gathers at once, int32 ids, and the two backward functions against
    torch autograd of the forward one (what test_moe_fused_linear_bwd.py:49-59 of the reference does)."""
    from qwen3_moe_fused import functional as F

    monkeypatch.setattr(F, "_NAIVE_ROWS_PER_STEP", 7)
    gen = torch.Generator().manual_seed(5)
    B, K, N, E = 50, 12, 9, 6
    x = torch.randn(B, K, generator=gen, requires_grad=True)
    w = torch.randn(E, N, K, generator=gen, requires_grad=True)
    s = torch.randint(0, E - 1, (B,), generator=gen).to(torch.int32)   # the last expert stays empty
    dy = torch.randn(B, N, generator=gen)
    y = F._moe_fused_linear_naive_fwd(x, w, s)
    y.backward(dy)
    with torch.no_grad():
        ref = torch.stack([w[int(s[b])] @ x[b] for b in range(B)])
        assert torch.allclose(y, ref, atol=1e-5)
        assert torch.allclose(F._moe_fused_linear_naive_bwd_input(dy, x, w, s), x.grad, atol=1e-5)
        dw = F._moe_fused_linear_naive_bwd_weight(dy, x, w, s)
        assert torch.allclose(dw, w.grad, atol=1e-5) and bool((dw[E - 1] == 0).all())
