"""Whole sparse-MoE block and the fused-LoRA expert MLP vs CPU references."""
import numpy as np
import pytest
import torch

from oracle import moe_oracle as O
from tests.helpers import assert_close, random_m_sizes, rounded, to_dev, to_np

pytestmark = pytest.mark.gpu


def test_block_golden_fp32(golden, cuda):
    from qwen3_moe_fused.moe_block import moe_block_forward

    g = golden("block_tiny")
    t = lambda a: torch.from_numpy(a).to(cuda)
    out, logits = moe_block_forward(t(g["hidden"]), t(g["gate"]), t(g["gate_proj"]), t(g["up_proj"]), t(g["down_proj"]),
                                    int(g["k"]), True)
    np.testing.assert_allclose(to_np(logits), g["logits"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(to_np(out), g["out"], rtol=1e-3, atol=1e-5)


def test_block_bf16_vs_oracle(cuda):
    from qwen3_moe_fused.moe_block import moe_block_forward

    rng = np.random.default_rng(0)
    T, H, I, E, k = 512, 256, 128, 16, 4
    hidden = rounded(rng.standard_normal((T, H)), "bf16")
    # fp32 router on the host side of the test keeps expert choice identical on both sides
    gate = rounded(rng.standard_normal((E, H)) * 0.02, "bf16")
    gp = rounded(rng.standard_normal((E, I, H)) * 0.05, "bf16")
    up = rounded(rng.standard_normal((E, I, H)) * 0.05, "bf16")
    dp = rounded(rng.standard_normal((E, H, I)) * 0.05, "bf16")
    out, logits = moe_block_forward(to_dev(hidden, "bf16", cuda).view(1, T, H), to_dev(gate, "bf16", cuda),
                                    to_dev(gp, "bf16", cuda), to_dev(up, "bf16", cuda), to_dev(dp, "bf16", cuda), k, True)
    # feed the device's logits to the oracle so that a 1-ulp difference in the router GEMM
    # cannot flip an expert choice
    lg = to_np(logits)
    weights, experts = O.router_softmax_topk(lg, k, True, "bf16")
    m_sizes, sort_idx, inv_sort_idx = O.get_expert_counts_and_idx_fast(experts.reshape(-1), E)
    xs = O.gather_rows(hidden, sort_idx, k)
    h = O.silu_mul_fwd(O.grouped_gemm_fwd(xs, gp, m_sizes, "bf16"), O.grouped_gemm_fwd(xs, up, m_sizes, "bf16"), "bf16")
    ref = O.combine(O.grouped_gemm_fwd(h, dp, m_sizes, "bf16"), inv_sort_idx, weights, "bf16")
    assert_close(to_np(out).reshape(T, H), ref, "bf16", "block", scale=2)


def test_block_backward_fp32(cuda):
    from qwen3_moe_fused.moe_block import moe_block_forward

    torch.manual_seed(0)
    T, H, I, E, k = 96, 32, 48, 6, 2
    hidden = torch.randn(1, T, H, device=cuda, requires_grad=True)
    gate = (torch.randn(E, H, device=cuda) * 0.5).requires_grad_()
    gp = (torch.randn(E, I, H, device=cuda) * 0.2).requires_grad_()
    up = (torch.randn(E, I, H, device=cuda) * 0.2).requires_grad_()
    dp = (torch.randn(E, H, I, device=cuda) * 0.2).requires_grad_()
    out, _ = moe_block_forward(hidden, gate, gp, up, dp, k, True)
    out.square().sum().backward()

    # dense per-token torch definition on the CPU
    hc, gc, gpc, upc, dpc = (t.detach().cpu().clone().requires_grad_() for t in (hidden, gate, gp, up, dp))
    x = hc.view(T, H)
    p = torch.softmax(x @ gc.T, dim=1)
    tw, ti = torch.topk(p, k, dim=-1)
    tw = tw / tw.sum(-1, keepdim=True)
    ref = torch.zeros(T, H)
    for j in range(k):
        e = ti[:, j]
        hmid = torch.nn.functional.silu(torch.einsum("tih,th->ti", gpc[e], x)) * torch.einsum("tih,th->ti", upc[e], x)
        ref = ref + tw[:, j:j + 1] * torch.einsum("thi,ti->th", dpc[e], hmid)
    ref.square().sum().backward()
    assert torch.allclose(out.detach().cpu().view(T, H), ref.detach(), rtol=1e-3, atol=1e-4)
    for got, want, name in ((hidden.grad, hc.grad, "hidden"), (gate.grad, gc.grad, "gate"), (gp.grad, gpc.grad, "gate_proj"),
                            (up.grad, upc.grad, "up_proj"), (dp.grad, dpc.grad, "down_proj")):
        assert torch.allclose(got.cpu(), want, rtol=2e-3, atol=2e-4), name


def _fast_lora_reference(x, G, Ag, Bg, Sg, U, Au, Bu, Su, W, Aw, Bw, Sw, m_sizes):
    """fp32 torch definition of the fused-LoRA expert MLP (math notes at
    qwen3_moe_fused/kernels/fast_lora.py:1-46 of the reference)."""
    out = []
    row = 0
    for e, n in enumerate(m_sizes.tolist()):
        xe = x[row:row + n]
        Gp = G[e] + Sg * Bg[e] @ Ag[e]
        Up = U[e] + Su * Bu[e] @ Au[e]
        Wp = W[e] + Sw * Bw[e] @ Aw[e]
        h = torch.nn.functional.silu(xe @ Gp.T) * (xe @ Up.T)
        out.append(h @ Wp.T)
        row += n
    return torch.cat(out)


@pytest.mark.parametrize("dtype,quant", [("f32", False), ("bf16", False), ("bf16", True)])
def test_fast_lora_forward_backward(cuda, dtype, quant):
    from qwen3_moe_fused.kernels.fast_lora import fast_lora
    from qwen3_moe_fused.quantize.nf4 import dequantize_4bit, quantize_nf4
    from tests.helpers import DT

    torch.manual_seed(1)
    rng = np.random.default_rng(1)
    B, H, I, E, R = 384, 128, 192, 6, 16
    dt = DT[dtype]
    m_sizes = torch.from_numpy(random_m_sizes(rng, B, E, 0.2)).to(cuda)
    mk = lambda *s, scale=1.0: (torch.randn(*s, device=cuda) * scale).to(dt)
    x = mk(B, H).requires_grad_()
    G, U, W = mk(E, I, H, scale=H ** -0.5), mk(E, I, H, scale=H ** -0.5), mk(E, H, I, scale=I ** -0.5)
    loras = [mk(E, R, H, scale=H ** -0.5), mk(E, I, R, scale=0.1), mk(E, R, H, scale=H ** -0.5), mk(E, I, R, scale=0.1),
             mk(E, R, I, scale=I ** -0.5), mk(E, H, R, scale=0.1)]
    Ag, Bg, Au, Bu, Aw, Bw = (t.requires_grad_() for t in loras)
    Sg, Su, Sw = 0.5, 2.0, 1.0
    if quant:
        (Gq, Gs), (Uq, Us), (Wq, Ws) = (quantize_nf4(t, 64) for t in (G, U, W))
        G, U, W = (dequantize_4bit(q, s, dt) for q, s in ((Gq, Gs), (Uq, Us), (Wq, Ws)))
    else:
        Gq, Uq, Wq, Gs, Us, Ws = G, U, W, None, None, None
    y = fast_lora(x, Gq, Gs, Ag, Bg, Sg, Uq, Us, Au, Bu, Su, Wq, Ws, Aw, Bw, Sw, m_sizes)
    dy = mk(B, H)
    y.backward(dy)

    cpu = lambda t: t.detach().float().cpu().clone().requires_grad_()
    xr, Agr, Bgr, Aur, Bur, Awr, Bwr = map(cpu, (x, Ag, Bg, Au, Bu, Aw, Bw))
    yr = _fast_lora_reference(xr, G.float().cpu(), Agr, Bgr, Sg, U.float().cpu(), Aur, Bur, Su, W.float().cpu(), Awr, Bwr, Sw,
                              m_sizes.cpu())
    yr.backward(dy.float().cpu())
    # bf16 against the fp32 definition: storing e, g, h, A x and the gradients' intermediates in bf16 moves every
    # result by 0.5-1 % of its largest element, in the reference's order of operations as much as in this one
    # (tests/test_fast_lora_rounding.py measures both on the CPU), so 1e-2 has no margin; 2e-2 is the bar
    tol = 2e-4 if dtype == "f32" else 2e-2
    def rel(a, b):
        return float((a.float().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))
    assert rel(y, yr.detach()) < tol, "y"
    for got, want, name in ((x.grad, xr.grad, "dx"), (Ag.grad, Agr.grad, "dAg"), (Bg.grad, Bgr.grad, "dBg"),
                            (Au.grad, Aur.grad, "dAu"), (Bu.grad, Bur.grad, "dBu"), (Aw.grad, Awr.grad, "dAw"),
                            (Bw.grad, Bwr.grad, "dBw")):
        assert rel(got, want) < tol, name


def test_block_patch_installs_the_fused_forward(cuda):
    """`patch_Qwen3MoeFusedSparseMoeBlock_forward` on a class with the reference block's attributes
    (modular_qwen3_moe_fused.py:62-77 of the reference): same output and gradients as the block's own
    sequence of calls, and LoRA-wrapped projections are refused."""
    from torch import nn

    from qwen3_moe_fused.moe_block import MoeFusedLinear, moe_block_forward, patch_Qwen3MoeFusedSparseMoeBlock_forward

    class Block(nn.Module):
        def __init__(self, H, I, E, k):
            super().__init__()
            self.num_experts, self.num_selected, self.norm_topk_prob = E, k, True
            self.gate = nn.Linear(H, E, bias=False)
            self.gate_proj, self.up_proj, self.down_proj = MoeFusedLinear(H, I, E), MoeFusedLinear(H, I, E), MoeFusedLinear(I, H, E)

        def forward(self, hidden_states):
            raise AssertionError("the patch replaces this")

    torch.manual_seed(4)
    H, I, E, k, T = 256, 192, 8, 2, 300
    blk = Block(H, I, E, k).to(cuda).to(torch.bfloat16)
    patch_Qwen3MoeFusedSparseMoeBlock_forward(Block)
    x = torch.randn(1, T, H, device=cuda).to(torch.bfloat16).requires_grad_()
    out, logits = blk(x)
    out.float().square().sum().backward()
    x2 = x.detach().clone().requires_grad_()
    ref, ref_logits = moe_block_forward(x2, blk.gate.weight.detach(), blk.gate_proj.weight.detach(), blk.up_proj.weight.detach(),
                                        blk.down_proj.weight.detach(), k, True)
    ref.float().square().sum().backward()
    assert torch.equal(out, ref) and torch.equal(logits, ref_logits) and torch.equal(x.grad, x2.grad)
    assert blk.down_proj.weight.grad is not None and blk.gate.weight.grad is not None
    with torch.no_grad():  # inference: gate, up and SiLU-mul in one kernel, same bits
        out_ng, _ = blk(x)
    assert torch.equal(out_ng, out)
    object.__setattr__(blk.up_proj, "base_layer", object())  # what a LoRA wrapper looks like
    with pytest.raises(NotImplementedError):
        blk(x)
