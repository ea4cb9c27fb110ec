"""Generates tests/golden/*.npz by running the REFERENCE's own Python code on CPU.

Run in a container that has the reference checkout:
    python tests/golden/make_golden.py /path/to/reference
The fixtures pin oracle/moe_oracle.py (and through it the CUDA kernels) to the reference:
  indexing_*.npz : get_expert_counts_and_idx / sort_experts / get_expert_counts /
                   get_batch_begins_ends run eagerly (qwen3_moe_fused/kernels/indexing.py)
  linear_*.npz   : _moe_fused_linear_naive_fwd / _bwd_input / _bwd_weight
                   (qwen3_moe_fused/functional.py:7-61)
  block_tiny.npz : Qwen3MoeFusedSparseMoeBlock.forward
                   (qwen3_moe_fused/modular_qwen3_moe_fused.py:64-118) with the reference's
                   own naive functions standing in for the Triton grouped GEMM
All inputs are seeded; nothing here is used at test time except the saved arrays.
"""
import sys
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import torch._dynamo

    torch._dynamo.config.disable = True  # run the @torch.compile'd indexing functions eagerly
    from qwen3_moe_fused import functional as F_ref
    from qwen3_moe_fused.kernels import indexing as I_ref

    # ---- indexing ----
    cases = {
        "c1": (256, 8, 0),          # the small fp32 case
        "ragged": (1000, 11, 1),    # E = 11 as in the reference's tiny model
        "empty_groups": (300, 16, 2),
        "single": (1, 4, 3),
        "wide": (4096, 128, 4),
    }
    for name, (M, E, seed) in cases.items():
        g = torch.Generator().manual_seed(seed)
        s = torch.randint(0, E, (M,), generator=g, dtype=torch.int64)
        if name == "empty_groups":
            s[s % 3 == 0] = 1  # several experts get no rows
        counts, inv_idx, idx = I_ref.get_expert_counts_and_idx(s, E)
        s_sorted, inv2, idx2 = I_ref.sort_experts(s, E)
        counts2 = I_ref.get_expert_counts(s, E)
        be = I_ref.get_batch_begins_ends(torch.sort(s).values, E)
        assert torch.equal(inv_idx, inv2) and torch.equal(idx, idx2) and torch.equal(counts, counts2)
        np.savez_compressed(
            OUT / f"indexing_{name}.npz", s=s.numpy(), E=E, counts=counts.numpy(), inv_idx=inv_idx.numpy(),
            idx=idx.numpy(), s_sorted=s_sorted.numpy(), begins_ends=be.numpy(),
        )

    # ---- moe_fused_linear fwd / dX / dW ----
    lin_cases = {
        "c1": (256, 64, 128, 8, 0),      # the small fp32 case: E=8, in=64, out=128, B=256
        "odd": (37, 3, 4, 11, 1),        # K=3, N=4, E=11: the reference's tiny-model shapes
        "empty": (96, 16, 24, 6, 2),
    }
    for name, (B, K, N, E, seed) in lin_cases.items():
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(B, K, generator=g)
        w = torch.randn(E, N, K, generator=g) / K**0.5
        s = torch.randint(0, E, (B,), generator=g)
        if name == "empty":
            s[s == 2] = 0
            s[s == 5] = 4
        dy = torch.randn(B, N, generator=g)
        y = F_ref._moe_fused_linear_naive_fwd(x, w, s)
        dx = F_ref._moe_fused_linear_naive_bwd_input(dy, x, w, s)
        dw = F_ref._moe_fused_linear_naive_bwd_weight(dy, x, w, s)
        np.savez_compressed(OUT / f"linear_{name}.npz", x=x.numpy(), w=w.numpy(), s=s.numpy(), dy=dy.numpy(),
                            y=y.numpy(), dx=dx.numpy(), dw=dw.numpy())

    # ---- whole block (tiny, fp32) ----
    from transformers import Qwen3MoeConfig

    from qwen3_moe_fused import modular_qwen3_moe_fused as M_ref

    def linear_via_naive(input, weight, m_sizes):
        experts = torch.repeat_interleave(torch.arange(weight.shape[0]), m_sizes.long())
        return F_ref._moe_fused_linear_naive_fwd(input, weight, experts)

    M_ref.moe_fused_linear = linear_via_naive
    torch.manual_seed(42)
    cfg = Qwen3MoeConfig(hidden_size=16, moe_intermediate_size=24, num_experts=11, num_experts_per_tok=3,
                         norm_topk_prob=True, hidden_act="silu")
    block = M_ref.Qwen3MoeFusedSparseMoeBlock(cfg)
    hidden = torch.randn(2, 13, 16)
    with torch.no_grad():
        out, logits = block(hidden)
    np.savez_compressed(
        OUT / "block_tiny.npz", hidden=hidden.numpy(), out=out.numpy(), logits=logits.numpy(),
        gate=block.gate.weight.detach().numpy(), gate_proj=block.gate_proj.weight.detach().numpy(),
        up_proj=block.up_proj.weight.detach().numpy(), down_proj=block.down_proj.weight.detach().numpy(),
        k=3,
    )
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <reference checkout>")
    main(sys.argv[1])
