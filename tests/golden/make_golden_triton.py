"""Fixtures made by EXECUTING the reference's Triton kernels on the CPU.

    python tests/golden/make_golden_triton.py /path/to/transformers-qwen3-moe-fused

Triton's interpreter (TRITON_INTERPRET=1) runs a `@triton.jit` function program by program with numpy, so
the reference's own kernel sources produce these vectors: SiLU-mul forward / backward / in-place backward
(kernels/silu_mul.py), the grouped GEMM forward, transposed forward (dX) and weight gradient
(grouped_gemm/forward.py, forward_transposed.py, backward_dw.py) and the forward with the 4-bit weight decoded
inside the kernel (grouped_gemm/forward_4bit.py), and the whole fused-LoRA expert MLP with its hand-written
backward (kernels/fast_lora.py, the reference's autograd function running on those kernels).  The kernels are
launched directly (`kernel.fn[grid](...)`, the function under the autotuner) with the argument lists of the reference's wrappers
(forward.py:138-159, forward_transposed.py:128-149, backward_dw.py:111-133, forward_4bit.py:183-207,
silu_mul.py:121-161), because the wrappers insist on CUDA tensors.  The interpreter has no bfloat16 (numpy
has none), so the fixtures are float16 and float32; the kernels' rounding points do not depend on which
16-bit type is stored.

`bitsandbytes` is imported by forward_4bit.py for two names only (a type annotation and the nested-absmax
call, neither on the path taken here); stand-ins are registered for them.  The packed weights, code table
and absmax of the 4-bit case are INPUTS made here (any table would do: the kernel receives it at run time),
so this pins the decode (nibble order, absmax indexing, rounding), not bitsandbytes' quantiser.

Writes tests/golden/triton_*.npz (a few hundred KB).
"""
import os
import sys
import types
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def _register_stand_ins():
    bnb = types.ModuleType("bitsandbytes")
    fn = types.ModuleType("bitsandbytes.functional")
    fn.QuantState = type("QuantState", (), {})
    fn.dequantize_blockwise = None
    fn.dequantize_4bit = None
    bnb.functional = fn
    sys.modules.setdefault("bitsandbytes", bnb)
    sys.modules.setdefault("bitsandbytes.functional", fn)


def _ragged_sizes(rng, M, E, empty):
    cuts = np.sort(rng.integers(0, M + 1, E - 1))
    sizes = np.diff(np.concatenate([[0], cuts, [M]])).astype(np.int64)
    for e in empty:
        if e + 1 < E:
            sizes[e + 1] += sizes[e]
        else:
            sizes[e - 1] += sizes[e]
        sizes[e] = 0
    assert sizes.sum() == M
    return sizes


def silu_cases(out):
    import triton
    from qwen3_moe_fused.kernels import silu_mul as S

    for name, dt in (("f16", torch.float16), ("f32", torch.float32)):
        g = torch.Generator().manual_seed(7)
        n = 1000  # not a multiple of the block: the mask is exercised
        e = (torch.randn(n, generator=g) * 3).to(dt)
        gate = torch.randn(n, generator=g).to(dt)
        dh = torch.randn(n, generator=g).to(dt)
        grid = (triton.cdiv(n, 128),)
        h = torch.empty_like(e)
        S._silu_mul_forward_kernel.fn[grid](e, gate, h, n, BLOCK_SIZE=128)
        de, dg = torch.empty_like(e), torch.empty_like(e)
        S._silu_mul_backward_kernel.fn[grid](dh, e, gate, de, dg, n, BLOCK_SIZE=128)
        dh2, e2, g2 = dh.clone(), e.clone(), gate.clone()
        S._silu_mul_backward_inplace_kernel.fn[grid](dh2, e2, g2, n, BLOCK_SIZE=128)
        f32 = lambda t: t.float().numpy()
        np.savez_compressed(out / f"triton_silu_mul_{name}.npz", e=f32(e), g=f32(gate), dh=f32(dh), h=f32(h), de=f32(de),
                            dg=f32(dg), inplace_h=f32(dh2), inplace_de=f32(e2), inplace_dg=f32(g2))
        print("silu", name, "ok")


def gemm_cases(out):
    forward, forward_transposed, backward_dw, _, _ = _interpreted_wrappers()
    for name, dt, M, N, K, E, empty in (("f16", torch.float16, 150, 48, 40, 6, (2,)),
                                        ("f32", torch.float32, 97, 24, 36, 5, (0, 4))):
        rng = np.random.default_rng(M)
        g = torch.Generator().manual_seed(M)
        sizes = _ragged_sizes(rng, M, E, empty)
        m_sizes = torch.from_numpy(sizes).to(torch.int32)
        x = torch.randn(M, K, generator=g).to(dt)
        w = (torch.randn(E, N, K, generator=g) * K ** -0.5).to(dt)
        dy = torch.randn(M, N, generator=g).to(dt)
        y = forward(x, w, m_sizes)
        dx = forward_transposed(dy, w, m_sizes)  # rows dy (M, N) times w (E, N, K) read transposed -> (M, K)
        dw = backward_dw(x, dy, m_sizes, dt)
        f32 = lambda t: t.float().numpy()
        np.savez_compressed(out / f"triton_grouped_gemm_{name}.npz", x=f32(x), w=f32(w), dy=f32(dy), m_sizes=sizes,
                            y=f32(y), dx=f32(dx), dw=f32(dw))
        print("gemm", name, "ok")


def _interpreted_wrappers(sms=4, block=32):
    """The reference's five wrappers (same arguments, same results) for CPU tensors: each launches the reference's
    kernel under the interpreter exactly as the wrapper in the reference does."""
    import triton
    from qwen3_moe_fused.grouped_gemm import backward_dw as DW
    from qwen3_moe_fused.grouped_gemm import forward as FW
    from qwen3_moe_fused.grouped_gemm import forward_transposed as FT
    from qwen3_moe_fused.kernels import silu_mul as S

    blocks = dict(BLOCK_SIZE_M=block, BLOCK_SIZE_N=block, BLOCK_SIZE_K=block)

    def forward(x, w, m_sizes, dtype=None):
        (M, K), (E, N, _) = x.shape, w.shape
        y = torch.zeros((M, N), dtype=dtype or x.dtype)
        FW._grouped_gemm_forward_kernel.fn[(sms,)](x, w, m_sizes, y, M, N, K, E, sms, x.stride(0), x.stride(1), w.stride(0),
                                                   w.stride(1), w.stride(2), y.stride(0), y.stride(1), **blocks)
        return y

    def forward_transposed(x, w, m_sizes, dtype=None):
        (M, K), (E, _, N) = x.shape, w.shape
        y = torch.zeros((M, N), dtype=dtype or x.dtype)
        FT._grouped_gemm_forward_transposed_kernel.fn[(sms,)](x, w, m_sizes, y, M, N, K, E, sms, x.stride(0), x.stride(1),
                                                              w.stride(0), w.stride(1), w.stride(2), y.stride(0), y.stride(1),
                                                              **blocks)
        return y

    def backward_dw(x, y, m_sizes, dtype):
        (M, K), N, E = x.shape, y.shape[1], m_sizes.numel()
        w = torch.zeros((E, N, K), dtype=dtype)
        DW._grouped_gemm_backward_dw_kernel.fn[(sms,)](x, y, m_sizes, w, M, N, K, E, sms, x.stride(0), x.stride(1), y.stride(0),
                                                       y.stride(1), w.stride(0), w.stride(1), w.stride(2), **blocks)
        return w

    def silu_forward(e, g):
        h = torch.empty_like(e)
        S._silu_mul_forward_kernel.fn[(triton.cdiv(e.numel(), 128),)](e, g, h, e.numel(), BLOCK_SIZE=128)
        return h

    def silu_backward_inplace(dh, e, g):
        S._silu_mul_backward_inplace_kernel.fn[(triton.cdiv(e.numel(), 128),)](dh, e, g, e.numel(), BLOCK_SIZE=128)

    return forward, forward_transposed, backward_dw, silu_forward, silu_backward_inplace


def fast_lora_case(out):
    """The reference's `FastLora` autograd function (kernels/fast_lora.py:66-175), unchanged, with the five kernel
    wrappers it imports rebound to the interpreter-backed ones: forward and all seven gradients in float16."""
    import qwen3_moe_fused.kernels.fast_lora as FL

    (FL.grouped_gemm_forward, FL.grouped_gemm_forward_transposed, FL.grouped_gemm_backward_dw, FL.silu_mul_forward,
     FL.silu_mul_backward_inplace) = _interpreted_wrappers()
    B, H, I, E, R = 120, 32, 48, 4, 8
    rng = np.random.default_rng(11)
    g = torch.Generator().manual_seed(11)
    dt = torch.float16
    sizes = _ragged_sizes(rng, B, E, (2,))
    m_sizes = torch.from_numpy(sizes).to(torch.int32)
    mk = lambda *s, scale=1.0: (torch.randn(*s, generator=g) * scale).to(dt)
    x = mk(B, H).requires_grad_()
    G, U, W = mk(E, I, H, scale=H ** -0.5), mk(E, I, H, scale=H ** -0.5), mk(E, H, I, scale=I ** -0.5)
    loras = [mk(E, R, H, scale=H ** -0.5), mk(E, I, R, scale=0.1), mk(E, R, H, scale=H ** -0.5), mk(E, I, R, scale=0.1),
             mk(E, R, I, scale=I ** -0.5), mk(E, H, R, scale=0.1)]
    Ag, Bg, Au, Bu, Aw, Bw = (t.requires_grad_() for t in loras)
    Sg, Su, Sw = 0.5, 2.0, 1.0
    dy = mk(B, H)
    y = FL.fast_lora(x, G, None, Ag, Bg, Sg, U, None, Au, Bu, Su, W, None, Aw, Bw, Sw, m_sizes)
    y.backward(dy)
    f32 = lambda t: t.detach().float().numpy()
    np.savez_compressed(out / "triton_fast_lora_f16.npz", x=f32(x), G=f32(G), U=f32(U), W=f32(W), Ag=f32(Ag), Bg=f32(Bg),
                        Au=f32(Au), Bu=f32(Bu), Aw=f32(Aw), Bw=f32(Bw), scalings=np.array([Sg, Su, Sw]), dy=f32(dy),
                        m_sizes=sizes, y=f32(y), dx=f32(x.grad), dAg=f32(Ag.grad), dBg=f32(Bg.grad), dAu=f32(Au.grad),
                        dBu=f32(Bu.grad), dAw=f32(Aw.grad), dBw=f32(Bw.grad))
    print("fast_lora ok")


def nf4_case(out):
    from oracle import moe_oracle as O
    from qwen3_moe_fused.grouped_gemm import forward_4bit as F4

    M, N, K, E, bs = 90, 32, 64, 4, 32
    rng = np.random.default_rng(4)
    g = torch.Generator().manual_seed(4)
    sizes = _ragged_sizes(rng, M, E, (1,))
    m_sizes = torch.from_numpy(sizes).to(torch.int32)
    x = torch.randn(M, K, generator=g).to(torch.float16)
    packed = torch.from_numpy(rng.integers(0, 256, E * N * K // 2, dtype=np.uint8))  # every nibble value occurs
    code = torch.from_numpy(O.nf4_code().astype(np.float32))
    absmax = torch.from_numpy((rng.random(E * N * K // bs) * 0.2 + 0.01).astype(np.float32))
    y = torch.zeros((M, N), dtype=torch.float16)
    sms = 4
    F4._grouped_gemm_forward_4bit_kernel.fn[(sms,)](x, packed, code, absmax, bs, m_sizes, y, M, N, K, E, sms, x.stride(0),
                                                    x.stride(1), N * K, K, 1, y.stride(0), y.stride(1),
                                                    BLOCK_SIZE_M=32, BLOCK_SIZE_N=32, BLOCK_SIZE_K=32)
    np.savez_compressed(out / "triton_forward_4bit_f16.npz", x=x.float().numpy(), packed=packed.numpy(), code=code.numpy(),
                        absmax=absmax.numpy(), blocksize=bs, m_sizes=sizes, shape=np.array([E, N, K]), y=y.float().numpy())
    print("nf4 ok")


def main():
    ref = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QWEN3_MOE_FUSED_REFERENCE_CHECKOUT", ""))
    assert (ref / "qwen3_moe_fused" / "kernels" / "silu_mul.py").exists(), "pass the reference checkout's directory"
    sys.path.insert(0, str(ref))
    _register_stand_ins()
    silu_cases(HERE)
    gemm_cases(HERE)
    nf4_case(HERE)
    fast_lora_case(HERE)


if __name__ == "__main__":
    main()
