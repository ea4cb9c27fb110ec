"""The reference's caller modules, loaded unchanged through the overlay, bind to this package.

`QWEN3_MOE_FUSED_REFERENCE` makes the files of a reference checkout importable as sub-modules
of this package (qwen3_moe_fused/__init__.py).  The callers are `modular_qwen3_moe_fused.py`,
`fast_lora.py`, `lora.py` and `quantize/layer.py`; the last three import `peft` / `bitsandbytes`,
which are not installed here, so the test supplies minimal stand-ins for the names they import.
Runs in a child process because the variable is read when the package is first imported.
Needs a reference checkout (skipped without one); no GPU.
"""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG_ROOT = ROOT / "transformers-qwen3-moe-fused_b200"
REFERENCE = Path(os.environ.get("QWEN3_MOE_FUSED_REFERENCE_CHECKOUT", "/root/reference"))

CHILD = textwrap.dedent(
    """
    import sys, types
    import torch
    from torch import nn

    def module(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        sys.modules[name] = m
        return m

    # stand-ins for the names the reference's callers import from peft / bitsandbytes
    class LoraLayer:
        def __init__(self, base_layer, **kw):
            self.base_layer = base_layer
            self.lora_A, self.lora_B, self.lora_dropout = nn.ModuleDict(), nn.ModuleDict(), nn.ModuleDict()
            self.scaling, self.r, self.lora_alpha = {}, {}, {}
    module("peft", LoraConfig=type("LoraConfig", (), {}))
    module("peft.tuners"); module("peft.tuners.lora"); module("peft.tuners.lora.layer", LoraLayer=LoraLayer)
    class Params4bit(torch.nn.Parameter):
        pass
    module("bitsandbytes")
    module("bitsandbytes.functional", QuantState=type("QuantState", (), {}), dequantize_4bit=lambda w, s: w)
    module("bitsandbytes.nn", Linear4bit=type("Linear4bit", (nn.Module,), {}))
    module("bitsandbytes.nn.modules", Params4bit=Params4bit, fix_4bit_weight_quant_state_from_module=lambda m: None)

    import qwen3_moe_fused
    from qwen3_moe_fused import functional, kernels
    from qwen3_moe_fused.kernels import indexing, fast_lora as fast_lora_kernel
    pkg_dir = PKG_DIR
    ref_dir = REF_DIR

    def from_reference(mod):
        assert mod.__file__.startswith(ref_dir), (mod.__name__, mod.__file__)
    def from_package(obj):
        assert sys.modules[obj.__module__].__file__.startswith(pkg_dir), (obj, sys.modules[obj.__module__].__file__)

    # modules that exist in both places resolve to this package
    for mod in (functional, indexing, fast_lora_kernel):
        assert mod.__file__.startswith(pkg_dir), mod.__file__

    import qwen3_moe_fused.modular_qwen3_moe_fused as modular
    from_reference(modular)
    from_package(modular.moe_fused_linear)
    from_package(modular.get_expert_counts_and_idx)
    assert modular.moe_fused_linear is functional.moe_fused_linear

    import qwen3_moe_fused.fast_lora as fl
    from_reference(fl)
    assert fl.fast_lora is fast_lora_kernel.fast_lora
    assert fl.get_expert_counts_and_idx is indexing.get_expert_counts_and_idx
    assert callable(fl.patch_Qwen3MoeFusedSparseMoeBlock_forward)

    import qwen3_moe_fused.lora as lora
    from_reference(lora)
    assert lora.MoeFusedLinear is modular.MoeFusedLinear

    import qwen3_moe_fused.quantize.layer as qlayer
    from_reference(qlayer)
    from_package(qlayer.moe_fused_linear)
    assert issubclass(qlayer.MoeFusedLinear4bit, modular.MoeFusedLinear)

    # the import lines of the reference's kernel tests and benchmarks (test_moe_fused_linear.py:9-11,
    # test_moe_fused_linear_bwd.py:8-14, benchmark_moe_fused_linear*.py:10-13) resolve to this package
    from qwen3_moe_fused.functional import (_moe_fused_linear_naive_bwd_input, _moe_fused_linear_naive_bwd_weight,
                                            _moe_fused_linear_naive_fwd, moe_fused_linear)
    from qwen3_moe_fused.grouped_gemm.backward_dw import grouped_gemm_backward_dw
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_4bit import grouped_gemm_forward_4bit
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
    from qwen3_moe_fused.kernels.indexing import get_expert_counts
    for fn in (_moe_fused_linear_naive_fwd, _moe_fused_linear_naive_bwd_input, _moe_fused_linear_naive_bwd_weight,
               moe_fused_linear, grouped_gemm_forward, grouped_gemm_forward_transposed, grouped_gemm_backward_dw,
               grouped_gemm_forward_4bit, get_expert_counts):
        from_package(fn)

    # the reference's module classes build on the CPU and call this package's function
    lin = modular.MoeFusedLinear(8, 16, 4)
    assert tuple(lin.weight.shape) == (4, 16, 8)
    calls = []
    real = functional.moe_fused_linear
    modular.moe_fused_linear = lambda *a: calls.append(a) or torch.zeros(3, 16)
    lin(torch.zeros(3, 8), torch.tensor([1, 1, 1, 0]))
    assert len(calls) == 1 and calls[0][1] is lin.weight
    modular.moe_fused_linear = real
    # the block patch of this package installs on the reference's block class
    from qwen3_moe_fused import moe_block
    moe_block.patch_Qwen3MoeFusedSparseMoeBlock_forward()
    assert modular.Qwen3MoeFusedSparseMoeBlock.forward is moe_block.fused_sparse_moe_block_forward
    from transformers import Qwen3MoeConfig
    cfg = Qwen3MoeConfig(hidden_size=16, moe_intermediate_size=8, num_experts=4, num_experts_per_tok=2, norm_topk_prob=True)
    blk = modular.Qwen3MoeFusedSparseMoeBlock(cfg)
    seen = []
    moe_block.moe_block_forward = lambda *a: seen.append(a) or (torch.zeros(1, 3, 16), torch.zeros(3, 4))
    out, logits = blk(torch.zeros(1, 3, 16))
    assert seen and seen[0][1] is blk.gate.weight and seen[0][2] is blk.gate_proj.weight and seen[0][5] == 2
    print("overlay ok")
    """
)


@pytest.mark.skipif(not (REFERENCE / "qwen3_moe_fused" / "modular_qwen3_moe_fused.py").exists(),
                    reason="no reference checkout on this machine")
def test_reference_callers_bind_to_this_package():
    env = dict(os.environ)
    env["QWEN3_MOE_FUSED_REFERENCE"] = str(REFERENCE)
    env["PYTHONPATH"] = str(PKG_ROOT) + os.pathsep + env.get("PYTHONPATH", "")
    src = CHILD.replace("PKG_DIR", repr(str(PKG_ROOT))).replace("REF_DIR", repr(str(REFERENCE)))
    res = subprocess.run([sys.executable, "-c", src], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "overlay ok" in res.stdout
