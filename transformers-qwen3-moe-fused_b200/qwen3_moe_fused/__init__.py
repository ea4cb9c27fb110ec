"""B200-native implementation of the `qwen3_moe_fused` hot path.

The package keeps the import paths of the reference project for the modules it
replaces (`functional`, `grouped_gemm.*`, `kernels.*`).  Modules of the reference that
are pure callers of this path (`modular_qwen3_moe_fused`, `lora`, `fast_lora`,
`quantize.layer`) can be layered underneath unchanged: set the environment variable
`QWEN3_MOE_FUSED_REFERENCE` to the directory that holds the reference's
`qwen3_moe_fused/` package and its files become importable as sub-modules of this one,
bound to the kernels here.
"""
import os as _os

_ref = _os.environ.get("QWEN3_MOE_FUSED_REFERENCE")
if _ref:
    _ref_pkg = _os.path.join(_ref, "qwen3_moe_fused")
    if _os.path.isdir(_ref_pkg) and _ref_pkg not in __path__:
        __path__.append(_ref_pkg)
