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


def check_errors() -> None:
    """Raises if a kernel of this library recorded an error since the last check.

    The tensor-core kernels bound every wait inside them (2 s); a wait that runs out makes the
    kernel return early with its output incomplete and records a code in a device-side word, and
    a misaligned per-group output address is recorded the same way.  Launches never read that word
    (it would cost a device synchronisation per call), so a program that wants to know calls this
    at a point where a synchronisation is acceptable, for instance once per training step.
    """
    from . import _lib

    flag = _lib.read_error_flag()
    if flag:
        raise _lib.MoeB200Error(f"a kernel reported error code {flag >> 16} (first reporter: CTA {flag & 0xffff}); "
                                "outputs of the calls since the last check may be incomplete")
