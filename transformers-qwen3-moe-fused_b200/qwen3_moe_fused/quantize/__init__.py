import os as _os

_ref = _os.environ.get("QWEN3_MOE_FUSED_REFERENCE")
if _ref:
    _ref_pkg = _os.path.join(_ref, "qwen3_moe_fused", "quantize")
    if _os.path.isdir(_ref_pkg) and _ref_pkg not in __path__:
        __path__.append(_ref_pkg)
