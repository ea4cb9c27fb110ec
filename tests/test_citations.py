"""Every `path.py:line` citation of the reference in the header, the oracle and the package points at lines that
exist in a reference checkout (skipped without one; no GPU)."""
import os
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("QWEN3_MOE_FUSED_REFERENCE_CHECKOUT", "/root/reference"))
CITATION = re.compile(r"((?:qwen3_moe_fused/)?(?:[A-Za-z_0-9]+/)*[A-Za-z_0-9]+\.py):(\d+)(?:-(\d+))?")


def _cited_files():
    files = list((ROOT / "include").glob("*.h")) + list((ROOT / "oracle").glob("*.py"))
    pkg = ROOT / "transformers-qwen3-moe-fused_b200"
    files += [p for p in pkg.rglob("*") if p.suffix in (".py", ".cu", ".cuh", ".h")]
    return files


def _resolve(rel: str):
    """A cited path may be written from the reference's root or from inside its package."""
    for base in (REFERENCE, REFERENCE / "qwen3_moe_fused", REFERENCE / "qwen3_moe_fused" / "grouped_gemm",
                 REFERENCE / "qwen3_moe_fused" / "kernels", REFERENCE / "qwen3_moe_fused" / "quantize"):
        if (base / rel).is_file():
            return base / rel
    return None


@pytest.mark.skipif(not (REFERENCE / "qwen3_moe_fused" / "functional.py").exists(), reason="no reference checkout on this machine")
def test_cited_reference_lines_exist():
    lengths, bad, seen = {}, [], 0
    for f in _cited_files():
        for m in CITATION.finditer(f.read_text(errors="ignore")):
            rel, a, b = m.group(1), int(m.group(2)), int(m.group(3) or m.group(2))
            target = _resolve(rel)
            if target is None:
                continue  # a file of this repository (bench.py:…, tests/…), not of the reference
            seen += 1
            n = lengths.setdefault(target, len(target.read_text().splitlines()))
            if not (1 <= a <= b <= n):
                bad.append(f"{f.relative_to(ROOT)}: {m.group(0)} (file has {n} lines)")
    assert seen > 50, "the citation pattern no longer matches the sources"
    assert not bad, "\n".join(bad)
