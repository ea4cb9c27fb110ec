"""Builds libmoe_b200.so (sm_100a) from csrc/ with nvcc, in-tree.

Usage:  python build.py [--force]
The shared library is written next to the Python package (qwen3_moe_fused/libmoe_b200.so)
so that it is found by `qwen3_moe_fused._lib` without any install step.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "qwen3_moe_fused" / "libmoe_b200.so"
OBJ_DIR = HERE / "build"
SOURCES = ["sort.cu", "simt_gemm.cu", "elementwise.cu", "router.cu", "ep.cu", "tc_gemm.cu", "gemm_api.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libmoe_b200.so cannot be built")
    return exe


def _stale() -> bool:
    if not OUT.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + [HERE.parent / "include" / "moe_b200.h"])
    return newest > OUT.stat().st_mtime


def _compile(src: str) -> Path:
    obj = OBJ_DIR / (src + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return obj


def build_library(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return OUT
    OBJ_DIR.mkdir(exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(_compile, SOURCES))
    cmd = [_nvcc(), "-shared", "-o", str(OUT), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(f"built {OUT}")
    return OUT


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose=True)
