"""Timed CPU restatements of the reference's torch implementation of `moe_fused_linear`.

TEST / BENCHMARK INFRASTRUCTURE ONLY (see oracle/moe_oracle.py).  The reference's CPU
path is a Python loop with one torch mat-vec (or outer product) per row
(qwen3_moe_fused/functional.py:7-61); `rowloop_*` below perform the same sequence of torch
calls so that their timing stands for the reference's on the same host cores.
`vectorised_*` is the fairer CPU figure: one GEMM per expert over the sorted rows.
"""
from __future__ import annotations

import time

import torch


def rowloop_fwd(x: torch.Tensor, w: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
    """functional.py:7-32."""
    out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype)
    for b in range(x.shape[0]):
        out[b, :] = w[experts[b], :, :] @ x[b, :]
    return out


def rowloop_bwd_input(dy: torch.Tensor, w: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
    """functional.py:36-47."""
    out = torch.empty(dy.shape[0], w.shape[2], dtype=dy.dtype)
    for b in range(dy.shape[0]):
        out[b, :] = dy[b, :] @ w[experts[b], :, :]
    return out


def rowloop_bwd_weight(dy: torch.Tensor, x: torch.Tensor, w_like: torch.Tensor, experts: torch.Tensor) -> torch.Tensor:
    """functional.py:51-61."""
    out = torch.zeros_like(w_like)
    for b in range(dy.shape[0]):
        out[experts[b], :, :] += dy[b, :, None] * x[b, None, :]
    return out


def vectorised_fwd(x: torch.Tensor, w: torch.Tensor, m_sizes: torch.Tensor) -> torch.Tensor:
    out = torch.empty(x.shape[0], w.shape[1], dtype=x.dtype)
    row = 0
    for e, n in enumerate(m_sizes.tolist()):
        if n:
            out[row:row + n] = x[row:row + n] @ w[e].T
            row += n
    return out


def vectorised_bwd_input(dy: torch.Tensor, w: torch.Tensor, m_sizes: torch.Tensor) -> torch.Tensor:
    out = torch.empty(dy.shape[0], w.shape[2], dtype=dy.dtype)
    row = 0
    for e, n in enumerate(m_sizes.tolist()):
        if n:
            out[row:row + n] = dy[row:row + n] @ w[e]
            row += n
    return out


def vectorised_bwd_weight(dy: torch.Tensor, x: torch.Tensor, w_like: torch.Tensor, m_sizes: torch.Tensor) -> torch.Tensor:
    out = torch.zeros_like(w_like)
    row = 0
    for e, n in enumerate(m_sizes.tolist()):
        if n:
            out[e] = dy[row:row + n].T @ x[row:row + n]
            row += n
    return out


def time_call(fn, *args, repeats: int = 1) -> float:
    """Best wall time in seconds over `repeats` calls."""
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn(*args)
        best = min(best, time.perf_counter() - t0)
    return best
