"""Shared helpers for the GPU parity tests."""
import numpy as np
import torch

from oracle import moe_oracle as O

DT = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
# max |got - ref| / max |ref| bars: bf16/fp16 1e-2 (the path's stated tolerance);
# fp32 runs on CUDA cores in full precision
TOL = {"f32": 2e-5, "bf16": 1e-2, "f16": 1e-2}


def rounded(a: np.ndarray, dtype: str) -> np.ndarray:
    return O.round_to(np.asarray(a, np.float32), dtype)


def to_dev(a: np.ndarray, dtype: str, device) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=DT[dtype])


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def random_m_sizes(rng: np.random.Generator, M: int, E: int, empty_frac: float = 0.0) -> np.ndarray:
    p = rng.random(E) + 0.05
    if empty_frac > 0:
        p[rng.random(E) < empty_frac] = 0.0
        if p.sum() == 0:
            p[0] = 1.0
    p /= p.sum()
    return rng.multinomial(M, p).astype(np.int32)


def assert_close(got, ref, dtype: str, what: str = "", scale: float = 1.0):
    err = O.rel_err(got, ref)
    assert err <= TOL[dtype] * scale, f"{what}: rel err {err:.3e} > {TOL[dtype] * scale:.1e}"
    return err
