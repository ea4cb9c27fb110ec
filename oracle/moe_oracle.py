"""CPU restatement (numpy) of the `moe_fused_linear` hot path of transformers-qwen3-moe-fused.

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA kernels are compared with;
it is imported by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark, and by nothing else.  No product code path may call into it.

Parity status: the sort / permutation functions, the three grouped-GEMM definitions, the
plain SiLU-mul and the block composition are pinned against outputs of the reference's
own Python code (fixtures under tests/golden/, produced by tests/golden/make_golden.py);
SiLU-mul's rounding points, the three grouped GEMMs and the 4-bit decode inside the forward
are pinned against the reference's Triton kernels executed under Triton's CPU interpreter
(tests/golden/make_golden_triton.py, float16 / float32).
The NF4 code table and quantiser come from bitsandbytes, which is neither part of the
reference tree nor installed: "parity unpinned" for those two (the table is rebuilt from its
published construction and checked against the published constants).

Every function cites the reference lines it follows (paths inside the reference project).
Floating-point inputs are taken as float32 arrays holding values already rounded to the
storage dtype under test; `round_to` applies the storage rounding where the reference does.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------
# storage-dtype rounding
# ----------------------------------------------------------------------------------

def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even) -> float32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(x)
    out[nan] = np.nan
    return out


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "bf16":
        return round_bf16(x)
    if dtype == "f16":
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
    raise ValueError(dtype)


# ----------------------------------------------------------------------------------
# sort / permutation  (qwen3_moe_fused/kernels/indexing.py)
# ----------------------------------------------------------------------------------

def get_expert_counts(s: np.ndarray, E: int) -> np.ndarray:
    """indexing.py:18-23: counts[e] = #{b : s[b] == e}, int32."""
    return np.bincount(np.asarray(s, dtype=np.int64), minlength=E)[:E].astype(np.int32)


def get_expert_counts_and_idx(s: np.ndarray, E: int):
    """indexing.py:48-65.  idx[b] = offsets[s[b]] + (rank of b among the rows of expert s[b],
    in original order); inv_idx[idx[b]] = b.  Returns (counts, inv_idx, idx), int32."""
    s = np.asarray(s, dtype=np.int64)
    counts = get_expert_counts(s, E)
    offsets = np.cumsum(counts) - counts
    idx = np.empty(s.shape[0], dtype=np.int32)
    seen = np.zeros(E, dtype=np.int64)
    # literal restatement; the vectorised identity below is asserted in the tests
    for b in range(s.shape[0]):
        e = s[b]
        idx[b] = offsets[e] + seen[e]
        seen[e] += 1
    inv_idx = np.empty_like(idx)
    inv_idx[idx] = np.arange(s.shape[0], dtype=np.int32)
    return counts, inv_idx, idx


def get_expert_counts_and_idx_fast(s: np.ndarray, E: int):
    """Same result through a stable argsort (used at sizes where the loop above is slow)."""
    s = np.asarray(s, dtype=np.int64)
    counts = get_expert_counts(s, E)
    inv_idx = np.argsort(s, kind="stable").astype(np.int32)
    idx = np.empty_like(inv_idx)
    idx[inv_idx] = np.arange(s.shape[0], dtype=np.int32)
    return counts, inv_idx, idx


def sort_experts(s: np.ndarray, E: int):
    """indexing.py:27-45: (s_sorted, inv_idx, idx)."""
    counts, inv_idx, idx = get_expert_counts_and_idx_fast(s, E)
    s_sorted = np.repeat(np.arange(E, dtype=np.int32), counts)
    return s_sorted, inv_idx, idx


def get_batch_begins_ends(s: np.ndarray, E: int) -> np.ndarray:
    """indexing.py:7-14: [e,0] = #{s < e}, [e,1] = #{s <= e}."""
    s = np.asarray(s, dtype=np.int64)
    ar = np.arange(E)
    begins = (ar[:, None] > s[None, :]).sum(axis=1)
    ends = (ar[:, None] >= s[None, :]).sum(axis=1)
    return np.stack([begins, ends], axis=1).astype(np.int32)


def experts_from_m_sizes(m_sizes: np.ndarray) -> np.ndarray:
    return np.repeat(np.arange(len(m_sizes)), np.asarray(m_sizes, dtype=np.int64))


# ----------------------------------------------------------------------------------
# moe_fused_linear and its gradients  (qwen3_moe_fused/functional.py:7-61)
# Accumulation in float32 over float32 copies of the (already rounded) inputs, one
# rounding of the result to the storage dtype: what the kernels do (fp32 accumulator,
# cast on store: grouped_gemm/forward.py:82,94).
# ----------------------------------------------------------------------------------

def moe_fused_linear_fwd_rowloop(x, w, selected_experts):
    """functional.py:7-32, literal: one mat-vec per row."""
    out = np.empty((x.shape[0], w.shape[1]), dtype=np.float32)
    for b in range(x.shape[0]):
        out[b] = w[selected_experts[b]] @ x[b]
    return out


def moe_fused_linear_bwd_input_rowloop(dy, w, selected_experts):
    """functional.py:36-47."""
    out = np.empty((dy.shape[0], w.shape[2]), dtype=np.float32)
    for b in range(dy.shape[0]):
        out[b] = dy[b] @ w[selected_experts[b]]
    return out


def moe_fused_linear_bwd_weight_rowloop(dy, x, E, selected_experts):
    """functional.py:51-61."""
    out = np.zeros((E, dy.shape[1], x.shape[1]), dtype=np.float32)
    for b in range(dy.shape[0]):
        out[selected_experts[b]] += dy[b][:, None] * x[b][None, :]
    return out


def _groups(m_sizes):
    m = np.asarray(m_sizes, dtype=np.int64)
    ends = np.cumsum(m)
    return [(int(e), int(end - n), int(end)) for e, (n, end) in enumerate(zip(m, ends)) if n > 0]


def grouped_gemm_fwd(x, w, m_sizes, dtype="f32"):
    """y[m,n] = sum_k w[e(m),n,k] x[m,k]  (grouped_gemm/forward.py:22-103), per expert."""
    x = np.asarray(x, np.float32); w = np.asarray(w, np.float32)
    y = np.zeros((x.shape[0], w.shape[1]), dtype=np.float32)
    for e, a, b in _groups(m_sizes):
        y[a:b] = x[a:b] @ w[e].T
    return round_to(y, dtype)


def grouped_gemm_dx(dy, w, m_sizes, dtype="f32"):
    """y[m,n] = sum_k w[e(m),k,n] dy[m,k]  (grouped_gemm/forward_transposed.py:23-104)."""
    dy = np.asarray(dy, np.float32); w = np.asarray(w, np.float32)
    y = np.zeros((dy.shape[0], w.shape[2]), dtype=np.float32)
    for e, a, b in _groups(m_sizes):
        y[a:b] = dy[a:b] @ w[e]
    return round_to(y, dtype)


def grouped_gemm_dw(x, dy, m_sizes, dtype="f32"):
    """w[e,n,k] = sum_{m in e} dy[m,n] x[m,k]; empty experts stay zero
    (grouped_gemm/backward_dw.py:21-89, :110)."""
    x = np.asarray(x, np.float32); dy = np.asarray(dy, np.float32)
    w = np.zeros((len(m_sizes), dy.shape[1], x.shape[1]), dtype=np.float32)
    for e, a, b in _groups(m_sizes):
        w[e] = dy[a:b].T @ x[a:b]
    return round_to(w, dtype)


# ----------------------------------------------------------------------------------
# NF4  (decode: qwen3_moe_fused/grouped_gemm/forward_4bit.py:99-104; layout :142-153,173-176)
# ----------------------------------------------------------------------------------

def nf4_code() -> np.ndarray:
    """16 NormalFloat-4 levels from their published construction: equal-area quantiles of
    N(0,1), 8 on the positive side and 7 on the negative side of an exact zero, tail offset
    0.9677083, normalised to [-1, 1].  PARITY UNPINNED against bitsandbytes' own table
    (not available here); the kernels take the table as an input, as the reference does
    (forward_4bit.py:146-147)."""
    from statistics import NormalDist

    nd = NormalDist()
    offset = 0.9677083
    pos = [nd.inv_cdf(p) for p in np.linspace(offset, 0.5, 9)[:-1]]
    neg = [-nd.inv_cdf(p) for p in np.linspace(offset, 0.5, 8)[:-1]]
    vals = np.sort(np.array(pos + [0.0] + neg, dtype=np.float64))
    return (vals / np.abs(vals).max()).astype(np.float32)


def nf4_quantize(w: np.ndarray, blocksize: int, code: np.ndarray | None = None):
    """Blockwise absmax quantiser (PARITY UNPINNED, see module header): nearest level of
    value/absmax.  Returns (packed uint8 [numel/2], absmax float32 [numel/blocksize])."""
    code = nf4_code() if code is None else code
    flat = np.asarray(w, np.float32).reshape(-1, blocksize)
    absmax = np.abs(flat).max(axis=1).astype(np.float32)
    scaled = flat / np.maximum(absmax, np.finfo(np.float32).tiny)[:, None]
    mids = (code[1:] + code[:-1]) / 2
    idx = np.searchsorted(mids, scaled.reshape(-1), side="left").astype(np.uint8)
    packed = (idx[0::2] << 4) | idx[1::2]
    return packed, absmax


def nf4_dequantize(packed: np.ndarray, absmax: np.ndarray, code: np.ndarray, blocksize: int, shape, dtype="f32"):
    """forward_4bit.py:99-104: byte -> (byte // 16, byte % 16) interleaved (high nibble is
    the even element), table lookup, times absmax[flat_index // blocksize], cast to dtype."""
    packed = np.asarray(packed, np.uint8).reshape(-1)
    idx = np.empty(packed.size * 2, dtype=np.int64)
    idx[0::2] = packed // 16
    idx[1::2] = packed % 16
    vals = code.astype(np.float32)[idx] * np.repeat(np.asarray(absmax, np.float32), blocksize)
    return round_to(vals.reshape(shape), dtype)


def absmax_unnest(q: np.ndarray, code2: np.ndarray, absmax2: np.ndarray, blocksize2: int, offset: float) -> np.ndarray:
    """forward_4bit.py:149-153: a double-quantised absmax back to fp32: table lookup of the byte,
    times the second-level absmax of its block, plus the offset; each step rounded to fp32."""
    vals = code2.astype(np.float32)[np.asarray(q, np.uint8)] * np.repeat(np.asarray(absmax2, np.float32), blocksize2)
    return (vals.astype(np.float32) + np.float32(offset)).astype(np.float32)


# ----------------------------------------------------------------------------------
# SiLU-mul  (qwen3_moe_fused/kernels/silu_mul.py:23-111; plain path
# qwen3_moe_fused/modular_qwen3_moe_fused.py:108)
# ----------------------------------------------------------------------------------

def _sigmoid(x):
    x = np.asarray(x, np.float32)
    return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)


def silu_mul_fwd(e, g, dtype="f32"):
    """silu_mul.py:34-39: f = dtype(e * sigmoid(e)) in fp32; h = f * g in dtype."""
    e = np.asarray(e, np.float32); g = np.asarray(g, np.float32)
    f = round_to(e * _sigmoid(e), dtype)
    return round_to(f * g, dtype)


def silu_mul_bwd(dh, e, g, dtype="f32"):
    """silu_mul.py:62-73 (and :97-111 for the in-place form): returns (h, de, dg)."""
    dh = np.asarray(dh, np.float32); e = np.asarray(e, np.float32); g = np.asarray(g, np.float32)
    se = _sigmoid(e)
    ese = (e * se).astype(np.float32)
    f = round_to(ese, dtype)
    h = round_to(f * g, dtype)
    df = round_to(dh * g, dtype)
    dg = round_to(f * dh, dtype)
    de = round_to(df * se * (np.float32(1.0) + e - ese), dtype)
    return h, de, dg


# ----------------------------------------------------------------------------------
# router, expand/gather, combine  (qwen3_moe_fused/modular_qwen3_moe_fused.py:85-115)
# ----------------------------------------------------------------------------------

def router_softmax_topk(logits, k, norm_topk_prob=True, dtype="f32"):
    """modular_qwen3_moe_fused.py:87-93: softmax in fp32, top-k (values descending),
    optional division by the winners' sum, cast.  Tie rule (the reference leaves it to
    torch.topk, which does not define one): equal probabilities -> lower expert id first.
    Returns (weights (T,k) float32 holding dtype-rounded values, experts (T,k) int64)."""
    z = np.asarray(logits, np.float32)
    z = z - z.max(axis=1, keepdims=True)
    p = np.exp(z).astype(np.float32)
    p = (p / p.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    top = np.take_along_axis(p, order, axis=1)
    if norm_topk_prob:
        top = top / top.sum(axis=1, keepdims=True, dtype=np.float32)
    return round_to(top.astype(np.float32), dtype), order.astype(np.int64)


def gather_rows(hidden, sort_idx, k):
    """modular_qwen3_moe_fused.py:95-103: expand every token k times, then gather."""
    return np.asarray(hidden)[np.asarray(sort_idx, np.int64) // k]


def combine(y, inv_sort_idx, weights, dtype="f32"):
    """modular_qwen3_moe_fused.py:112-115: y[inv_sort_idx] viewed (T,k,H), einsum with the
    routing weights (fp32 accumulation, one rounding)."""
    T, k = weights.shape
    ys = np.asarray(y, np.float32)[np.asarray(inv_sort_idx, np.int64)].reshape(T, k, -1)
    out = np.einsum("tkh,tk->th", ys, np.asarray(weights, np.float32)).astype(np.float32)
    return round_to(out, dtype)


def moe_block_forward(hidden, gate_w, gate_proj, up_proj, down_proj, k, norm_topk_prob=True, dtype="f32"):
    """modular_qwen3_moe_fused.py:79-118 end to end (storage rounding after every op)."""
    T, H = hidden.shape
    E = gate_w.shape[0]
    logits = round_to(np.asarray(hidden, np.float32) @ np.asarray(gate_w, np.float32).T, dtype)
    weights, experts = router_softmax_topk(logits, k, norm_topk_prob, dtype)
    m_sizes, sort_idx, inv_sort_idx = get_expert_counts_and_idx_fast(experts.reshape(-1), E)
    xs = gather_rows(hidden, sort_idx, k)
    gate_h = grouped_gemm_fwd(xs, gate_proj, m_sizes, dtype)
    up_h = grouped_gemm_fwd(xs, up_proj, m_sizes, dtype)
    h = silu_mul_fwd(gate_h, up_h, dtype)
    y = grouped_gemm_fwd(h, down_proj, m_sizes, dtype)
    return combine(y, inv_sort_idx, weights, dtype), logits


# ----------------------------------------------------------------------------------
# error metric  (test_quantize.py:17-28 of the reference)
# ----------------------------------------------------------------------------------

def rel_err(got, ref) -> float:
    """max |got - ref| / max |ref|: the figure the 1e-2 output/gradient bar is stated in."""
    got = np.asarray(got, np.float64); ref = np.asarray(ref, np.float64)
    denom = max(float(np.abs(ref).max()), 1e-30)
    return float(np.abs(got - ref).max() / denom)
