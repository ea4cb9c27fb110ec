"""Router and token movement kernels of the sparse MoE block.

These replace sequences of ATen calls inside the reference block forward
(qwen3_moe_fused/modular_qwen3_moe_fused.py:87-115): softmax -> topk -> renormalise ->
cast; expand -> gather; un-permute -> weighted sum.
"""
import torch

from .. import _lib


@torch.no_grad()
def softmax_topk(router_logits: torch.Tensor, k: int, norm_topk_prob: bool, out_dtype: torch.dtype):
    """(weights (T,k) out_dtype, experts (T,k) int64); winners ordered by probability
    descending, equal probabilities by ascending expert id."""
    assert router_logits.is_cuda and router_logits.ndim == 2 and router_logits.is_contiguous()
    T, E = router_logits.shape
    weights = torch.empty((T, k), device=router_logits.device, dtype=out_dtype)
    experts = torch.empty((T, k), device=router_logits.device, dtype=torch.int64)
    with torch.cuda.device(router_logits.device):
        status = _lib.load().moe_router_softmax_topk(
            _lib.ptr(router_logits), _lib.float_code(router_logits.dtype), T, E, k, int(norm_topk_prob),
            _lib.ptr(weights), _lib.float_code(out_dtype), _lib.ptr(experts), _lib.stream_ptr(router_logits.device),
        )
    _lib.check(status, "moe_router_softmax_topk")
    return weights, experts


class SoftmaxTopk(torch.autograd.Function):
    """Differentiable wrapper: the forward is one kernel; the backward recomputes the fp32
    softmax of the (T, E) logits and differentiates gather -> renormalise -> cast, which is
    what autograd does for the reference's sequence of ATen calls."""

    @staticmethod
    def forward(ctx, router_logits, k, norm_topk_prob, out_dtype):
        weights, experts = softmax_topk(router_logits, k, norm_topk_prob, out_dtype)
        ctx.save_for_backward(router_logits, experts)
        ctx.norm = norm_topk_prob
        ctx.out_dtype = out_dtype
        ctx.mark_non_differentiable(experts)
        return weights, experts

    @staticmethod
    def backward(ctx, dweights, _dexperts):
        logits, experts = ctx.saved_tensors
        with torch.enable_grad():
            lg = logits.detach().requires_grad_()
            sel = torch.softmax(lg, dim=1, dtype=torch.float32).gather(1, experts)
            if ctx.norm:
                sel = sel / sel.sum(dim=-1, keepdim=True)
            (grad,) = torch.autograd.grad(sel.to(ctx.out_dtype), lg, dweights)
        return grad, None, None, None


def softmax_topk_autograd(router_logits, k, norm_topk_prob, out_dtype):
    return SoftmaxTopk.apply(router_logits, k, norm_topk_prob, out_dtype)


def _gather_rows(hidden: torch.Tensor, sort_idx: torch.Tensor, k: int) -> torch.Tensor:
    assert hidden.is_cuda and hidden.ndim == 2 and hidden.is_contiguous()
    assert sort_idx.dtype == torch.int32 and sort_idx.is_contiguous()
    rows = sort_idx.numel()
    out = torch.empty((rows, hidden.shape[1]), device=hidden.device, dtype=hidden.dtype)
    with torch.cuda.device(hidden.device):
        status = _lib.load().moe_gather_rows(
            _lib.ptr(hidden), _lib.ptr(sort_idx), k, _lib.ptr(out), rows, hidden.shape[1],
            _lib.float_code(hidden.dtype), _lib.stream_ptr(hidden.device),
        )
    _lib.check(status, "moe_gather_rows")
    return out


def _expand_rows(hidden: torch.Tensor, inv_sort_idx: torch.Tensor, k: int) -> torch.Tensor:
    """The result of _gather_rows computed through the inverse index (out[inv_sort_idx[t*k+j]] =
    hidden[t]): every token row is read once instead of k times."""
    assert hidden.is_cuda and hidden.ndim == 2 and hidden.is_contiguous()
    assert inv_sort_idx.dtype == torch.int32 and inv_sort_idx.is_contiguous()
    tokens = hidden.shape[0]
    assert inv_sort_idx.numel() == tokens * k
    out = torch.empty((tokens * k, hidden.shape[1]), device=hidden.device, dtype=hidden.dtype)
    with torch.cuda.device(hidden.device):
        status = _lib.load().moe_expand_rows(
            _lib.ptr(hidden), _lib.ptr(inv_sort_idx), k, _lib.ptr(out), tokens, hidden.shape[1],
            _lib.float_code(hidden.dtype), _lib.stream_ptr(hidden.device),
        )
    _lib.check(status, "moe_expand_rows")
    return out


def _combine(y: torch.Tensor, inv_sort_idx: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    assert y.is_cuda and y.ndim == 2 and y.is_contiguous()
    assert inv_sort_idx.dtype == torch.int32 and inv_sort_idx.is_contiguous()
    assert weights.is_contiguous() and weights.dtype == y.dtype
    T, k = weights.shape
    out = torch.empty((T, y.shape[1]), device=y.device, dtype=y.dtype)
    with torch.cuda.device(y.device):
        status = _lib.load().moe_combine(
            _lib.ptr(y), _lib.ptr(inv_sort_idx), _lib.ptr(weights), _lib.ptr(out), T, k, y.shape[1],
            _lib.float_code(y.dtype), _lib.stream_ptr(y.device),
        )
    _lib.check(status, "moe_combine")
    return out


class GatherRows(torch.autograd.Function):
    """out[j] = hidden[sort_idx[j] // k].  Backward: each token sums the gradients of its k copies."""

    @staticmethod
    def forward(ctx, hidden, sort_idx, inv_sort_idx, k):
        ctx.save_for_backward(inv_sort_idx)
        ctx.k = k
        if inv_sort_idx.numel() == hidden.shape[0] * k:
            return _expand_rows(hidden, inv_sort_idx, k)  # same rows, each token read once
        return _gather_rows(hidden, sort_idx, k)

    @staticmethod
    def backward(ctx, dout):
        (inv_sort_idx,) = ctx.saved_tensors
        k = ctx.k
        T = inv_sort_idx.numel() // k
        ones = torch.ones((T, k), device=dout.device, dtype=dout.dtype)
        return _combine(dout.contiguous(), inv_sort_idx, ones), None, None, None


class Combine(torch.autograd.Function):
    """out[t] = sum_j weights[t, j] * y[inv_sort_idx[t*k + j]]."""

    @staticmethod
    def forward(ctx, y, sort_idx, inv_sort_idx, weights):
        ctx.save_for_backward(y, sort_idx, inv_sort_idx, weights)
        return _combine(y, inv_sort_idx, weights)

    @staticmethod
    def backward(ctx, dout):
        y, sort_idx, inv_sort_idx, weights = ctx.saved_tensors
        T, k = weights.shape
        dout = dout.contiguous()
        dy = dw = None
        if ctx.needs_input_grad[0]:
            # dy[j] = weights.flat[sort_idx[j]] * dout[sort_idx[j] // k]
            dy = _expand_rows(dout, inv_sort_idx, k) * weights.reshape(-1)[sort_idx.long()].unsqueeze(1)
        if ctx.needs_input_grad[3]:
            # dweights[t, j] = <dout[t], y[inv_sort_idx[t*k+j]]>
            dw = torch.einsum("tkh,th->tk", y[inv_sort_idx.long()].view(T, k, -1).float(), dout.float()).to(weights.dtype)
        return dy, None, None, dw


def gather_rows(hidden, sort_idx, inv_sort_idx, k):
    return GatherRows.apply(hidden, sort_idx, inv_sort_idx, k)


def combine(y, sort_idx, inv_sort_idx, weights):
    return Combine.apply(y, sort_idx, inv_sort_idx, weights)
