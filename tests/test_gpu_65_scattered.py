"""The peer-memory building blocks on one GPU: the row push to per-expert addresses and the
scattered forward / dX (several groups per weight slice, one output address per group).  The
"peer" buffers here are ordinary local buffers; on several GPUs only the addresses differ."""
import numpy as np
import pytest
import torch

from tests.helpers import random_m_sizes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("E,M,W", [(8, 1000, 256), (128, 20000, 2048), (5, 7, 8), (16, 513, 776)])
def test_push_rows(dev, E, M, W):
    from qwen3_moe_fused.parallel_ep import push_rows

    rng = np.random.default_rng(E * 7 + M)
    m = random_m_sizes(rng, M, E, empty_frac=0.2)
    rows = torch.randn(M, W, device=dev).to(torch.bfloat16)
    # every expert gets a slot of its own in one of two buffers, in a shuffled order; one expert's
    # slot is shorter than its rows (the rest is dropped and counted), another expert is left out
    # of the push altogether (negative limit: not written, not counted)
    order = rng.permutation(E)
    limit = m.copy()
    big = int(np.argmax(m))
    limit[big] = m[big] // 2
    others = [e for e in np.argsort(-m) if e != big and m[e] > 0]
    skip = int(others[0]) if others else -1
    if skip >= 0:
        limit[skip] = -1
    bufs = [torch.full((M + 8, W), -1.0, device=dev, dtype=torch.bfloat16) for _ in range(2)]
    ptrs = np.zeros(E, np.int64)
    slot = {}
    fill = [0, 0]
    for e in order:
        b = int(e) % 2
        slot[int(e)] = (b, fill[b])
        ptrs[e] = bufs[b].data_ptr() + fill[b] * W * 2
        fill[b] += max(int(limit[e]), 0)
    dropped = torch.zeros(1, dtype=torch.int32, device=dev)
    push_rows(rows, torch.from_numpy(m).to(dev), torch.from_numpy(ptrs).to(dev), torch.from_numpy(limit.astype(np.int32)).to(dev),
              first_expert=(E * 2) // 3, dropped=dropped)
    torch.cuda.synchronize()
    begins = np.concatenate([[0], np.cumsum(m)])
    for e in range(E):
        b, at = slot[e]
        n = max(int(limit[e]), 0)
        assert torch.equal(bufs[b][at:at + n], rows[begins[e]:begins[e] + n]), f"expert {e}"
    for b in range(2):
        assert bool((bufs[b][fill[b]:] == -1.0).all()), "rows past the limits were written"
    assert int(dropped) == int(m[big] - limit[big]), "every row that did not fit is counted, skipped experts are not"


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("E_w,world,M,N,K", [(4, 2, 3000, 384, 256), (8, 4, 9000, 768, 512), (3, 1, 700, 200, 72)])
def test_scattered_gemm(dev, transposed, dtype, E_w, world, M, N, K):
    from qwen3_moe_fused.grouped_gemm.forward import grouped_gemm_forward
    from qwen3_moe_fused.grouped_gemm.forward_transposed import grouped_gemm_forward_transposed
    from qwen3_moe_fused.parallel_ep import scattered_grouped_gemm

    rng = np.random.default_rng(M + N)
    G = E_w * world
    sizes = random_m_sizes(rng, M, G, empty_frac=0.15)
    x = torch.randn(M, K, device=dev).to(dtype)
    w = (torch.randn(E_w, N, K, device=dev) * 0.05).to(dtype)
    if transposed:
        w = w.transpose(1, 2).contiguous()  # (E_w, K, N): dX reads the weight (E, out=K, in=N)
    widx = torch.arange(G, device=dev, dtype=torch.int32) // world
    # reference: the plain grouped GEMM over per-group copies of the weight slices
    w_rep = w[widx.long()].contiguous()
    fn = grouped_gemm_forward_transposed if transposed else grouped_gemm_forward
    ref = fn(x, w_rep, torch.from_numpy(sizes).to(dev))
    # group g's results go to buffer g % world, groups packed there in reverse order
    bufs = [torch.full((M + 4, N), 7.0, device=dev, dtype=dtype) for _ in range(world)]
    ptrs = np.zeros(G, np.int64)
    where = {}
    fill = [0] * world
    for g in reversed(range(G)):
        b = g % world
        where[g] = (b, fill[b])
        ptrs[g] = bufs[b].data_ptr() + fill[b] * N * 2
        fill[b] += int(sizes[g])
    scattered_grouped_gemm(x, w, torch.from_numpy(sizes).to(dev), widx, torch.from_numpy(ptrs).to(dev), bufs[0], transposed)
    torch.cuda.synchronize()
    begins = np.concatenate([[0], np.cumsum(sizes)])
    for g in range(G):
        b, at = where[g]
        n = int(sizes[g])
        assert torch.equal(bufs[b][at:at + n], ref[begins[g]:begins[g] + n]), f"group {g}"
    for b in range(world):
        assert bool((bufs[b][fill[b]:] == 7.0).all()), "rows outside the groups were written"


def test_push_rows_expands_tokens(dev):
    """With the sort's gather index the push reads token rows and delivers the expanded rows."""
    from oracle import moe_oracle as O
    from qwen3_moe_fused.parallel_ep import push_rows

    rng = np.random.default_rng(9)
    T, k, E, W = 300, 4, 12, 256
    sel = rng.integers(0, E, T * k)
    counts, sort_idx, _ = O.get_expert_counts_and_idx_fast(sel, E)
    tokens = torch.randn(T, W, device=dev).to(torch.bfloat16)
    out = torch.zeros(T * k, W, device=dev, dtype=torch.bfloat16)
    begins = np.concatenate([[0], np.cumsum(counts)])[:-1]
    ptrs = torch.from_numpy(out.data_ptr() + begins.astype(np.int64) * W * 2).to(dev)
    push_rows(tokens, torch.from_numpy(counts).to(dev), ptrs, None, src_index=torch.from_numpy(sort_idx).to(dev), src_div=k)
    torch.cuda.synchronize()
    assert torch.equal(out, tokens[torch.from_numpy(sort_idx).to(dev).long() // k])


def test_scattered_rejects_thin(dev):
    from qwen3_moe_fused import _lib
    from qwen3_moe_fused.parallel_ep import scattered_grouped_gemm

    x = torch.randn(64, 64, device=dev).to(torch.bfloat16)
    w = torch.randn(2, 64, 64, device=dev).to(torch.bfloat16)
    out = torch.empty(64, 64, device=dev, dtype=torch.bfloat16)
    ptrs = torch.tensor([out.data_ptr(), out.data_ptr() + 32 * 128], device=dev)
    with pytest.raises(_lib.MoeB200Error):
        scattered_grouped_gemm(x, w, torch.tensor([32, 32], device=dev, dtype=torch.int32), None, ptrs, out)


@pytest.mark.parametrize("world,E,rng_", [(2, 16, None), (4, 128, None), (8, 128, (4, 9)), (4, 32, (0, 3)), (1, 8, None),
                                          (8, 1024, None), (16, 1024, None)])  # the last two need more than 48 KB of shared memory
def test_plan_kernel_matches_tensor_plan(dev, world, E, rng_):
    """`moe_ep_plan` (one launch) against the same plan computed with tensor operations on the host."""
    from qwen3_moe_fused.parallel_ep import PeerPlan

    g = torch.Generator().manual_seed(world * 1000 + E)
    counts = torch.randint(0, 700, (world, E), generator=g, dtype=torch.int32)
    counts[counts % 7 == 0] = 0
    for rank in range(world):
        a = PeerPlan.from_counts(counts.to(dev), world, rank, rng_)
        b = PeerPlan.from_counts(counts, world, rank, rng_)
        for f in ("m_sizes", "dst_rank", "send_row", "group_sizes", "weight_index", "group_src", "return_row", "local_m_sizes"):
            assert torch.equal(getattr(a, f).cpu().long(), getattr(b, f).long()), f"{f} rank {rank}"
        assert int(a.recv_rows) == int(b.recv_rows) and a.expert_lo == b.expert_lo and a.e_local == b.e_local
        if rng_ is None:
            assert a.send_mask is None and b.send_mask is None
        else:
            assert torch.equal(a.send_mask.cpu(), b.send_mask)


class _LocalChannel:
    """Stand-in for a PeerChannel on one GPU: the buffers of all "ranks" are local tensors."""

    def __init__(self, bufs):
        self.bufs = bufs
        self.ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=bufs[0].device)
        self.capacity_rows = bufs[0].shape[0]
        self.row_bytes = bufs[0].shape[1] * bufs[0].element_size()


@pytest.mark.parametrize("world,E,T,k,W", [(2, 16, 500, 4, 256), (4, 128, 3000, 8, 512), (8, 128, 1024, 8, 2048)])
def test_token_deduplicated_dispatch(dev, world, E, T, k, W):
    """All ranks of an expert-parallel group emulated on one GPU: every token row is stored once per
    destination rank, every expanded row sends the index of its token there, and the owner's expansion
    reproduces, bit for bit, the expert-major rows that the one-row-per-(token, expert) push delivers."""
    from oracle import moe_oracle as O
    from qwen3_moe_fused.parallel_ep import (PeerPlan, expand_received, peer_push, peer_push_index, peer_push_tokens, slot_bases,
                                             token_positions)

    rng = np.random.default_rng(world * 100 + T)
    e_all = E // world
    sel = [np.stack([rng.choice(E, k, replace=False) for _ in range(T)]) for _ in range(world)]
    tokens = [torch.randn(T, W, device=dev).to(torch.bfloat16) for _ in range(world)]
    sorts = [O.get_expert_counts_and_idx_fast(sel[s].reshape(-1), E) for s in range(world)]
    counts_all = torch.from_numpy(np.stack([c for c, _, _ in sorts])).to(dev)
    poss, n_tok = zip(*[token_positions(torch.from_numpy(sel[s]).to(dev), E, world) for s in range(world)])
    tokens_all = torch.stack(n_tok)
    # the kernel's bookkeeping equals the tensor-op definition
    for s in range(world):
        ref_pos, ref_n = token_positions(torch.from_numpy(sel[s]), E, world)
        assert torch.equal(poss[s].cpu(), ref_pos) and torch.equal(n_tok[s].cpu(), ref_n)
    # fewer stores than rows: that is the point
    assert int(tokens_all.sum()) < world * T * k
    cap = int(counts_all.view(world, world, e_all).sum(dim=(0, 2)).max()) + 8
    tok_ch = _LocalChannel([torch.zeros(world * T, W, device=dev, dtype=torch.bfloat16) for _ in range(world)])
    idx_ch = _LocalChannel([torch.full((cap, 1), -7, device=dev, dtype=torch.int32) for _ in range(world)])
    row_ch = _LocalChannel([torch.zeros(cap, W, device=dev, dtype=torch.bfloat16) for _ in range(world)])
    plans = [PeerPlan.from_counts(counts_all, world, s) for s in range(world)]
    for s in range(world):
        sort_idx = torch.from_numpy(sorts[s][1]).to(dev)
        base = slot_bases(tokens_all, s)
        assert int((poss[s] >= 0).sum()) == int(tokens_all[s].sum())
        peer_push_tokens(tokens[s], poss[s], base, tok_ch, s)
        peer_push_index(plans[s], poss[s], base, sort_idx, k, idx_ch)
        peer_push(plans[s], tokens[s], row_ch, src_index=sort_idx, src_div=k)   # the reference dispatch
    for d in range(world):
        n = int(plans[d].recv_rows)
        assert int(tokens_all[:, d].sum()) <= world * T
        out = torch.full((cap, W), 3.0, device=dev, dtype=torch.bfloat16)
        expand_received(tok_ch.bufs[d], idx_ch.bufs[d].view(-1), plans[d].recv_rows, out)
        torch.cuda.synchronize()
        assert torch.equal(out[:n], row_ch.bufs[d][:n]), f"owner {d}"
        assert bool((out[n:] == 3.0).all()), "rows past the received count were written"
