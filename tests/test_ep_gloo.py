"""Expert-parallel bookkeeping on CPU ranks (gloo, world size 2 and 4): split sizes, the
wire-order <-> expert-major permutations, and the round trip dispatch -> per-expert work ->
combine against a single-process computation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_take_rows(x, index):
    return x[index.long()]


def _cpu_sort(ids, E):
    counts, inv_idx, idx = O.get_expert_counts_and_idx_fast(ids.numpy(), E)
    return torch.from_numpy(counts), torch.from_numpy(inv_idx), torch.from_numpy(idx)


def _worker(rank, world, port, E, rows_per_rank, H, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qwen3_moe_fused.parallel_ep import ExpertParallelPlan, split_sizes

        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, E, (rows_per_rank,), generator=g)
        if rank == 0:
            ids[ids == 1] = 0  # an expert that receives nothing from rank 0
        counts, inv_idx, idx = _cpu_sort(ids, E)
        x = torch.randn(rows_per_rank, H, generator=g)
        xs = x[inv_idx.long()]
        plan = ExpertParallelPlan.build(counts, world, rank, "cpu", take_rows=_cpu_take_rows, sort_fn=_cpu_sort)
        assert plan.send_splits == split_sizes(counts, world)
        assert sum(plan.recv_splits) == int(plan.local_group_sizes.sum())
        local = plan.dispatch(xs)
        # per-expert work: multiply the rows of local expert e by (global expert id + 1)
        e_local = E // world
        scale = torch.repeat_interleave(torch.arange(e_local) + rank * e_local + 1, plan.local_group_sizes.long())
        back = plan.combine(local * scale.unsqueeze(1).float())
        expect = xs * (ids[inv_idx.long()] + 1).unsqueeze(1).float()
        assert torch.allclose(back, expect), f"rank {rank}: round trip mismatch"
        torch.save({"local": local, "sizes": plan.local_group_sizes, "xs": xs, "ids_sorted": ids[inv_idx.long()]},
                   os.path.join(out_dir, f"r{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_dispatch_combine_roundtrip(tmp_path, world):
    E, rows, H = 8, 300, 5
    mp.spawn(_worker, args=(world, _free_port(), E, rows, H, str(tmp_path)), nprocs=world, join=True)
    # global check: rank r's expert-major rows = all ranks' rows of r's experts, source-major inside each expert
    saved = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    e_local = E // world
    for r in range(world):
        chunks = []
        for e in range(r * e_local, (r + 1) * e_local):
            for src in range(world):
                chunks.append(saved[src]["xs"][saved[src]["ids_sorted"] == e])
        assert torch.equal(saved[r]["local"], torch.cat(chunks))
        sizes = [sum(int((saved[src]["ids_sorted"] == e).sum()) for src in range(world))
                 for e in range(r * e_local, (r + 1) * e_local)]
        assert saved[r]["sizes"].tolist() == sizes


def test_split_sizes_and_row_ids():
    from qwen3_moe_fused.parallel_ep import local_expert_of_received_rows, split_sizes

    m = torch.tensor([3, 0, 2, 5, 1, 1, 0, 4])
    assert split_sizes(m, 2) == [10, 6]
    assert split_sizes(m, 4) == [3, 7, 2, 4]
    rc = torch.tensor([[2, 0, 1], [1, 1, 0]])
    assert local_expert_of_received_rows(rc).tolist() == [0, 0, 2, 0, 1]


def _peer_worker(rank, world, port, E, rows_per_rank, H, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from qwen3_moe_fused.parallel_ep import PeerPlan

        g = torch.Generator().manual_seed(100 + rank)
        ids = torch.randint(0, E, (rows_per_rank,), generator=g)
        if rank == 0:
            ids[ids == 1] = 0
        counts, inv_idx, _ = _cpu_sort(ids, E)
        x = torch.randn(rows_per_rank, H, generator=g)
        plan = PeerPlan.build(counts, world, rank)
        # the same exchange as two independent plans over halves of every rank's experts
        all_counts = PeerPlan.gather_counts(counts, world)
        half = E // world // 2
        halves = [PeerPlan.from_counts(all_counts, world, rank, (0, half)).__dict__,
                  PeerPlan.from_counts(all_counts, world, rank, (half, E // world)).__dict__] if half > 0 else []
        torch.save({"xs": x[inv_idx.long()], "ids_sorted": ids[inv_idx.long()], "plan": plan.__dict__, "halves": halves},
                   os.path.join(out_dir, f"p{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_peer_plan_addresses(tmp_path, world):
    """The peer-memory plan: replaying every rank's pushes on the host fills each owner's buffer
    in (local expert, source rotated to start after the owner) order, and replaying the scattered GEMM outputs puts every row back
    at its position on its source rank."""
    E, rows, H = 8, 300, 5
    mp.spawn(_peer_worker, args=(world, _free_port(), E, rows, H, str(tmp_path)), nprocs=world, join=True)
    saved = [torch.load(tmp_path / f"p{r}.pt", weights_only=False) for r in range(world)]
    e_local = E // world
    cap = rows * world
    recv = [torch.full((cap, H), float("nan")) for _ in range(world)]
    for s in range(world):
        p, xs = saved[s]["plan"], saved[s]["xs"]
        begins = torch.cumsum(p["m_sizes"].long(), 0) - p["m_sizes"].long()
        for e in range(E):
            n, d = int(p["m_sizes"][e]), int(p["dst_rank"][e])
            assert d == e // e_local
            recv[d][int(p["send_row"][e]):int(p["send_row"][e]) + n] = xs[int(begins[e]):int(begins[e]) + n]
    back = [torch.full((rows, H), float("nan")) for _ in range(world)]
    for r in range(world):
        p = saved[r]["plan"]
        chunks = []
        for e in range(r * e_local, (r + 1) * e_local):
            for j in range(world):
                src = (r + 1 + j) % world
                chunks.append(saved[src]["xs"][saved[src]["ids_sorted"] == e])
        expect = torch.cat(chunks)
        assert int(p["recv_rows"]) == expect.shape[0]
        assert torch.equal(recv[r][:expect.shape[0]], expect)
        assert p["local_m_sizes"].tolist() == [sum(int((saved[s]["ids_sorted"] == e).sum()) for s in range(world))
                                               for e in range(r * e_local, (r + 1) * e_local)]
        assert p["weight_index"].tolist() == [g // world for g in range(E)]
        # results of group g (here: the rows themselves) go to their source rank
        start = 0
        for gi in range(e_local * world):
            n, s = int(p["group_sizes"][gi]), int(p["group_src"][gi])
            back[s][int(p["return_row"][gi]):int(p["return_row"][gi]) + n] = recv[r][start:start + n]
            start += n
    for s in range(world):
        assert torch.equal(back[s], saved[s]["xs"])


@pytest.mark.parametrize("world", [2, 4])
def test_peer_plan_sub_ranges(tmp_path, world):
    """Two plans over disjoint halves of the local experts: each fills its own buffer from row 0
    with its experts' rows only, and together they return every row to its place."""
    E, rows, H = 16, 300, 3
    mp.spawn(_peer_worker, args=(world, _free_port(), E, rows, H, str(tmp_path)), nprocs=world, join=True)
    saved = [torch.load(tmp_path / f"p{r}.pt", weights_only=False) for r in range(world)]
    e_local = E // world
    half = e_local // 2
    back = [torch.full((rows, H), float("nan")) for _ in range(world)]
    for hi_, (lo, hi) in enumerate(((0, half), (half, e_local))):
        recv = [torch.full((rows * world, H), float("nan")) for _ in range(world)]
        for s in range(world):
            p, xs = saved[s]["halves"][hi_], saved[s]["xs"]
            begins = torch.cumsum(p["m_sizes"].long(), 0) - p["m_sizes"].long()
            for e in range(E):
                if not bool(p["send_mask"][e]):
                    assert not (lo <= e % e_local < hi)
                    continue
                n, d = int(p["m_sizes"][e]), int(p["dst_rank"][e])
                recv[d][int(p["send_row"][e]):int(p["send_row"][e]) + n] = xs[int(begins[e]):int(begins[e]) + n]
        for r in range(world):
            p = saved[r]["halves"][hi_]
            chunks = [saved[(r + 1 + j) % world]["xs"][saved[(r + 1 + j) % world]["ids_sorted"] == e]
                      for e in range(r * e_local + lo, r * e_local + hi) for j in range(world)]
            expect = torch.cat(chunks)
            assert int(p["recv_rows"]) == expect.shape[0] and p["expert_lo"] == lo
            assert torch.equal(recv[r][:expect.shape[0]], expect)
            assert p["weight_index"].tolist() == [g // world for g in range((hi - lo) * world)]
            start = 0
            for gi in range((hi - lo) * world):
                n, s = int(p["group_sizes"][gi]), int(p["group_src"][gi])
                back[s][int(p["return_row"][gi]):int(p["return_row"][gi]) + n] = recv[r][start:start + n]
                start += n
    for s in range(world):
        assert torch.equal(back[s], saved[s]["xs"])


@pytest.mark.parametrize("world", [2, 4])
def test_push_limits_when_a_receive_buffer_is_too_small(world):
    """A routing that sends more rows to one owner than its buffer holds: the limits handed to the push
    kernel keep exactly the rows that fit (in the owner's layout order) and the rest is what the
    kernel counts as dropped; experts outside a sub-range plan are marked -1."""
    from qwen3_moe_fused.parallel_ep import PeerPlan, push_limits

    E, e_local = 8, 8 // world
    g = torch.Generator().manual_seed(world)
    counts = torch.randint(0, 40, (world, E), generator=g, dtype=torch.int32)
    counts[:, :e_local] += 100  # everybody sends most rows to rank 0's experts
    recv = counts.view(world, world, e_local).sum(dim=(0, 2))  # rows each owner receives
    capacity = int(recv[0]) - 57  # rank 0's buffer is 57 rows short; the others' are large enough
    assert capacity > int(recv[1:].max())
    dropped = 0
    kept_on_owner0 = 0
    for rank in range(world):
        plan = PeerPlan.from_counts(counts, world, rank)
        limit = push_limits(plan, capacity)
        assert limit.dtype == torch.int32 and (limit >= 0).all()
        m = counts[rank]
        kept = torch.minimum(m, limit)
        dropped += int((m - kept).sum())
        kept_on_owner0 += int(kept[:e_local].sum())
        # rows kept never reach past the end of the owner's buffer
        assert ((plan.send_row + kept.long())[kept > 0] <= capacity).all()
        # owners with room lose nothing
        assert torch.equal(kept[e_local:], m[e_local:])
    assert dropped == 57 and kept_on_owner0 == capacity
    sub = PeerPlan.from_counts(counts, world, 0, (0, 1))
    lim = push_limits(sub, 10 ** 6)
    inside = torch.zeros(E, dtype=torch.bool)
    inside[torch.arange(world) * e_local] = True
    assert (lim[~inside] == -1).all() and torch.equal(lim[inside], counts[0][inside].clamp(min=0) * 0 + lim[inside]) and (lim[inside] >= 0).all()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_token_slots_are_dense_and_unique(world):
    """Token-deduplicated dispatch bookkeeping: on every destination the slots of all ranks' tokens are
    exactly 0 .. n-1, rank by rank, each rank's tokens in their own order; a token is sent to a rank iff
    one of its experts lives there."""
    from qwen3_moe_fused.parallel_ep import slot_bases, token_positions

    E, T, k = 32, 200, 4
    e_all = E // world
    g = torch.Generator().manual_seed(world)
    sel = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]) for _ in range(world)]
    poss, n_tok = zip(*[token_positions(s, E, world) for s in sel])
    tokens_all = torch.stack(n_tok)
    for s in range(world):
        want = torch.zeros(T, world, dtype=torch.bool)
        for d in range(world):
            want[:, d] = ((sel[s] // e_all) == d).any(dim=1)
        assert torch.equal(poss[s] >= 0, want)
    for d in range(world):
        got = torch.cat([(poss[s][:, d] + slot_bases(tokens_all, s)[d])[poss[s][:, d] >= 0] for s in range(world)])
        assert torch.equal(got.long(), torch.arange(int(tokens_all[:, d].sum())))
