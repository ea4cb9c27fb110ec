"""Expert-parallel execution of the grouped GEMMs: the E experts are split evenly over the
ranks of a process group (expert e lives on rank e // (E / world)), tokens stay where they
were routed, and rows travel to the owner of their expert and back by all-to-all.

The reference has no multi-GPU path (its README leaves multi-GPU support open); this module
is the data-parallel extension of `moe_fused_linear` described by the build's scope.

Dispatch order.  A rank's rows are already sorted by global expert id, hence by destination
rank, so the send buffer needs no packing.  Received rows arrive ordered (source rank, local
expert); one stable sort by local expert (the same kernel that sorts tokens) turns them into
the expert-major order the grouped GEMMs expect, and its inverse permutation restores the
wire order before results are sent back.  No collective is needed for dW: each expert's
weight lives on exactly one rank.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch
import torch.distributed as dist


def split_sizes(m_sizes_host: torch.Tensor, world: int) -> list[int]:
    """Rows this rank sends to each rank: sums of m_sizes over each rank's block of experts."""
    E = m_sizes_host.numel()
    assert E % world == 0, "experts must divide evenly over the ranks"
    return m_sizes_host.view(world, E // world).sum(dim=1).tolist()


def local_expert_of_received_rows(recv_counts: torch.Tensor) -> torch.Tensor:
    """recv_counts (world, E_local): rows from each source for each local expert, in wire
    order.  Returns the local expert id of every received row (int64)."""
    world, e_local = recv_counts.shape
    ids = torch.arange(e_local, device=recv_counts.device).repeat(world)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).long())


def _cuda_take_rows(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    from .kernels.routing import _gather_rows

    assert x.is_cuda, "expert-parallel row movement runs on the GPU"
    return _gather_rows(x.contiguous(), index.to(torch.int32).contiguous(), 1)


def _cuda_sort(ids: torch.Tensor, E: int):
    from .kernels.indexing import get_expert_counts_and_idx

    return get_expert_counts_and_idx(ids, E)


@dataclass
class ExpertParallelPlan:
    world: int
    rank: int
    send_splits: list[int]
    recv_splits: list[int]
    local_group_sizes: torch.Tensor      # (E_local,) int32 rows per local expert after dispatch
    to_expert_major: torch.Tensor        # gather index: wire order -> expert-major
    to_wire: torch.Tensor                # gather index: expert-major -> wire order
    group: Optional[dist.ProcessGroup]
    take_rows: Callable

    @staticmethod
    def build(m_sizes: torch.Tensor, world: int, rank: int, device, group=None,
              take_rows: Callable = _cuda_take_rows, sort_fn: Callable = _cuda_sort) -> "ExpertParallelPlan":
        """m_sizes (E,): rows of this rank per GLOBAL expert (rows sorted by expert)."""
        E = m_sizes.numel()
        e_local = E // world
        send_counts = m_sizes.to(torch.int32).view(world, e_local).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        # split sizes are host integers for the variable-size all-to-all: one small D2H copy
        host = torch.stack([send_counts.sum(dim=1), recv_counts.sum(dim=1)]).cpu()
        send_splits, recv_splits = host[0].tolist(), host[1].tolist()
        ids = local_expert_of_received_rows(recv_counts)
        counts, inv_idx, idx = sort_fn(ids, e_local)
        return ExpertParallelPlan(world, rank, send_splits, recv_splits, counts, inv_idx, idx, group, take_rows)

    # rows (sorted by global expert) -> rows of my experts, expert-major
    def dispatch(self, rows: torch.Tensor) -> torch.Tensor:
        recv = rows.new_empty((sum(self.recv_splits), rows.shape[1]))
        dist.all_to_all_single(recv, rows.contiguous(), self.recv_splits, self.send_splits, group=self.group)
        return self.take_rows(recv, self.to_expert_major)

    # expert-major results -> back to the ranks the rows came from, in their sorted order
    def combine(self, rows: torch.Tensor) -> torch.Tensor:
        wire = self.take_rows(rows, self.to_wire)
        back = rows.new_empty((sum(self.send_splits), rows.shape[1]))
        dist.all_to_all_single(back, wire, self.send_splits, self.recv_splits, group=self.group)
        return back

    def grouped(self, fn: Callable, rows: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return fn(rows, weight, self.local_group_sizes)

    def grouped_dw(self, fn: Callable, x: torch.Tensor, dy: torch.Tensor, dtype, e_local: int) -> torch.Tensor:
        return fn(x, dy, self.local_group_sizes, dtype)


# ------------------------------------------------------------------------------------------
# Expert parallelism over peer memory: no all-to-all.  Every rank maps every other rank's
# receive buffers (symmetric memory over NVLink); rows are pushed by a copy kernel straight to
# their expert-major position on the owner of their expert, and the forward / dX GEMMs write
# each (local expert, source rank) group of results with TMA stores straight into the source
# rank's memory, at the position the rows had there.  One small count all-gather per routing
# decision and one fence per phase are the only collectives.
# ------------------------------------------------------------------------------------------
_DST_RANK_TABLES: dict = {}


def _dst_rank_table(E: int, e_all: int, dev) -> torch.Tensor:
    """Owner of every global expert (a constant of the configuration, built once per device)."""
    key = (E, e_all, str(dev))
    if key not in _DST_RANK_TABLES:
        _DST_RANK_TABLES[key] = torch.arange(E, device=dev) // e_all
    return _DST_RANK_TABLES[key]


@dataclass
class PeerPlan:
    """Row bookkeeping of one routing decision, all tensors on the device, no host sync.

    Groups on rank d are ordered (local expert, slot): g = el * world + j, holding the rows of
    source rank (d + 1 + j) % world.
    """

    world: int
    rank: int
    e_local: int
    m_sizes: torch.Tensor          # (E,) int32: this rank's rows per global expert
    dst_rank: torch.Tensor         # (E,) int64: owner of each global expert
    send_row: torch.Tensor         # (E,) int64: first row, in the owner's receive buffer, of my rows of expert e
    group_sizes: torch.Tensor      # (G,) int32: rows of each (local expert, source) group received here
    weight_index: torch.Tensor     # (G,) int32: local expert of each group
    group_src: torch.Tensor        # (G,) int64: source rank of each group
    return_row: torch.Tensor       # (G,) int64: first row of the group in its source rank's sorted order
    local_m_sizes: torch.Tensor    # (E_local,) int32: rows per local expert after dispatch
    recv_rows: torch.Tensor        # () int64: rows this rank receives in total
    send_mask: Optional[torch.Tensor] = None  # (E,) bool: experts this plan moves (None: all)
    expert_lo: int = 0             # first local expert of this plan (plans over a sub-range of the local experts)
    cache: dict = field(default_factory=dict, repr=False)  # address tables per channel, built on first use

    @staticmethod
    def gather_counts(m_sizes: torch.Tensor, world: int, group=None) -> torch.Tensor:
        """(world, E) int32: rows of every rank per global expert (one all-gather)."""
        E = m_sizes.numel()
        assert E % world == 0, "experts must divide evenly over the ranks"
        mine = m_sizes.to(torch.int32).contiguous()
        counts = torch.empty(world * E, dtype=torch.int32, device=mine.device)
        dist.all_gather_into_tensor(counts, mine, group=group)
        return counts.view(world, E)

    @staticmethod
    def build(m_sizes: torch.Tensor, world: int, rank: int, group=None) -> "PeerPlan":
        return PeerPlan.from_counts(PeerPlan.gather_counts(m_sizes, world, group), world, rank)

    @staticmethod
    def from_counts(counts: torch.Tensor, world: int, rank: int, local_range: Optional[tuple] = None) -> "PeerPlan":
        """counts (world, E): rows of every rank per global expert.

        `local_range` = (lo, hi) restricts the plan to local experts lo..hi-1 of every rank: their
        rows are laid out from row 0 of the (sub-)buffer they are pushed into, the groups are
        those experts' only, and `weight_index` counts from expert lo.  Plans over disjoint ranges
        are independent, so the exchange of one range can overlap the GEMMs of another."""
        E = counts.shape[1]
        e_all = E // world
        dev = counts.device
        lo, hi = local_range if local_range is not None else (0, e_all)
        assert 0 <= lo < hi <= e_all
        e_local = hi - lo
        if counts.is_cuda:
            # one kernel instead of two dozen small tensor operations
            from . import _lib

            counts = counts.to(torch.int32).contiguous()
            G = e_local * world
            i64 = torch.empty(E + 2 * G + 1, dtype=torch.int64, device=dev)
            i32 = torch.empty(E + 2 * G + e_local, dtype=torch.int32, device=dev)
            send_row, group_src, return_row, recv_rows = i64[:E], i64[E:E + G], i64[E + G:E + 2 * G], i64[E + 2 * G:]
            send_ok, group_sizes, weight_index, local_m = i32[:E], i32[E:E + G], i32[E + G:E + 2 * G], i32[E + 2 * G:]
            with torch.cuda.device(dev):
                _lib.check(_lib.load().moe_ep_plan(
                    _lib.ptr(counts), world, rank, E, lo, hi, _lib.ptr(send_row), _lib.ptr(send_ok), _lib.ptr(group_sizes),
                    _lib.ptr(weight_index), _lib.ptr(group_src), _lib.ptr(return_row), _lib.ptr(local_m), _lib.ptr(recv_rows),
                    _lib.stream_ptr(dev)), "moe_ep_plan")
            return PeerPlan(
                world=world, rank=rank, e_local=e_local, m_sizes=counts[rank], dst_rank=_dst_rank_table(E, e_all, dev),
                send_row=send_row, group_sizes=group_sizes, weight_index=weight_index, group_src=group_src,
                return_row=return_row, local_m_sizes=local_m, recv_rows=recv_rows[0],
                send_mask=None if local_range is None else send_ok.bool(), expert_lo=lo)
        c = counts.view(world, world, e_all).long()[:, :, lo:hi]   # [source, owner, local expert of the range]
        # On owner d the sources of an expert are laid out d+1, d+2, ..., d (mod world): when every
        # rank walks its groups in order, the ranks' result stores go to distinct ranks at any one time.
        owners = torch.arange(world, device=dev)
        src_of = (owners.view(world, 1) + 1 + torch.arange(world, device=dev).view(1, world)) % world   # [owner, slot] -> source
        per_owner = c.permute(1, 2, 0)                             # [owner, local expert, source]
        per_owner = torch.gather(per_owner, 2, src_of.view(world, 1, world).expand(world, e_local, world)).contiguous()  # [owner, el, slot]
        flat = per_owner.view(world, e_local * world)
        first = flat.cumsum(dim=1) - flat                          # exclusive: first row of each group on its owner
        my_slot = (rank - owners - 1) % world                      # slot of this rank's rows on each owner
        send_sub = torch.gather(first.view(world, e_local, world), 2,
                                my_slot.view(world, 1, 1).expand(world, e_local, 1)).view(world, e_local)
        send_row = torch.zeros((world, e_all), dtype=torch.int64, device=dev)
        send_row[:, lo:hi] = send_sub
        send_mask = torch.zeros((world, e_all), dtype=torch.bool, device=dev)
        send_mask[:, lo:hi] = True
        begins = counts.long().cumsum(dim=1) - counts.long()       # [source, global expert]: first row in the source's order
        mine = per_owner[rank]                                     # [local expert, slot]
        g = torch.arange(e_local * world, device=dev)
        group_src = (rank + 1 + g % world) % world
        group_expert = rank * e_all + lo + g // world
        return_row = begins[group_src, group_expert]
        return PeerPlan(
            world=world, rank=rank, e_local=e_local, m_sizes=counts[rank].contiguous(),
            dst_rank=torch.arange(E, device=dev) // e_all, send_row=send_row.reshape(E).contiguous(),
            group_sizes=mine.reshape(-1).to(torch.int32).contiguous(), weight_index=(g // world).to(torch.int32),
            group_src=group_src, return_row=return_row.contiguous(),
            local_m_sizes=mine.sum(dim=1).to(torch.int32).contiguous(), recv_rows=mine.sum(),
            send_mask=None if local_range is None else send_mask.reshape(E), expert_lo=lo)


class PeerChannel:
    """A (capacity, width) buffer on every rank that every rank can address."""

    def __init__(self, capacity_rows: int, width: int, dtype: torch.dtype, device, group=None):
        import os

        # this module never uses multicast addresses: keep the allocation off NVLink multicast objects
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.local = symm_mem.empty((capacity_rows, width), dtype=dtype, device=device)
        handle = symm_mem.rendezvous(self.local, group)
        self.handle = handle
        self.capacity_rows = capacity_rows
        self.row_bytes = width * self.local.element_size()
        self.ptrs = torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64, device=device)
        assert int(self.ptrs[dist.get_rank(group)]) == self.local.data_ptr()

    def rows(self, first_row: int, n_rows: int) -> "PeerChannelRows":
        """Rows first_row .. first_row + n_rows - 1 of the buffer on every rank, as a channel of their own."""
        assert 0 <= first_row and first_row + n_rows <= self.capacity_rows
        return PeerChannelRows(self.local[first_row:first_row + n_rows], self.ptrs + first_row * self.row_bytes,
                               n_rows, self.row_bytes)


@dataclass
class PeerChannelRows:
    local: torch.Tensor
    ptrs: torch.Tensor
    capacity_rows: int
    row_bytes: int


def peer_fence(token: torch.Tensor, group=None) -> None:
    """Orders this rank's earlier work on the current stream (peer stores included) before every
    rank's later work on theirs: a one-element all-reduce."""
    dist.all_reduce(token, group=group)


def push_rows(rows: torch.Tensor, m_sizes: torch.Tensor, dst_ptrs: torch.Tensor,
              dst_limit: Optional[torch.Tensor] = None, max_ctas: int = 0, first_expert: int = 0,
              src_index: Optional[torch.Tensor] = None, src_div: int = 1,
              dropped: Optional[torch.Tensor] = None) -> None:
    """rows (M, W) sorted by expert, m_sizes (E,): row i of expert e is copied to the address
    dst_ptrs[e] + i * row_bytes (int64 device tensor of addresses, local or peer memory).
    `dst_limit` (int32 per expert): negative = the expert's rows are not part of this push;
    otherwise rows with i >= dst_limit[e] do not fit into the receiver's buffer: they are not
    written and are counted in `dropped` (int32 device scalar, incremented per dropped row).
    The copy starts with the rows of `first_expert`.
    With `src_index` (int32, one entry per sorted row) sorted row r is read from
    rows[src_index[r] // src_div]: token rows are expanded while they are pushed."""
    from . import _lib

    assert rows.is_cuda and rows.is_contiguous() and rows.dim() == 2
    assert dst_ptrs.dtype == torch.int64 and dst_ptrs.is_contiguous() and dst_ptrs.numel() == m_sizes.numel()
    m_sizes = _lib.as_index_tensor(m_sizes).contiguous()
    if dst_limit is not None:
        assert dst_limit.dtype == torch.int32 and dst_limit.is_contiguous() and dst_limit.numel() == m_sizes.numel()
    if dropped is not None:
        assert dropped.dtype == torch.int32 and dropped.is_cuda and dropped.numel() == 1
    n_rows = rows.shape[0]
    if src_index is not None:
        assert src_index.dtype == torch.int32 and src_index.is_contiguous()
        n_rows = src_index.numel()
    _lib.check(_lib.load().moe_ep_push_rows(
        _lib.ptr(rows), n_rows, rows.shape[1] * rows.element_size(), _lib.ptr(m_sizes), _lib.int_code(m_sizes.dtype),
        m_sizes.numel(), _lib.ptr(dst_ptrs), _lib.ptr(dst_limit), first_expert, _lib.ptr(src_index), src_div, max_ctas,
        _lib.ptr(dropped), _lib.stream_ptr(rows.device)), "moe_ep_push_rows")


def scattered_grouped_gemm(x: torch.Tensor, weight: torch.Tensor, group_sizes: torch.Tensor,
                           weight_index: Optional[torch.Tensor], out_ptrs: torch.Tensor, out_template: torch.Tensor,
                           transposed: bool = False) -> None:
    """Forward (weight (E_w, N, K)) or dX (`transposed`: weight (E_w, K, N)) over G groups of the
    rows of x; group g uses weight slice weight_index[g] and its results start at the address
    out_ptrs[g] (int64 device tensor, local or peer memory) with row pitch N."""
    from . import _lib

    assert x.is_cuda and x.is_contiguous() and weight.is_contiguous() and x.dim() == 2 and weight.dim() == 3
    M, K = x.shape
    e_w, N, kw = weight.shape if not transposed else (weight.shape[0], weight.shape[2], weight.shape[1])
    assert kw == K and weight.dtype == x.dtype
    G = group_sizes.numel()
    group_sizes = _lib.as_index_tensor(group_sizes).contiguous()
    assert out_ptrs.dtype == torch.int64 and out_ptrs.is_contiguous() and out_ptrs.numel() == G
    # out_ptrs are buffer bases plus whole rows: with a row pitch of a multiple of 16 bytes every entry is
    # 16-byte aligned (what the output tensor maps need) without reading the device tensor here
    assert (N * x.element_size()) % 16 == 0 and out_template.data_ptr() % 16 == 0
    if weight_index is not None:
        assert weight_index.dtype == torch.int32 and weight_index.is_contiguous() and weight_index.numel() == G
    lib = _lib.load()
    ws_ptr, ws_bytes = _lib.workspace(x.device, lib.moe_grouped_gemm_workspace_bytes(0, M, N, K, G))
    name = "moe_grouped_gemm_dx_scattered" if transposed else "moe_grouped_gemm_fwd_scattered"
    dt = _lib.float_code(x.dtype)
    _lib.check(getattr(lib, name)(
        _lib.ptr(x), _lib.ptr(weight), _lib.ptr(group_sizes), _lib.int_code(group_sizes.dtype), _lib.ptr(weight_index), e_w,
        _lib.ptr(out_ptrs), _lib.ptr(out_template), M, N, K, G, dt, dt, ws_ptr, ws_bytes, _lib.stream_ptr(x.device)), name)


def push_limits(plan: PeerPlan, capacity_rows: int) -> torch.Tensor:
    """(E,) int32 for `push_rows`: how many of this rank's rows of each expert fit into the owner's
    buffer of `capacity_rows` rows (the rows start at plan.send_row there); -1 for experts that another
    plan moves."""
    limit = (capacity_rows - plan.send_row).clamp(min=0, max=2**31 - 1).to(torch.int32)
    if plan.send_mask is not None:
        limit = torch.where(plan.send_mask, limit, torch.full_like(limit, -1))
    return limit.contiguous()


def peer_push(plan: PeerPlan, rows: torch.Tensor, channel, max_ctas: int = 0,
              src_index: Optional[torch.Tensor] = None, src_div: int = 1,
              dropped: Optional[torch.Tensor] = None) -> None:
    """Rows sorted by global expert -> expert-major (local expert, source) order in the owners' `channel`.
    With `src_index` / `src_div` the sorted rows are rows[src_index // src_div] (see push_rows).
    Rows that do not fit into an owner's buffer are never written past its end; they are counted
    in `dropped` (see push_rows), and the owner's results for them do not exist."""
    row_bytes = rows.shape[1] * rows.element_size()
    assert row_bytes == channel.row_bytes
    key = ("push", id(channel))
    if key not in plan.cache:
        dst = (channel.ptrs[plan.dst_rank] + plan.send_row * row_bytes).contiguous()
        plan.cache[key] = (dst, push_limits(plan, channel.capacity_rows), channel)  # the channel object is kept alive with its key
    dst, limit, _ = plan.cache[key]
    # every rank starts with the rows of the next rank's experts, so the ranks' writes fan out
    # over distinct destinations instead of converging on one receiver at a time
    e_all = plan.m_sizes.numel() // plan.world
    push_rows(rows, plan.m_sizes, dst, limit, max_ctas, first_expert=((plan.rank + 1) % plan.world) * e_all,
              src_index=src_index, src_div=src_div, dropped=dropped)


def peer_grouped_gemm(plan: PeerPlan, rows_in, weight: torch.Tensor, rows_out, transposed: bool = False) -> None:
    """Forward or dX over the rows received in `rows_in`; each (local expert, source) group's
    results are stored into the source rank's `rows_out` at the rows' position in that rank's order.
    `weight` holds the plan's local experts only."""
    assert weight.shape[0] == plan.e_local
    key = ("gemm", id(rows_out))
    if key not in plan.cache:
        plan.cache[key] = ((rows_out.ptrs[plan.group_src] + plan.return_row * rows_out.row_bytes).contiguous(), rows_out)
    scattered_grouped_gemm(rows_in.local, weight, plan.group_sizes, plan.weight_index, plan.cache[key][0], rows_out.local, transposed)


# ------------------------------------------------------------------------------------------
# Token-deduplicated dispatch.  With top-k routing a token has k rows, but its experts live on
# fewer than k ranks (on average 1.99 / 3.6 / 5.25 of 2 / 4 / 8 ranks for k = 8 of 128 experts):
# the token travels once per destination RANK, and each of its rows sends a 4-byte index.
# ------------------------------------------------------------------------------------------
def token_positions(selected: torch.Tensor, E: int, world: int):
    """selected (T, k) expert ids.  Returns (pos (T, world) int32: number of earlier tokens of this rank
    that also have an expert on rank d, -1 where token t has none there; n_tokens (world,) int32: tokens
    this rank sends to each rank).  One kernel on the GPU."""
    T, k = selected.shape
    if selected.is_cuda:
        from . import _lib

        selected = _lib.as_index_tensor(selected).contiguous()
        pos = torch.empty((T, world), dtype=torch.int32, device=selected.device)
        n_tokens = torch.empty(world, dtype=torch.int32, device=selected.device)
        with torch.cuda.device(selected.device):
            _lib.check(_lib.load().moe_ep_token_positions(
                _lib.ptr(selected), _lib.int_code(selected.dtype), T, k, E, world, _lib.ptr(pos), _lib.ptr(n_tokens),
                _lib.stream_ptr(selected.device)), "moe_ep_token_positions")
        return pos, n_tokens
    mask = torch.zeros((T, world), dtype=torch.bool)
    mask.scatter_(1, torch.div(selected, E // world, rounding_mode="floor"), True)
    pos = mask.to(torch.int32).cumsum(dim=0, dtype=torch.int32) - 1
    return torch.where(mask, pos, torch.full_like(pos, -1)).contiguous(), mask.sum(dim=0).to(torch.int32)


def gather_counts_and_tokens(m_sizes: torch.Tensor, n_tokens: torch.Tensor, world: int, group=None):
    """One all-gather for both tables: (counts (world, E) int32: rows of every rank per global expert;
    tokens (world, world) int32: tokens rank s sends to rank d)."""
    E = m_sizes.numel()
    mine = torch.cat([m_sizes.to(torch.int32), n_tokens.to(torch.int32)]).contiguous()
    out = torch.empty(world * (E + world), dtype=torch.int32, device=mine.device)
    dist.all_gather_into_tensor(out, mine, group=group)
    out = out.view(world, E + world)
    return out[:, :E].contiguous(), out[:, E:].contiguous()


def slot_bases(tokens_all: torch.Tensor, rank: int) -> torch.Tensor:
    """(world,) int32: where this rank's tokens start in each rank's token buffer.  Rank d's buffer holds
    the tokens of rank 0, then rank 1, ...; a rank's tokens keep their order, so the slot of token t on
    rank d is slot_bases[d] + pos[t, d]."""
    return tokens_all[:rank].sum(dim=0, dtype=torch.int32).contiguous()


def peer_push_tokens(tokens: torch.Tensor, pos: torch.Tensor, slot_base: torch.Tensor, channel, rank: int,
                     dropped: Optional[torch.Tensor] = None, max_ctas: int = 0) -> None:
    """Every token row goes once to each rank that owns one of its experts (pos / slot_base: see
    token_positions and slot_bases)."""
    from . import _lib

    assert tokens.is_cuda and tokens.is_contiguous() and tokens.dim() == 2
    world = pos.shape[1]
    assert pos.dtype == torch.int32 and pos.is_contiguous() and pos.shape[0] == tokens.shape[0]
    assert slot_base.dtype == torch.int32 and slot_base.numel() == world
    row_bytes = tokens.shape[1] * tokens.element_size()
    assert row_bytes == channel.row_bytes
    _lib.check(_lib.load().moe_ep_push_tokens(
        _lib.ptr(tokens), tokens.shape[0], row_bytes, _lib.ptr(pos), _lib.ptr(slot_base), world, (rank + 1) % world,
        _lib.ptr(channel.ptrs), channel.capacity_rows, max_ctas, _lib.ptr(dropped), _lib.stream_ptr(tokens.device)), "moe_ep_push_tokens")


def peer_push_index(plan: PeerPlan, pos: torch.Tensor, slot_base: torch.Tensor, sort_idx: torch.Tensor, k: int, channel,
                    dropped: Optional[torch.Tensor] = None) -> None:
    """The 4-byte companion of peer_push_tokens: for every expanded row (sorted by expert) the slot of its
    token on the expert's owner, stored at the row's expert-major position in the owners' `channel`
    (a PeerChannel of int32 rows of width 1)."""
    from . import _lib

    assert channel.row_bytes == 4 and sort_idx.dtype == torch.int32 and sort_idx.is_contiguous()
    key = ("index", id(channel))
    if key not in plan.cache:
        dst = (channel.ptrs[plan.dst_rank] + plan.send_row * 4).contiguous()
        plan.cache[key] = (dst, push_limits(plan, channel.capacity_rows), channel)
    dst, limit, _ = plan.cache[key]
    _lib.check(_lib.load().moe_ep_push_index(
        _lib.ptr(pos), _lib.ptr(slot_base), plan.world, _lib.ptr(sort_idx), k, sort_idx.numel(), _lib.ptr(plan.m_sizes),
        _lib.int_code(plan.m_sizes.dtype), plan.m_sizes.numel(), _lib.ptr(dst), _lib.ptr(limit), _lib.ptr(dropped),
        _lib.stream_ptr(pos.device)), "moe_ep_push_index")


def expand_received(tokens: torch.Tensor, index: torch.Tensor, n_rows: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = tokens[index[r]] for the first n_rows rows (n_rows: int64 device scalar, e.g. plan.recv_rows;
    never read on the host).  Rows beyond stay as they are."""
    from . import _lib

    assert tokens.is_contiguous() and out.is_contiguous() and index.dtype == torch.int32 and n_rows.dtype == torch.int64
    assert tokens.shape[1] == out.shape[1] and tokens.dtype == out.dtype
    max_rows = min(out.shape[0], index.numel())
    _lib.check(_lib.load().moe_ep_expand_rows(
        _lib.ptr(tokens), tokens.shape[0], tokens.shape[1] * tokens.element_size(), _lib.ptr(index), _lib.ptr(n_rows), max_rows,
        _lib.ptr(out), _lib.stream_ptr(tokens.device)), "moe_ep_expand_rows")
    return out


class ReceiveOverflow(RuntimeError):
    """Rows of an earlier expert-parallel call did not fit into an owner's receive buffer."""


class PeerMoeBlock:
    """Forward of the sparse MoE block with the experts split over the ranks (inference; no autograd).

    What `moe_block.moe_block_forward` computes for this rank's tokens, with every token sent to the
    ranks that own its experts: router and sort run locally; each token row is stored ONCE into the
    token buffer of every rank that owns one of its experts, and each of its k rows sends a 4-byte
    index to its expert-major position there (token-deduplicated dispatch); the owner expands its
    rows from the received tokens, runs gate / up / SiLU-mul, and the down projection's epilogue
    stores every result row straight back into the token's rank, where the weighted combine runs.
    Two fences per call, no all-to-all.  (`max_tokens=None` selects the older dispatch that sends
    one row per (token, expert).)

    Receive capacity.  In the worst routing every rank sends all its rows to one owner, world *
    max_rows rows.  By default the receive buffers have that size, so no routing can overflow them.
    With a smaller `capacity_factor` a skewed routing can: rows that do not fit are never written
    (nothing is stored out of bounds), the push kernels count them on the sending rank, and the
    outputs of the tokens they belong to are WRONG for that call (their result rows hold whatever an
    earlier call left there, or NaN with `poison_results=True`).  The counts of all ranks are summed
    inside the call's first fence and copied to the host without stalling the stream; a non-zero
    sum raises `ReceiveOverflow` on EVERY rank at the start of the NEXT call on this object (so no
    rank is left waiting in a collective), or when `check()` is called; `check_capacity=True` tests
    this rank's own receive count before pushing (one host read).
    """

    def __init__(self, world: int, rank: int, device, hidden: int, max_rows: int, dtype: torch.dtype,
                 capacity_factor: Optional[float] = None, group=None, max_tokens: Optional[int] = None,
                 poison_results: bool = False):
        """max_rows: tokens * top_k per rank; max_tokens: tokens per rank (enables the token-deduplicated
        dispatch); a rank can receive up to capacity_factor * max_rows rows (None: world * max_rows, which
        every routing fits into).  poison_results: with a capacity that can overflow, fill the result buffer
        with NaN before every call, so that the outputs of tokens whose rows were dropped are NaN instead of
        numbers of an earlier call (costs one pass over max_rows * hidden; the overflow is reported either way)."""
        self.world, self.rank, self.group = world, rank, group
        factor = float(world) if capacity_factor is None else float(capacity_factor)
        cap = (int(max_rows * factor) + 7) // 8 * 8
        self.can_overflow = cap < world * max_rows
        self.poison_results = poison_results and self.can_overflow
        self.dedup = max_tokens is not None
        if self.dedup:
            self.ch_tok = PeerChannel(world * max_tokens, hidden, dtype, device, group)  # every rank's tokens fit
            self.ch_idx = PeerChannel(cap, 1, torch.int32, device, group)
            self.rows = torch.empty((cap, hidden), dtype=dtype, device=device)           # expanded locally
        else:
            self.ch_x = PeerChannel(cap, hidden, dtype, device, group)
        self.capacity_rows = cap
        self.ch_y = PeerChannel(max_rows, hidden, dtype, device, group)
        self.token = torch.zeros(2, device=device)   # fence payload: [0] nothing, [1] rows dropped by all ranks
        self.dropped = torch.zeros(1, dtype=torch.int32, device=device)   # rows this rank could not deliver, all calls
        self.dropped_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.dropped_seen = torch.cuda.Event()
        self.dropped_seen.record()
        peer_fence(self.token, group)

    def check(self) -> None:
        """Raises ReceiveOverflow if rows of an earlier call were dropped by any rank (waits for that call's
        first fence only).  The count is summed over the ranks inside the fence, so every rank raises at
        the same call and none is left waiting in a collective."""
        self.dropped_seen.synchronize()
        n = int(self.dropped_host[0])
        if n:
            raise ReceiveOverflow(f"{n} rows did not fit into their owners' receive buffers (capacity {self.capacity_rows} rows "
                                  f"per rank); the outputs of the affected tokens were wrong. Build PeerMoeBlock with a larger capacity_factor.")

    @torch.no_grad()
    def forward(self, x: torch.Tensor, gate_weight: torch.Tensor, gate_proj: torch.Tensor, up_proj: torch.Tensor,
                down_proj: torch.Tensor, num_selected: int, norm_topk_prob: bool = True, check_capacity: bool = False):
        """x (T, H): this rank's tokens; gate_weight (E, H) on every rank; gate_proj / up_proj (E_local, I, H) and
        down_proj (E_local, H, I): this rank's experts.  Returns (out (T, H), router_logits (T, E))."""
        from .kernels.fused_mlp import gate_up_silu_forward
        from .kernels.indexing import get_expert_counts_and_idx
        from .kernels.routing import _combine, softmax_topk

        T, H = x.shape
        E, k = gate_weight.shape[0], num_selected
        assert T * k <= self.ch_y.capacity_rows
        if self.can_overflow:
            self.check()  # an overflow of the previous call is reported before more work is queued
        x = x.contiguous()
        router_logits = torch.nn.functional.linear(x, gate_weight)
        weights, selected = softmax_topk(router_logits, k, norm_topk_prob, x.dtype)
        m_sizes, sort_idx, inv_sort_idx = get_expert_counts_and_idx(selected.view(T * k), E)
        if self.dedup:
            assert T * self.world <= self.ch_tok.capacity_rows
            pos, n_tokens = token_positions(selected, E, self.world)
            counts_all, tokens_all = gather_counts_and_tokens(m_sizes, n_tokens, self.world, self.group)
            plan = PeerPlan.from_counts(counts_all, self.world, self.rank)
        else:
            plan = PeerPlan.build(m_sizes, self.world, self.rank, self.group)
        if check_capacity:  # one host read
            assert int(plan.recv_rows) <= self.capacity_rows, "receive buffer too small for this routing"
        if self.poison_results:
            # result rows that never arrive (their input was dropped) must not be whatever an earlier call left there
            self.ch_y.local[:T * k].fill_(float("nan"))
        if self.dedup:
            base = slot_bases(tokens_all, self.rank)
            peer_push_tokens(x, pos, base, self.ch_tok, self.rank)
            peer_push_index(plan, pos, base, sort_idx, k, self.ch_idx, dropped=self.dropped)
        else:
            peer_push(plan, x, self.ch_x, src_index=sort_idx, src_div=k, dropped=self.dropped)  # rows are expanded while they travel
        if self.can_overflow:
            self.token[1:2].copy_(self.dropped)  # summed over the ranks by the fence
        peer_fence(self.token, self.group)  # every rank's rows have arrived (and the previous call's reads are over)
        if self.can_overflow:
            self.dropped_host.copy_(self.token[1:2], non_blocking=True)
            self.dropped_seen.record()
        if self.dedup:
            rows = expand_received(self.ch_tok.local, self.ch_idx.local.view(-1), plan.recv_rows, self.rows)
        else:
            rows = self.ch_x.local
        h = gate_up_silu_forward(rows, gate_proj, up_proj, plan.local_m_sizes)
        out_ptrs = (self.ch_y.ptrs[plan.group_src] + plan.return_row * self.ch_y.row_bytes).contiguous()
        scattered_grouped_gemm(h, down_proj, plan.group_sizes, plan.weight_index, out_ptrs, self.ch_y.local)
        peer_fence(self.token, self.group)  # every rank's results have arrived
        out = _combine(self.ch_y.local[:T * k], inv_sort_idx, weights)
        return out, router_logits
