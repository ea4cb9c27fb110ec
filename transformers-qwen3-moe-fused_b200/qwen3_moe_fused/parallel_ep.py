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

from dataclasses import dataclass
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
