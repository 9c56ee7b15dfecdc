"""Host-side partitioning of the two matmuls over the GPUs of one box (one process per GPU).

* W8A8: the weight matrix ``B [N, K]`` (with its per-channel scale and bias) is split into ``world`` column
  blocks of the output; every rank holds all of ``A``.  After the local matmul an all-gather of the
  ``[M, N/world]`` blocks reassembles ``C``; :func:`interleave_column_blocks` turns the gathered
  ``[world, M, N/world]`` buffer into the row-major ``[M, N]`` result.
* MX-FP4 grouped matmul: whole groups go to ranks, largest first onto the least loaded rank (LPT), because group
  sizes are uneven; each rank computes the rows of its groups and :func:`scatter_group_rows` puts the gathered
  row blocks back in the original order.

Only ``torch.distributed`` collectives are used, so the same code runs on NCCL (GPU) and gloo (CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch


def column_shard(N: int, world: int, rank: int):
    """(first column, column count) of rank's block; N must divide evenly so that the gather is regular."""
    if N % world:
        raise ValueError(f"N={N} is not divisible by the number of ranks {world}")
    nl = N // world
    return rank * nl, nl


def all_gather_blocks(local: torch.Tensor, world: int, out: torch.Tensor = None) -> torch.Tensor:
    """All-gather equally shaped 2-D blocks; returns [world, rows, cols] (rank-major).  ``out`` may hold a
    preallocated [world*rows, cols] buffer."""
    import torch.distributed as dist
    rows, cols = local.shape
    if out is None:
        out = torch.empty((world * rows, cols), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local)
    return out.view(world, rows, cols)


def interleave_column_blocks(gathered: torch.Tensor) -> torch.Tensor:
    """[world, M, nl] (rank-major all-gather result) -> [M, world*nl] row-major."""
    world, M, nl = gathered.shape
    return gathered.permute(1, 0, 2).reshape(M, world * nl)


@dataclass
class GroupPlan:
    owner: List[int]              # rank that computes group g
    groups_of: List[List[int]]    # per rank: its groups in ascending order
    rows_of: List[int]            # per rank: total rows
    max_rows: int                 # padding target of the gather


def assign_groups_lpt(group_rows: Sequence[int], world: int) -> GroupPlan:
    """Longest-processing-time-first assignment of groups to ranks."""
    order = sorted(range(len(group_rows)), key=lambda g: (-int(group_rows[g]), g))
    load = [0] * world
    owner = [0] * len(group_rows)
    for g in order:
        r = min(range(world), key=lambda i: (load[i], i))
        owner[g] = r
        load[r] += int(group_rows[g])
    groups_of = [[g for g in range(len(group_rows)) if owner[g] == r] for r in range(world)]
    return GroupPlan(owner, groups_of, load, max(load) if load else 0)


def local_row_index(group_rows: Sequence[int], groups: Sequence[int]) -> torch.Tensor:
    """Global row numbers of the rows a rank owns, in the order it stores them (its groups back to back)."""
    starts = [0]
    for v in group_rows:
        starts.append(starts[-1] + int(v))
    parts = [torch.arange(starts[g], starts[g + 1]) for g in groups]
    return torch.cat(parts) if parts else torch.zeros(0, dtype=torch.long)


def scatter_group_rows(gathered: torch.Tensor, plan: GroupPlan, group_rows: Sequence[int]) -> torch.Tensor:
    """[world, max_rows, N] padded per-rank results -> [sum(group_rows), N] in the original row order."""
    world, _, N = gathered.shape
    out = torch.empty((sum(int(v) for v in group_rows), N), dtype=gathered.dtype, device=gathered.device)
    for r in range(world):
        idx = local_row_index(group_rows, plan.groups_of[r]).to(gathered.device)
        out.index_copy_(0, idx, gathered[r, :idx.numel()])
    return out
