"""Partitioning of events (and heads) across the GPUs of one box.

The path has no exchange step: every kernel grid has an independent (sequence, head) axis
(e.g. models/hattention/chunk_delta_h.py:58-59 in the reference), so ranks work on disjoint
events or head slices.  This module holds the host-side plan; collectives are only used to
agree on it or, optionally, to gather results.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def lpt_assign(costs: Sequence[int], n_ranks: int) -> List[List[int]]:
    """Greedy longest-processing-time assignment of events to ranks by cost (hit count).

    Returns, per rank, the event indices it owns (in input order).  Deterministic: ties go to the
    lower event index, then to the lower rank.
    """
    if n_ranks <= 0:
        raise ValueError("n_ranks must be positive")
    order = sorted(range(len(costs)), key=lambda i: (-int(costs[i]), i))
    load = [0] * n_ranks
    owned: List[List[int]] = [[] for _ in range(n_ranks)]
    for i in order:
        r = min(range(n_ranks), key=lambda j: (load[j], j))
        owned[r].append(i)
        load[r] += int(costs[i])
    return [sorted(o) for o in owned]


def head_slice(n_heads: int, rank: int, n_ranks: int) -> Tuple[int, int]:
    """Contiguous head range [h0, h1) of `rank` when a single event is split by head."""
    if n_heads % n_ranks:
        raise ValueError(f"{n_heads} heads do not split evenly over {n_ranks} ranks")
    per = n_heads // n_ranks
    return rank * per, (rank + 1) * per


def pack_events(lengths: Sequence[int], owned: Sequence[int]) -> Tuple[torch.Tensor, List[Tuple[int, int]]]:
    """cu_seqlens (int64 [n+1]) of the events a rank owns, packed back to back, and for each owned
    event its (start, end) row range in the global, event-ordered concatenation."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + int(n))
    cu = [0]
    spans = []
    for e in owned:
        cu.append(cu[-1] + int(lengths[e]))
        spans.append((starts[e], starts[e + 1]))
    return torch.tensor(cu, dtype=torch.int64), spans


def imbalance(lengths: Sequence[int], plan: Sequence[Sequence[int]]) -> float:
    """max / mean of per-rank total cost: the only loss term of event sharding."""
    loads = [sum(int(lengths[e]) for e in o) for o in plan]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


def agree_on_plan(lengths: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> List[List[int]]:
    """Every rank computes the same plan from rank 0's event lengths (one small broadcast)."""
    world = dist.get_world_size(group)
    t = lengths.clone()
    dist.broadcast(t, src=0, group=group)
    return lpt_assign(t.tolist(), world)


def gather_event_outputs(local: torch.Tensor, lengths: Sequence[int], plan: Sequence[Sequence[int]],
                         group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather ragged per-event outputs ([rows_owned, D] per rank) into the global event order.

    Pads every rank's block to the largest block so that one all_gather suffices (NCCL or gloo),
    then copies each event's rows to its position.  The only collective of the path.
    """
    world = dist.get_world_size(group)
    rows = [sum(int(lengths[e]) for e in o) for o in plan]
    width = local.shape[1]
    pad = max(rows)
    buf = local.new_zeros(pad, width)
    buf[: local.shape[0]] = local
    if local.is_cuda:
        parts = local.new_empty(world, pad, width)
        dist.all_gather_into_tensor(parts, buf, group=group)
    else:
        parts = [torch.empty_like(buf) for _ in range(world)]
        dist.all_gather(parts, buf, group=group)
    total = sum(int(n) for n in lengths)
    out = local.new_empty(total, width)
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + int(n))
    for r, owned in enumerate(plan):
        pos = 0
        for e in owned:
            n = int(lengths[e])
            out[starts[e]: starts[e] + n] = parts[r][pos: pos + n]
            pos += n
    return out


def shard_events(rows: torch.Tensor, lengths: Sequence[int], owned: Sequence[int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """The rows of the events a rank owns, packed back to back, and their cu_seqlens (int64, host).

    `rows` holds all events in event order ([sum(lengths), D], host or device)."""
    cu, spans = pack_events(lengths, owned)
    local = torch.cat([rows[s:e] for s, e in spans]) if spans else rows[:0]
    return local, cu


def gather_heads(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather the head slices of one event into the full head dimension.

    `local` is [..., H / world, V] (the heads head_slice() gave this rank, in rank order); returns [..., H, V].
    One collective, no arithmetic: the counterpart of gather_event_outputs when a single large event is split by
    head instead of a batch of events by event."""
    world = dist.get_world_size(group)
    local = local.contiguous()
    if local.is_cuda:
        parts = local.new_empty((world,) + tuple(local.shape))
        dist.all_gather_into_tensor(parts, local, group=group)
    else:
        chunks = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(chunks, local, group=group)
        parts = torch.stack(chunks)
    nd = local.dim()
    # [world, ..., h, V] -> [..., world, h, V] -> [..., world * h, V]
    perm = list(range(1, nd - 1)) + [0, nd - 1, nd]
    out = parts.permute(*perm)
    return out.reshape(tuple(local.shape[:-2]) + (world * local.shape[-2], local.shape[-1]))
