"""Partitioning of a stick-breaking attention call across the GPUs of one node.

Every (head, sequence) pair is independent in the forward and in the backward pass, so a call is
split with no exchange step: each rank runs the ordinary operator on its slice.  Collectives are
used only afterwards, to gather results for verification (``all_gather_tokens`` / ``all_gather_heads``).

Partition plans work on Python lists of sequence lengths (the caller knows them when it packs the
batch) and never touch device memory.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

__all__ = ["head_range", "contiguous_segments", "lpt_assignment", "slice_packed", "all_gather_tokens",
           "all_gather_heads", "imbalance"]


def head_range(num_heads: int, world: int, rank: int) -> Tuple[int, int]:
    """Heads ``[h0, h1)`` of ``rank``; the first ``num_heads % world`` ranks take one extra head."""
    base, extra = divmod(num_heads, world)
    h0 = rank * base + min(rank, extra)
    return h0, h0 + base + (1 if rank < extra else 0)


def _cost(n: int, by: str) -> float:
    return float(n) if by == "tokens" else float(n) * float(n)


def contiguous_segments(lengths: Sequence[int], world: int, by: str = "tokens") -> List[Tuple[int, int]]:
    """Splits the sequence list into ``world`` contiguous runs ``[s0, s1)`` whose cost (``"tokens"``:
    sum of L, ``"work"``: sum of L^2) is as even as a greedy sweep gets it: a run is closed as soon as
    adding the next sequence would move its total further from the ideal share than stopping does.
    Runs may be empty when there are fewer sequences than ranks."""
    costs = [_cost(n, by) for n in lengths]
    total = sum(costs)
    out, start, acc, done = [], 0, 0.0, 0.0
    for r in range(world):
        remaining_ranks = world - r
        target = (total - done) / remaining_ranks
        end = start
        acc = 0.0
        while end < len(costs):
            if r == world - 1:
                acc += costs[end]; end += 1
                continue
            if acc > 0 and abs(acc + costs[end] - target) > abs(acc - target):
                break
            acc += costs[end]; end += 1
            if acc >= target:
                break
        out.append((start, end))
        done += acc
        start = end
    return out


def lpt_assignment(lengths: Sequence[int], world: int, by: str = "work") -> List[List[int]]:
    """Longest-processing-time-first assignment of whole sequences to ranks (not contiguous):
    returns, per rank, the sorted indices of its sequences."""
    loads = [0.0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(lengths)), key=lambda i: -_cost(lengths[i], by)):
        r = min(range(world), key=lambda j: loads[j])
        loads[r] += _cost(lengths[idx], by)
        owned[r].append(idx)
    return [sorted(x) for x in owned]


def imbalance(lengths: Sequence[int], parts: Sequence[Sequence[int]], by: str = "work") -> float:
    """max over ranks of the cost / mean cost (1.0 = perfectly balanced)."""
    loads = [sum(_cost(lengths[i], by) for i in part) for part in parts]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


def slice_packed(tensors: Sequence[torch.Tensor], lengths: Sequence[int], seq_ids: Sequence[int]):
    """Takes the sequences ``seq_ids`` out of packed ``(H, T, ...)`` tensors.

    Returns ``(sliced tensors, lengths of the slice, token index)`` where ``token index`` are the
    positions of the slice's tokens in the full packing (to scatter results back)."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + int(n))
    if len(seq_ids) and list(seq_ids) == list(range(seq_ids[0], seq_ids[-1] + 1)):
        a, b = starts[seq_ids[0]], starts[seq_ids[-1] + 1]
        index = torch.arange(a, b)
        sliced = [t[:, a:b] for t in tensors]
    else:
        index = torch.cat([torch.arange(starts[i], starts[i + 1]) for i in seq_ids]) if len(seq_ids) \
            else torch.zeros(0, dtype=torch.long)
        sliced = [t.index_select(1, index.to(t.device)) for t in tensors]
    return sliced, [int(lengths[i]) for i in seq_ids], index


def all_gather_tokens(local: torch.Tensor, index: torch.Tensor, total_tokens: int, group=None) -> torch.Tensor:
    """Verification only: rebuilds the full ``(H, T, ...)`` tensor from per-rank token slices."""
    world = dist.get_world_size(group)
    counts = [torch.zeros(1, dtype=torch.long, device=local.device) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([local.shape[1]], dtype=torch.long, device=local.device), group=group)
    most = int(max(c.item() for c in counts))
    pad_shape = (local.shape[0], most, *local.shape[2:])
    padded = local.new_zeros(pad_shape)
    padded[:, : local.shape[1]] = local
    idx_pad = torch.full((most,), -1, dtype=torch.long, device=local.device)
    idx_pad[: index.numel()] = index.to(local.device)
    parts = [torch.empty_like(padded) for _ in range(world)]
    idxs = [torch.empty_like(idx_pad) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    dist.all_gather(idxs, idx_pad, group=group)
    full = local.new_zeros((local.shape[0], total_tokens, *local.shape[2:]))
    for part, idx, cnt in zip(parts, idxs, counts):
        n = int(cnt.item())
        if n:
            full[:, idx[:n]] = part[:, :n]
    return full


def all_gather_heads(local: torch.Tensor, num_heads: int, group=None) -> torch.Tensor:
    """Verification only: concatenates per-rank head slices (``head_range`` order) along axis 0."""
    world = dist.get_world_size(group)
    most = -(-num_heads // world)
    padded = local.new_zeros((most, *local.shape[1:]))
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    out = []
    for r, part in enumerate(parts):
        h0, h1 = head_range(num_heads, world, r)
        out.append(part[: h1 - h0])
    return torch.cat(out, 0)
