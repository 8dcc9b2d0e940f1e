"""Multi-GPU layer: one process per GPU, work sharded by whole segments.

Segmented operations need no communication at all: rank r owns the contiguous
segments ``shard_range(num_segments, r, world)`` and keeps its outputs.  The
full reduction and the full scan add ONE collective: an all-gather of one
double per rank (the per-shard totals).  The reference is single-GPU
(src/init/cuda.cpp:45 selects one device), so this layer has no counterpart
there.

The gather step is a parameter so that the host logic can be exercised on CPU
with the ``gloo`` backend: ``local_total`` / ``local_scan`` are callables that
run the device kernels in production and a CPU stand-in in the CPU tests.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_range(num_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced split of ``num_units`` whole units (segments or
    16-element groups) over ``world`` ranks: [begin, end) of rank ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    return num_units * rank // world, num_units * (rank + 1) // world


def gather_totals(local_total: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather one float64 per rank; returns float64[world] on the same device."""
    if local_total.dtype != torch.float64 or local_total.numel() != 1:
        raise TypeError("local_total must be a float64 tensor with one element")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local_total.reshape(1).clone()
    out = torch.empty(world, dtype=torch.float64, device=local_total.device)
    dist.all_gather_into_tensor(out, local_total.reshape(1), group=group)
    return out


def sharded_full_reduce(local_total_fn: Callable[[], torch.Tensor], group=None) -> torch.Tensor:
    """Each rank reduces its shard to one float64, the totals are gathered and
    every rank adds them in rank order (same result everywhere).  Returns a
    float64[1] tensor holding the global sum."""
    totals = gather_totals(local_total_fn(), group)
    return totals.sum(dtype=torch.float64).reshape(1)


def sharded_full_scan(local_total_fn: Callable[[], torch.Tensor],
                      local_scan_fn: Callable[[torch.Tensor, int], torch.Tensor],
                      group=None) -> torch.Tensor:
    """Full inclusive scan of an array sharded contiguously over the ranks.

    ``local_total_fn()`` -> float64[1]: sum of this rank's shard.
    ``local_scan_fn(totals, rank)`` -> the shard's scan seeded with the sum of
    ``totals[:rank]`` (the device kernel adds that carry itself, inside its
    first tile; no extra pass over the output).
    """
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    totals = gather_totals(local_total_fn(), group)
    return local_scan_fn(totals, rank)
