"""Partitioning of the decode path over the GPUs of one node (one process per GPU).

Attention over the compressed cache needs no collective: arenas are independent per (sequence,
KV head).  Two partitions are offered:

* by sequence (default): rank r owns a contiguous block of sequences with all their layers and heads;
* by KV head (a single long sequence, or tensor parallelism): rank r owns a contiguous block of KV
  heads with the query heads that share them; its attention output is the matching column block of
  ``[B, Hq*D]`` and feeds a row-parallel ``o_proj`` whose partial products are summed with one
  all-reduce (``row_parallel_linear``), the only communication step.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def block_range(n_items: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced block of ``n_items`` for ``rank`` (sizes differ by at most one)."""
    if not 0 <= rank < world_size:
        raise ValueError("rank out of range")
    base, rem = divmod(n_items, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_sequences(n_sequences: int, world_size: int, rank: int) -> Tuple[int, int]:
    return block_range(n_sequences, world_size, rank)


def balanced_sequence_partition(lengths, world_size: int):
    """Token-balanced assignment of ragged sequences to ranks: longest first, each to the rank with the fewest
    tokens so far (ties to the lower rank).  Returns one ascending index list per rank; every rank computes the
    same partition from the same lengths, so nothing is communicated."""
    if world_size < 1:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world_size
    parts = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        parts[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(p) for p in parts]


def shard_kv_heads(n_kv_heads: int, n_q_heads: int, world_size: int, rank: int):
    """Returns ((kv_lo, kv_hi), (q_lo, q_hi)): the rank's KV heads and the query heads that use them."""
    if n_kv_heads % world_size != 0:
        raise ValueError("the KV heads must divide evenly over the ranks")
    group = n_q_heads // n_kv_heads
    lo, hi = block_range(n_kv_heads, world_size, rank)
    return (lo, hi), (lo * group, hi * group)


def row_parallel_linear(x_local: torch.Tensor, weight_shard: torch.Tensor,
                        group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """y = sum_r x_r @ W_r^T with W split along its input columns; one all-reduce (NCCL on GPUs)."""
    y = x_local @ weight_shard.T
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
    return y


def max_over_ranks(value_ms: float, device) -> float:
    """Timing convention for multi-GPU numbers: the slowest rank's device time."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value_ms
    t = torch.tensor([value_ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
