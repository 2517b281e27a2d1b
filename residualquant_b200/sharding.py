"""How the hot path spreads over the GPUs of one node (one process per GPU, `torch.distributed`).

Both operators are independent per (sequence, head) -- the reference's CTAs never reduce across either
(quantize/launch.cuh:32, attention/launch.cuh:112-113) -- so there are two partitionings:

* by SEQUENCES (the default): every rank owns a slice of the batch with its own page pool and block tables; there is no
  data-path collective at all.
* by KV HEADS (for a model whose single sequence batch must be split, e.g. 55 heads over 8 GPUs): every rank holds all
  sequences but only its heads of the cache; after attention one all-gather of `[rows, local_heads, head_dim]`
  rebuilds the full `[rows, heads, head_dim]` that the output projection consumes.  Head counts may be uneven
  (55 = 7*7 + 6), so slices are padded to the largest count for the collective.

Timing helpers follow the benchmark contract: barrier on both sides, maximum over ranks.
"""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_counts(total: int, world: int) -> List[int]:
    """Sizes of `world` contiguous shards of `total` items, differing by at most one, larger shards first."""
    if world < 1 or total < 0:
        raise ValueError("world must be positive and total non-negative")
    base, extra = divmod(total, world)
    return [base + (1 if rank < extra else 0) for rank in range(world)]


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of `rank`'s shard."""
    if not 0 <= rank < world:
        raise ValueError("rank outside the world")
    counts = shard_counts(total, world)
    begin = sum(counts[:rank])
    return begin, begin + counts[rank]


def is_distributed() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def max_over_ranks(value: float, device) -> float:
    """The slowest rank's value (a duration measured with CUDA events on every rank)."""
    if not is_distributed():
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_heads(local: torch.Tensor, heads: int) -> torch.Tensor:
    """All-gather head-sharded attention outputs.

    local: `[rows, local_heads, head_dim]` of this rank, where local_heads = shard_counts(heads, world)[rank].
    Returns `[rows, heads, head_dim]` on every rank, heads in rank order.
    """
    if not is_distributed():
        if local.size(1) != heads:
            raise ValueError("a single rank must hold every head")
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    counts = shard_counts(heads, world)
    if local.size(1) != counts[rank]:
        raise ValueError(f"rank {rank} holds {local.size(1)} heads, expected {counts[rank]}")
    widest = max(counts)
    rows, _, dim = local.shape
    padded = local
    if counts[rank] < widest:
        padded = torch.zeros(rows, widest, dim, dtype=local.dtype, device=local.device)
        padded[:, : counts[rank]] = local
    flat = torch.empty(world * rows, widest, dim, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, padded.contiguous())   # rank-major concatenation along dim 0
    gathered = flat.view(world, rows, widest, dim)
    return torch.cat([gathered[r, :, : counts[r]] for r in range(world)], dim=1)
