"""Sizing of the packed paged KV pool: how many vLLM blocks fit a memory budget when every owner layer stores its own
packed format but all owners share one block-ID space.

Follows the arithmetic of the reference's cache hooks without vLLM
(plugins/residual_quantization/src/residual_quantization/install_cache.py:38-84, `mixed_cache_config`): one logical
block costs the sum of every owner's page (packed owners: 2 planes x heads x block_size x page_width bytes; native
bf16 owners: 2 x heads x block_size x head_dim x 2 bytes), the pool holds `budget // bytes_per_block` blocks, and it
must hold more than one full-length sequence (`ceil(max_model_len / block_size)`) because block 0 is the null block.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

HBM_BYTES_B200 = 180 * 10**9


def page_width(records: Sequence[Sequence[int]], head_dim: int) -> int:
    """Bytes per token of one (head, plane): packed codes + FP8 scale and offset per group + bf16 alpha per record
    (install_model.py:34-38; csrc/common/cache.cuh:14-17)."""
    width = 0
    for bits, group in records:
        if bits not in (2, 4) or group not in (16, 32) or head_dim % group:
            raise ValueError(f"unsupported record [{bits}, {group}] for head_dim {head_dim}")
        width += head_dim * bits // 8 + 2 * (head_dim // group) + 2
    return width


@dataclass(frozen=True)
class OwnerSpec:
    """One KV owner (a layer slot that has its own cache tensor)."""

    heads: int
    head_dim: int
    block_size: int
    records: Optional[Tuple[Tuple[int, int], ...]] = None   # None = native bf16 KV

    @property
    def page_bytes(self) -> int:
        """Bytes of one block of this owner, both planes (vLLM's `page_size_bytes`)."""
        per_token = page_width(self.records, self.head_dim) if self.records is not None else 2 * self.head_dim
        return 2 * self.heads * self.block_size * per_token

    def cache_shape(self, num_blocks: int) -> Tuple[int, ...]:
        if self.records is None:
            return (2, num_blocks, self.block_size, self.heads, self.head_dim)
        return (2, num_blocks, self.heads, self.block_size, page_width(self.records, self.head_dim))


@dataclass(frozen=True)
class CachePlan:
    num_blocks: int
    bytes_per_block: int
    owner_bytes: Dict[str, int]      # size of every owner's cache tensor
    tokens: int                      # cached tokens the pool can hold (the null block excluded)

    @property
    def total_bytes(self) -> int:
        return sum(self.owner_bytes.values())


def plan_cache(owners: Dict[str, OwnerSpec], budget_bytes: int, max_model_len: int) -> CachePlan:
    """Blocks that fit `budget_bytes` when every owner in `owners` gets one page per block."""
    if not owners:
        raise ValueError("no KV owners")
    block_sizes = {spec.block_size for spec in owners.values()}
    if len(block_sizes) != 1:
        raise ValueError("Group token block sizes differ")
    block_size = block_sizes.pop()
    bytes_per_block = sum(spec.page_bytes for spec in owners.values())
    num_blocks = budget_bytes // bytes_per_block
    required = (max_model_len + block_size - 1) // block_size
    if num_blocks <= required:
        raise ValueError("Layer buffers cannot hold max_model_len plus the null block")
    return CachePlan(num_blocks, bytes_per_block, {name: num_blocks * spec.page_bytes for name, spec in owners.items()},
                     (num_blocks - 1) * block_size)


def looped_model_owners(layers: int, groups_per_layer: int, records, heads: int, head_dim: int,
                        block_size: int = 16) -> Dict[str, OwnerSpec]:
    """Owners of a looped decoder: every (layer, KV group) has one packed cache shared by the loops of the group."""
    records = tuple(tuple(int(v) for v in r) for r in records)
    return {f"layers.{layer}.group.{group}": OwnerSpec(heads, head_dim, block_size, records)
            for layer in range(layers) for group in range(groups_per_layer)}


def kv_footprint(packed_groups, layers: int, loops: int, heads: int, head_dim: int) -> int:
    """Bytes of KV per cached token of the whole model: the reference's capacity experiment compares this figure
    between configurations (experiments/kv_memory_latency/capacity.py:33-51).  An empty `packed_groups` means native
    bf16 KV for every (layer, loop): 2 planes x layers x loops x heads x head_dim x 2 bytes.  Otherwise the groups'
    records, in loop order, must cover every loop exactly once; every physical layer stores one packed row of
    `page_width` bytes per head and plane for each group."""
    if not packed_groups:
        return 2 * layers * loops * heads * head_dim * 2
    records = [tuple(record) for group in packed_groups for record in group]
    if len(records) != loops:
        raise ValueError("Invalid precision schedule or quantization group size")
    try:
        stride = page_width(records, head_dim)
    except ValueError:
        raise ValueError("Invalid precision schedule or quantization group size") from None
    return 2 * layers * heads * stride


def sequences_that_fit(budget_bytes: int, context: int, bytes_per_token: int, block_size: int = 16) -> int:
    """Whole sequences of `context` tokens a KV budget holds when memory comes in blocks of `block_size` tokens and one
    block stays reserved as the null block."""
    blocks_per_sequence = (context + block_size - 1) // block_size
    blocks = budget_bytes // (bytes_per_token * block_size)
    return max(0, (blocks - 1) // blocks_per_sequence)
