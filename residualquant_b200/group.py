"""Host-side mirror of the reference's per-group state and of the decode branch of its attention hook.

`DeferredKVGroup` follows plugins/residual_quantization/src/residual_quantization/install_model.py:17-52: the K/V of
the loops of a KV group are held back (cloned) until the group's last loop arrives, then all records go to
`quantize` in one call.  `PackedDecodeAttention` follows the decode path of `PackedImpl.forward` and `_store_kv`
(packed_backend.py:28-137): attention over the packed cache plus the live token, then stage/quantize.
`batch_slices` follows the metadata builder's split of a reordered batch into its decode prefix and its
full-prompt suffix (`PackedBuilder.build`, packed_backend.py:153-199), and `PackedAttention` runs both parts: decode
rows through the packed kernel, full prompts through a caller-supplied prefill attention (the reference calls
flash-attn there, outside the two hot paths), then stages and quantizes the new K/V of the whole batch.  Nothing here
touches vLLM; a vLLM attention backend only has to forward its `forward(...)` arguments.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from . import _cuda


class DeferredKVGroup:
    """Owns the packed format of one KV group and keeps raw K/V until every loop of the group has been seen."""

    def __init__(self, records: Sequence[Sequence[int]], page_tokens: int, reference_mode: str = "anchor",
                 anchor_index: Optional[int] = None, coefficient_method: str = "ls", prefill_offload=None):
        self.records = tuple(tuple(int(v) for v in r) for r in records)
        if not self.records:
            raise ValueError("Every packed group must contain at least one record")
        if reference_mode not in ("adjacent", "anchor"):
            raise ValueError("Unsupported reference")
        self.anchor_index = len(self.records) - 1 if anchor_index is None else int(anchor_index)
        if reference_mode == "adjacent" and self.anchor_index != 0:
            raise ValueError("Adjacent reference currently requires anchor_index=0")
        if coefficient_method not in ("unit", "norm", "ls"):
            raise ValueError("Unsupported coefficient method")
        self.page_tokens = int(page_tokens)
        self.reference_mode = reference_mode
        self.coefficient_method = coefficient_method
        self.pending: List[Tuple[torch.Tensor, torch.Tensor]] = []
        # optional prefill_offload.PrefillHostStage: non-final loops of a prompt are parked in pinned host memory
        self.prefill_offload = prefill_offload
        self.host_buffers: List[Optional[torch.Tensor]] = [None] * (len(self.records) - 1)

    def page_width(self, head_dim: int) -> int:
        """Bytes per token of one (head, plane): codes + FP8 scale/offset per group + bf16 alpha, over all records
        (install_model.py:34-38)."""
        code_bytes = head_dim * sum(bits for bits, _ in self.records) // 8
        metadata_bytes = 2 * sum(head_dim // group for _, group in self.records)
        return code_bytes + metadata_bytes + 2 * len(self.records)

    def cache_shape(self, num_blocks: int, num_kv_heads: int, head_dim: int) -> Tuple[int, int, int, int, int]:
        """(2, blocks, heads, block_size, page_width), the reference's PackedBackend.get_kv_cache_shape
        (packed_backend.py:222-223)."""
        return (2, num_blocks, num_kv_heads, self.page_tokens, self.page_width(head_dim))

    def stage(self, key: torch.Tensor, value: torch.Tensor, offload: bool = False):
        """Non-final loops: keep a copy (on the device, or in pinned host memory with `offload`), return None.  Final
        loop: return every (K, V) pair in loop order and reset.  The completing call borrows its input, so a
        one-record group never copies."""
        if len(self.pending) + 1 == len(self.records):
            records = self.pending + [(key, value)]
            self.pending = []
            return records
        if offload:
            index = len(self.pending)
            buffer = self.prefill_offload.store(key, value, self.host_buffers[index])
            self.host_buffers[index] = buffer
            self.pending.append((buffer[0, : key.size(0)], buffer[1, : value.size(0)]))
        else:
            self.pending.append((key.clone(), value.clone()))
        return None


class PackedDecodeAttention:
    """One attention slot (loop `group_loop_index` of a group) of a looped decoder, decode path only."""

    def __init__(self, group: DeferredKVGroup, group_loop_index: int, key_rotation=None, value_rotation=None,
                 key_mean: Optional[torch.Tensor] = None):
        if not 0 <= group_loop_index < len(group.records):
            raise ValueError("loop index outside the group")
        self.packed_group = group
        self.group_loop_index = group_loop_index
        self.key_rotation = key_rotation
        self.value_rotation = value_rotation
        self.key_mean = key_mean

    def forward(self, query, key, value, kv_cache, query_start_loc, seq_lens, block_table, slot_mapping, output):
        """query/key/value/output: bf16 [tokens, heads, head_dim]; writes `output` in place and returns it."""
        if output is None:
            raise ValueError("BF16 output required")
        group = self.packed_group
        records = [list(r) for r in group.records]
        _cuda.attention(query, key, value, kv_cache, output, query_start_loc, seq_lens, block_table,
                        self.key_rotation, self.value_rotation, self.key_mean, records, group.reference_mode,
                        group.anchor_index, self.group_loop_index)
        actual = slot_mapping.numel()
        staged = group.stage(key[:actual], value[:actual])
        if staged is not None:
            _cuda.quantize(staged, kv_cache, slot_mapping, self.key_rotation, self.value_rotation, self.key_mean,
                           records, group.reference_mode, group.anchor_index, group.coefficient_method)
        return output


@dataclass(frozen=True)
class BatchSlice:
    """A run of requests of one kind inside a batch whose one-token requests come first."""

    first_request: int
    last_request: int     # exclusive
    first_token: int
    last_token: int       # exclusive
    decode: bool          # True: one query token per request; False: full prompts


def batch_slices(query_start_loc: Sequence[int], seq_lens: Sequence[int]) -> List[BatchSlice]:
    """Split a batch into its decode prefix and its full-prompt suffix.

    query_start_loc: host copy of the cumulative query lengths [requests + 1]; seq_lens: host copy [requests].
    The caller (vLLM's model runner with `reorder_batch_threshold = 1`) has put the one-token requests first.
    A request with more than one query token must be a whole prompt (query length == sequence length): chunked or
    recomputed partial prefill is rejected, as in the reference (packed_backend.py:175-178).
    """
    starts = [int(v) for v in query_start_loc]
    requests = len(starts) - 1
    if requests < 0 or len(seq_lens) < requests:
        raise ValueError("query_start_loc needs one entry per request plus the final boundary")
    first_prompt = None
    for request in range(requests):
        length = starts[request + 1] - starts[request]
        if length > 1:
            if length != int(seq_lens[request]):
                raise ValueError("Chunked/recomputed partial prefill is unsupported")
            if first_prompt is None:
                first_prompt = request
        elif first_prompt is not None and length == 1:
            raise ValueError("one-token requests must precede the prompts (reorder the batch)")
    if first_prompt is None:
        return [BatchSlice(0, requests, 0, starts[-1], True)] if requests else []
    slices = []
    if first_prompt > 0:
        slices.append(BatchSlice(0, first_prompt, 0, starts[first_prompt], True))
    slices.append(BatchSlice(first_prompt, requests, starts[first_prompt], starts[-1], False))
    return slices


def causal_prefill(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, output: torch.Tensor,
                   query_start_loc: Sequence[int]) -> None:
    """Full-prompt causal attention over the raw bf16 K/V of each prompt (plain PyTorch; any varlen attention kernel
    with the same contract can be passed to `PackedAttention` instead)."""
    starts = [int(v) for v in query_start_loc]
    for begin, end in zip(starts, starts[1:]):
        q = query[begin:end].transpose(0, 1).unsqueeze(0)
        k = key[begin:end].transpose(0, 1).unsqueeze(0)
        v = value[begin:end].transpose(0, 1).unsqueeze(0)
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
        output[begin:end].copy_(out.squeeze(0).transpose(0, 1))


class PackedAttention(PackedDecodeAttention):
    """Decode and full-prompt requests of one batch, then the KV write of the whole batch."""

    def __init__(self, *args, prefill: Callable = causal_prefill, **kwargs):
        super().__init__(*args, **kwargs)
        self.prefill = prefill

    def forward_batch(self, query, key, value, kv_cache, query_start_loc, seq_lens, block_table, slot_mapping, output,
                      query_start_loc_host: Sequence[int], seq_lens_host: Sequence[int]):
        """Device tensors as in `forward`; the host copies drive the split (the decode-only case needs none of their
        values beyond the request count, so graph replays may pass stale ones of the right length)."""
        if output is None:
            raise ValueError("BF16 output required")
        group = self.packed_group
        records = [list(r) for r in group.records]
        for part in batch_slices(query_start_loc_host, seq_lens_host):
            tokens = slice(part.first_token, part.last_token)
            if part.decode:
                rows = slice(part.first_request, part.last_request)
                starts = query_start_loc[part.first_request:part.last_request + 1]
                _cuda.attention(query[tokens], key[tokens], value[tokens], kv_cache, output[tokens], starts.contiguous(),
                                seq_lens[rows].contiguous(), block_table[rows], self.key_rotation, self.value_rotation,
                                self.key_mean, records, group.reference_mode, group.anchor_index, self.group_loop_index)
            else:
                base = int(query_start_loc_host[part.first_request])
                local = [int(v) - base for v in query_start_loc_host[part.first_request:part.last_request + 1]]
                self.prefill(query[tokens], key[tokens], value[tokens], output[tokens], local)
        actual = slot_mapping.numel()
        # prompts in the batch and a host stage on the group: park the held-back loops in pinned memory and bring them
        # back chunk by chunk for the write (packed_backend.py:45-52, 101-137)
        offload = group.prefill_offload is not None and any(
            int(b) - int(a) > 1 for a, b in zip(query_start_loc_host, query_start_loc_host[1:]))
        staged = group.stage(key[:actual], value[:actual], offload=offload)
        if staged is not None:
            parts = group.prefill_offload.chunks(staged, slot_mapping) if offload and len(staged) > 1 else ((staged, slot_mapping),)
            for chunk_records, chunk_slots in parts:
                _cuda.quantize(chunk_records, kv_cache, chunk_slots, self.key_rotation, self.value_rotation, self.key_mean,
                               records, group.reference_mode, group.anchor_index, group.coefficient_method)
        return output
