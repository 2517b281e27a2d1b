"""Host staging of raw K/V during a long prefill.

The K/V of a group's non-final loops have to be kept until the last loop arrives (`group.DeferredKVGroup`).  For a long
prompt that is `(records - 1) x 2 x tokens x heads x head_dim` bf16 values per (layer, group); the reference can park
them in pinned host memory and bring them back for the group's quantize
(plugins/residual_quantization/src/residual_quantization/prefill_offload.py:10-200).  `PrefillHostStage` offers the same
service through the same five calls (`reserve`, `store`, `preload`, `prepare`, `chunks`) so that an attention hook
written for the reference works with it, built from two small mechanisms:

  * `_DoubleBuffer`: the rows of one group come back `chunk_tokens` at a time through two device buffers; while the
    quantizer consumes one, the copy stream fills the other.
  * `_LayerRing` (optional look-ahead): whole layers' worth of parked rows are copied back AHEAD of their use.  The
    groups of the physical layers form a chain in execution order; while layer i quantizes, the rows of layers
    i+1 .. i+slots-1 are already on their way into the ring's device slots, so the completing loop of a layer finds its
    rows resident and writes them in a single quantize call.

All copies run on side streams and are ordered against the compute stream with events only; nothing synchronizes the
host.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import torch

Pair = Tuple[torch.Tensor, torch.Tensor]

# look-ahead ring: between 2 and 8 layers in flight, about 800 MiB of device memory (the reference's bounds,
# prefill_offload.py:5-7)
MIN_RING_LAYERS, MAX_RING_LAYERS, RING_TARGET_BYTES = 2, 8, 800 * 1024 ** 2


def ring_slots_for(tokens: int, pending_records: int, heads: int, head_dim: int, itemsize: int = 2) -> int:
    """How many layers the look-ahead ring holds for prompts of `tokens` tokens."""
    layer_bytes = max(1, pending_records * 2 * tokens * heads * head_dim * itemsize)
    return max(MIN_RING_LAYERS, min(MAX_RING_LAYERS, RING_TARGET_BYTES // layer_bytes))


@dataclass
class _Slot:
    """One device buffer with the two events that hand it back and forth between a copy stream and the compute stream."""

    filled: torch.cuda.Event = field(default_factory=torch.cuda.Event)
    drained: torch.cuda.Event = field(default_factory=torch.cuda.Event)
    in_use: bool = False

    def wait_until_drained(self, stream: torch.cuda.Stream) -> None:
        if self.in_use:
            stream.wait_event(self.drained)

    def mark_drained(self, stream: torch.cuda.Stream) -> None:
        self.drained.record(stream)
        self.in_use = True


class _DoubleBuffer:
    """Two chunk-sized device buffers [slot][record][K|V][chunk][heads][head_dim]."""

    def __init__(self, chunk_tokens: int):
        self.chunk_tokens = chunk_tokens
        self.buffers: Optional[torch.Tensor] = None

    def ensure(self, records: int, heads: int, head_dim: int, dtype, device) -> None:
        shape = (2, records, 2, self.chunk_tokens, heads, head_dim)
        if self.buffers is None or tuple(self.buffers.shape) != shape or self.buffers.dtype != dtype:
            self.buffers = torch.empty(shape, dtype=dtype, device=device)

    def stream_back(self, parked: Sequence[Pair], total: int, copy_stream, compute_stream):
        """Generator of (slot index, first row, last row): the chunk's rows are in `buffers[slot]` when it is yielded;
        the consumer queues its work on `compute_stream` before advancing."""
        slots = [_Slot(), _Slot()]
        bounds = [(begin, min(begin + self.chunk_tokens, total)) for begin in range(0, total, self.chunk_tokens)]

        def fill(which: int, begin: int, end: int) -> None:
            with torch.cuda.stream(copy_stream):
                slots[which].wait_until_drained(copy_stream)
                for index, (key, value) in enumerate(parked):
                    self.buffers[which, index, 0, : end - begin].copy_(key[begin:end], non_blocking=True)
                    self.buffers[which, index, 1, : end - begin].copy_(value[begin:end], non_blocking=True)
                slots[which].filled.record(copy_stream)

        if bounds:
            fill(0, *bounds[0])
        for step, (begin, end) in enumerate(bounds):
            which = step & 1
            compute_stream.wait_event(slots[which].filled)
            if step + 1 < len(bounds):
                fill(which ^ 1, *bounds[step + 1])     # overlaps the consumer's work on this chunk
            yield which, begin, end
            slots[which].mark_drained(compute_stream)


class _LayerRing:
    """Device slots [slot][record][K|V][tokens][heads][head_dim] that hold whole layers' parked rows ahead of use."""

    def __init__(self):
        self.stream = torch.cuda.Stream()
        self.buffers: Optional[torch.Tensor] = None
        self.slots: List[_Slot] = []
        self.resident: Dict[object, int] = {}      # group -> slot that holds (or is receiving) its rows

    @property
    def size(self) -> int:
        return len(self.slots)

    def ensure(self, tokens: int, records: int, heads: int, head_dim: int, dtype=torch.bfloat16, device="cuda") -> None:
        big_enough = (self.buffers is not None and self.buffers.size(3) >= tokens and self.buffers.size(1) >= records
                      and tuple(self.buffers.shape[4:]) == (heads, head_dim))
        if big_enough:
            return
        count = ring_slots_for(tokens, records, heads, head_dim, torch.empty((), dtype=dtype).element_size())
        self.buffers = torch.empty((count, records, 2, tokens, heads, head_dim), dtype=dtype, device=device)
        self.buffers.record_stream(self.stream)
        self.slots = [_Slot() for _ in range(count)]
        self.resident.clear()

    def fetch(self, group, tokens: int, after: Optional[torch.cuda.Event]) -> None:
        """Start copying `group`'s parked rows into its slot (slot = position in the chain modulo ring size)."""
        if group in self.resident:
            return
        which = group.offload_index % self.size
        self.stream.wait_stream(torch.cuda.current_stream())
        if after is not None:
            self.stream.wait_event(after)          # the parked rows must have reached the host first
        with torch.cuda.stream(self.stream):
            self.slots[which].wait_until_drained(self.stream)
            for index, (key, value) in enumerate(group.pending):
                self.buffers[which, index, 0, :tokens].copy_(key[:tokens], non_blocking=True)
                self.buffers[which, index, 1, :tokens].copy_(value[:tokens], non_blocking=True)
            self.slots[which].filled.record(self.stream)
        self.resident[group] = which

    def take(self, group, tokens: int, records: int) -> Optional[Tuple[List[Pair], int]]:
        which = self.resident.pop(group, None)
        if which is None:
            return None
        torch.cuda.current_stream().wait_event(self.slots[which].filled)
        rows = [(self.buffers[which, i, 0, :tokens], self.buffers[which, i, 1, :tokens]) for i in range(records)]
        return rows, which

    def release(self, which: int) -> None:
        self.slots[which].mark_drained(torch.cuda.current_stream())


class PrefillHostStage:
    def __init__(self, chunk_tokens: int = 512, device=None):
        if type(chunk_tokens) is not int or chunk_tokens <= 0:
            raise ValueError("prefill_offload_chunk_tokens must be a positive integer")
        self.chunk_tokens = chunk_tokens
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.copy_stream = torch.cuda.Stream(self.device)
        self.lookahead_enabled = False
        self._chunks = _DoubleBuffer(chunk_tokens)
        self._ring: Optional[_LayerRing] = None
        self._stored = torch.cuda.Event()
        self._any_store = False

    # kept for callers that looked at the chunk buffers directly
    @property
    def workspace(self) -> Optional[torch.Tensor]:
        return self._chunks.buffers

    def reserve(self, tokens: int, pending_records: int, heads: int, head_dim: int, dtype=torch.bfloat16) -> None:
        """Allocate the transfer buffers now -- before a serving engine measures free memory for its KV pool -- for
        prompts of up to `tokens` tokens."""
        self._chunks.ensure(pending_records, heads, head_dim, dtype, self.device)
        if self.lookahead_enabled:
            self._ring = self._ring or _LayerRing()
            self._ring.ensure(tokens, pending_records, heads, head_dim, dtype, self.device)

    def store(self, key: torch.Tensor, value: torch.Tensor, buffer: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Copy `key`/`value` ([tokens, heads, head_dim]) into pinned host memory, asynchronously.  `buffer` is a pinned
        tensor from an earlier call to reuse ([2, >= tokens, heads, head_dim]); the (possibly new) buffer is returned.
        The copies are ordered after everything already queued on the current stream."""
        tokens, heads, head_dim = key.shape
        if buffer is None or buffer.size(1) < tokens or tuple(buffer.shape[2:]) != (heads, head_dim):
            buffer = torch.empty((2, tokens, heads, head_dim), dtype=key.dtype, device="cpu", pin_memory=True)
        current = torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(current)
        with torch.cuda.stream(self.copy_stream):
            buffer[0, :tokens].copy_(key, non_blocking=True)
            buffer[1, :tokens].copy_(value, non_blocking=True)
            self._stored.record(self.copy_stream)
        # the sources may be freed or overwritten by the caller: keep their memory until the copy stream is done
        key.record_stream(self.copy_stream)
        value.record_stream(self.copy_stream)
        self._any_store = True
        return buffer

    # ---- look-ahead ring --------------------------------------------------------------------------------
    def _ring_for(self, group, tokens: int) -> _LayerRing:
        self._ring = self._ring or _LayerRing()
        heads, head_dim = group.pending[0][0].shape[1:]
        self._ring.ensure(tokens, len(group.pending), heads, head_dim, group.pending[0][0].dtype, self.device)
        return self._ring

    def preload(self, group, tokens: int) -> None:
        """Called when `group` has just parked the rows of its last held-back loop: the first layers of the chain start
        travelling back at once, during the loop that precedes the writes."""
        if group.offload_index == 0 and self._ring is not None:
            self._ring.resident.clear()            # a new prompt: nothing of the old one is wanted any more
        ring = self._ring_for(group, tokens)
        if group.offload_index < ring.size:
            ring.fetch(group, tokens, self._stored if self._any_store else None)

    def prepare(self, group, tokens: int) -> None:
        """Called at the start of `group`'s completing loop: top the ring up with the layers that follow it."""
        if group.offload_index == 0 and self._ring is not None and group not in self._ring.resident:
            self._ring.resident.clear()
        ring = self._ring_for(group, tokens)
        held_back = len(group.pending)
        for later in group.offload_chain[group.offload_index: group.offload_index + ring.size]:
            if len(later.pending) == held_back:
                ring.fetch(later, tokens, self._stored if self._any_store else None)

    # ---- bringing the rows back -------------------------------------------------------------------------
    def chunks(self, records: Sequence[Pair], slot_mapping: torch.Tensor, group=None) -> Iterator[Tuple[List[Pair], torch.Tensor]]:
        """Yield `(records on the device, their slots)` pieces that together cover `slot_mapping`.  All records but the
        last are host tensors written by `store`; the last one is the completing loop's device K/V.  With `group` given
        and its rows resident in the look-ahead ring there is a single piece; otherwise the rows come back
        `chunk_tokens` at a time.  The caller queues its quantize on the current stream before asking for the next
        piece."""
        parked = len(records) - 1
        total = slot_mapping.numel()
        if total == 0:
            return
        if parked == 0:
            yield list(records), slot_mapping
            return
        last_key, last_value = records[-1]
        if group is not None and self._ring is not None:
            taken = self._ring.take(group, total, parked)
            if taken is not None:
                rows, which = taken
                yield rows + [(last_key[:total], last_value[:total])], slot_mapping
                self._ring.release(which)
                return
        _, heads, head_dim = last_key.shape
        self._chunks.ensure(parked, heads, head_dim, last_key.dtype, self.device)
        current = torch.cuda.current_stream(self.device)
        self.copy_stream.wait_stream(current)      # the buffers may still be read by the previous group's quantize
        for which, begin, end in self._chunks.stream_back(records[:-1], total, self.copy_stream, current):
            buffers = self._chunks.buffers
            rows = [(buffers[which, i, 0, : end - begin], buffers[which, i, 1, : end - begin]) for i in range(parked)]
            rows.append((last_key[begin:end], last_value[begin:end]))
            yield rows, slot_mapping[begin:end]
