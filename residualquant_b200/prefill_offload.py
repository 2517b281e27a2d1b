"""Host staging of raw K/V during a long prefill.

The K/V of a group's non-final loops have to be kept until the last loop arrives (`group.DeferredKVGroup`).  For a long
prompt that is `(records - 1) x 2 x tokens x heads x head_dim` bf16 values per owner; the reference can park them in
pinned host memory and stream them back for the group's quantize
(plugins/residual_quantization/src/residual_quantization/prefill_offload.py:10-200).  This is the same service with a
smaller mechanism: one copy stream, device-to-host copies ordered after the producing stream by an event, and a
two-slot device workspace through which the rows come back `chunk_tokens` at a time while the previous chunk is being
quantized.  (The reference's optional whole-layer look-ahead ring is not reproduced: with 180 GB of HBM per GPU the
chunked path already keeps the device-side footprint at two chunks.)
"""

from __future__ import annotations

from typing import Iterator, List, Optional, Sequence, Tuple

import torch

Pair = Tuple[torch.Tensor, torch.Tensor]


class PrefillHostStage:
    def __init__(self, chunk_tokens: int = 512, device=None):
        if type(chunk_tokens) is not int or chunk_tokens <= 0:
            raise ValueError("prefill_offload_chunk_tokens must be a positive integer")
        self.chunk_tokens = chunk_tokens
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.copy_stream = torch.cuda.Stream(self.device)
        self.workspace: Optional[torch.Tensor] = None    # [2 slots][records - 1][K|V][chunk][heads][head_dim]
        self._stored = torch.cuda.Event()
        self._any_store = False

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

    def _ensure_workspace(self, pending: int, heads: int, head_dim: int, dtype) -> None:
        shape = (2, pending, 2, self.chunk_tokens, heads, head_dim)
        if self.workspace is None or tuple(self.workspace.shape) != shape or self.workspace.dtype != dtype:
            self.workspace = torch.empty(shape, dtype=dtype, device=self.device)

    def chunks(self, records: Sequence[Pair], slot_mapping: torch.Tensor) -> Iterator[Tuple[List[Pair], torch.Tensor]]:
        """Yield `(records of one chunk on the device, slots of that chunk)`.  All records but the last are host
        tensors written by `store`; the last one is the completing loop's device K/V.  The caller queues its quantize
        on the current stream before asking for the next chunk."""
        pending = len(records) - 1
        total = slot_mapping.numel()
        if pending == 0 or total == 0:
            if total:
                yield list(records), slot_mapping
            return
        last_key, last_value = records[-1]
        _, heads, head_dim = last_key.shape
        self._ensure_workspace(pending, heads, head_dim, last_key.dtype)
        current = torch.cuda.current_stream(self.device)
        # the workspace may still be read by quantize calls of the previous group
        self.copy_stream.wait_stream(current)
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        used = [False, False]

        def fetch(begin: int, slot: int) -> None:
            end = min(begin + self.chunk_tokens, total)
            with torch.cuda.stream(self.copy_stream):
                if used[slot]:
                    self.copy_stream.wait_event(consumed[slot])
                for index, (key, value) in enumerate(records[:-1]):
                    self.workspace[slot, index, 0, : end - begin].copy_(key[begin:end], non_blocking=True)
                    self.workspace[slot, index, 1, : end - begin].copy_(value[begin:end], non_blocking=True)
                ready[slot].record(self.copy_stream)

        fetch(0, 0)   # same stream as the stores: the host buffers are complete before they are read back
        for step, begin in enumerate(range(0, total, self.chunk_tokens)):
            slot = step % 2
            end = min(begin + self.chunk_tokens, total)
            current.wait_event(ready[slot])
            if end < total:
                fetch(end, 1 - slot)
            staged = [(self.workspace[slot, i, 0, : end - begin], self.workspace[slot, i, 1, : end - begin])
                      for i in range(pending)]
            staged.append((last_key[begin:end], last_value[begin:end]))
            yield staged, slot_mapping[begin:end]
            consumed[slot].record(current)
            used[slot] = True
