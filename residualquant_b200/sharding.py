"""How the hot path spreads over the GPUs of one node (one process per GPU, `torch.distributed`).

Both operators are independent per (sequence, head) -- the reference's CTAs never reduce across either
(quantize/launch.cuh:32, attention/launch.cuh:112-113) -- so there are two partitionings:

* by SEQUENCES (the default): every rank owns a slice of the batch with its own page pool and block tables; there is no
  data-path collective at all.
* by KV HEADS (for a model whose single sequence batch must be split, e.g. 55 heads over 8 GPUs): every rank holds all
  sequences but only its heads of the cache; after attention one all-gather of `[rows, local_heads, head_dim]`
  rebuilds the full `[rows, heads, head_dim]` that the output projection consumes.  Head counts may be uneven
  (55 = 7*7 + 6), so slices are padded to the largest count for the collective.

  `HeadGather` is the fused form: the attention kernel stores its rows straight into every GPU's gathered buffer over
  NVLink (CUDA IPC mappings) and a one-CTA barrier kernel replaces the collective, so the whole decode step stays
  CUDA-graph capturable; `gather_heads` (one NCCL all-gather per call) is the plain form.

Timing helpers follow the benchmark contract: barrier on both sides, maximum over ranks.
"""

from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch
import torch.distributed as dist

from . import _lib


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


class _DeviceBytes:
    """A raw device allocation seen through `__cuda_array_interface__`, so that torch can view it without owning it."""

    def __init__(self, pointer: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (pointer, False), "version": 2}


def gather_layout(rows: int, heads: int, head_dim: int, buffers: int) -> Tuple[int, int, int]:
    """(bytes of one gathered buffer, offset of the flag array, total bytes) of a rank's shared allocation:
    `buffers` gathered outputs bf16 [rows, heads, head_dim], each rounded up to 256 bytes, then 256 bytes of flags."""
    one = (rows * heads * head_dim * 2 + 255) // 256 * 256
    return one, buffers * one, buffers * one + 256


class HeadGather:
    """Gathered attention output for KV heads sharded over the GPUs of one node, written by the attention kernel itself.

    Every rank allocates `buffers` gathered outputs bf16 [rows, heads, head_dim] plus a flag array in one IPC-shareable
    allocation and maps every peer's allocation.  `_cuda.attention(..., gather=self, gather_buffer=i)` then stores this
    rank's heads into buffer i of every rank; `barrier()` (a kernel on the current stream, CUDA-graph capturable) returns
    once every rank's stores have landed.  With two buffers used alternately and one barrier per call, a rank can start
    the next call while a slower peer still reads the previous result, because nobody passes barrier n before everyone
    entered it, and entering barrier n means being done with buffer n-2.

    `signalled=True` drops the barrier kernel between calls: the attention kernel itself publishes "this rank's rows of
    call n are in place" from its last CTA, and the NEXT attention call -- which in a model depends on the gathered rows
    through the output projection -- waits for every peer's signal of call n before it reads its inputs.  The same
    two-buffer rule holds: a rank publishes call n+1 only after its own wait for call n, so whoever has seen every
    rank's signal n+1 knows that buffer n%2 is no longer being read.  `barrier()` then is the consumer's wait alone
    (no publish), to be called wherever something other than the next attention call reads the gathered rows.

    `complete=True` needs no barrier at all: the attention kernel's last CTA publishes and then stays until every peer's
    signal of the same call has arrived, so the call ends only when this GPU's gathered buffer is complete and any
    kernel that follows on the stream may read it.  `barrier()` does nothing in this form.
    """

    def __init__(self, rows: int, heads: int, head_dim: int, device, buffers: int = 2, signalled: bool = False,
                 complete: bool = False):
        if signalled and complete:
            raise ValueError("choose one of signalled and complete")
        self.signalled, self.complete = signalled, complete
        self.lib = _lib.load()
        self.device = torch.device(device)
        self.rows, self.heads, self.head_dim, self.buffers = rows, heads, head_dim, buffers
        self.world = dist.get_world_size() if is_distributed() else 1
        self.rank = dist.get_rank() if is_distributed() else 0
        if self.world > _lib.RQ_MAX_PEERS:
            raise RuntimeError(f"at most {_lib.RQ_MAX_PEERS} GPUs of one node")
        counts = shard_counts(heads, self.world)
        self.local_heads = counts[self.rank]
        self.head_offset = sum(counts[: self.rank])
        self.buffer_bytes, self.flag_offset, self.nbytes = gather_layout(rows, heads, head_dim, buffers)
        with torch.cuda.device(self.device):
            base = ctypes.c_void_p()
            _lib.check(self.lib.rq_peer_alloc(self.nbytes, ctypes.byref(base)))
            self.base = base.value
            handle = ctypes.create_string_buffer(_lib.RQ_PEER_HANDLE_BYTES)
            _lib.check(self.lib.rq_peer_export(self.base, handle))
            handles = [handle.raw]
            if self.world > 1:
                handles = [None] * self.world
                dist.all_gather_object(handles, handle.raw)
            self.bases = []
            for peer, raw in enumerate(handles):
                if peer == self.rank:
                    self.bases.append(self.base)
                    continue
                mapped = ctypes.c_void_p()
                _lib.check(self.lib.rq_peer_open(raw, ctypes.byref(mapped)))
                self.bases.append(mapped.value)
            self.state = torch.zeros(64, dtype=torch.int32, device=self.device)
            self._owner = _DeviceBytes(self.base, self.nbytes)
            self._bytes = torch.as_tensor(self._owner, device=self.device)
        # the zero fill of the allocation and of the barrier state is complete on this GPU ...
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier()   # ... and every rank has mapped every allocation before anyone writes

    def peer_pointers(self, buffer: int) -> List[int]:
        if not 0 <= buffer < self.buffers:
            raise ValueError("no such gathered buffer")
        return [base + buffer * self.buffer_bytes for base in self.bases]

    def gathered(self, buffer: int) -> torch.Tensor:
        """This rank's copy of gathered buffer `buffer`: bf16 [rows, heads, head_dim]."""
        begin = buffer * self.buffer_bytes
        flat = self._bytes[begin : begin + self.rows * self.heads * self.head_dim * 2].view(torch.bfloat16)
        return flat.view(self.rows, self.heads, self.head_dim)

    def barrier(self, timeout_ns: int = 0) -> None:
        if self.complete:
            return
        args = _lib.RqPeerBarrierArgs()
        args.world, args.rank = self.world, self.rank
        for i, base in enumerate(self.bases):
            args.flags[i] = base + self.flag_offset
        args.state = self.state.data_ptr()
        args.timeout_ns = timeout_ns
        args.wait_only = 1 if self.signalled else 0
        with torch.cuda.device(self.device):
            args.stream = torch.cuda.current_stream(self.device).cuda_stream
            _lib.check(self.lib.rq_peer_barrier(ctypes.byref(args)))

    def flag_pointers(self) -> List[int]:
        """Every rank's flag array as mapped into this process."""
        return [base + self.flag_offset for base in self.bases]

    def check(self) -> None:
        """Synchronize the current stream and raise if a barrier ever timed out."""
        with torch.cuda.device(self.device):
            _lib.check(self.lib.rq_peer_barrier_status(self.state.data_ptr(),
                                                       torch.cuda.current_stream(self.device).cuda_stream))

    def close(self) -> None:
        """Unmap the peers' allocations and free this rank's (collective: all ranks leave the barrier first)."""
        if self.base is None:
            return
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier()
        with torch.cuda.device(self.device):
            for peer, base in enumerate(self.bases):
                if peer != self.rank:
                    self.lib.rq_peer_close(base)
            if self.world > 1:
                dist.barrier()
            self._bytes = None
            self.lib.rq_peer_free(self.base)
        self.base = None
