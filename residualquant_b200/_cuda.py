"""Drop-in for the reference's extension module `residual_quantization._cuda`
(plugins/residual_quantization/csrc/dispatch/binding.cpp:19-37): the same two functions, the same keyword
names, argument meaning and error behaviour (RuntimeError on a rejected argument), implemented by the sm_100a
kernels behind the C ABI of include/rq_b200.h.

Differences a caller can see:
  * `key_rotation` / `value_rotation` are the dense fp16 `[heads, D, D]` tensors of the reference API or a
    `SignedHadamardRotation`.  A tensor that was passed once to `residualquant_b200.rotation.register_rotation` and
    recognised as diag(+-1) @ Hadamard runs the fused Walsh-Hadamard path; any other matrix is rotated by a
    tensor-core launch (TF32 products like the reference) in front of the quantizer / attention kernel.
  * scratch memory for the split-KV merge comes from one cached buffer per device instead of five allocations per
    call (attention/launch.cuh:85-98).  A buffer that was handed out once is never released: when a later call needs
    more, a larger buffer takes over and the old one stays alive for the CUDA graphs that captured its address.  A
    call made DURING capture that finds no buffer large enough takes its scratch from the graph's own memory pool, as
    the reference does.  All attention calls of a device share the buffer: issue them on one stream (the reference is
    called from vLLM's single model-runner thread), or order streams with events.
"""

from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib
from .rotation import SignedHadamardRotation, lookup

__all__ = ("attention", "quantize", "set_quantizer_chain", "set_attention_splits", "set_stable_metadata")

_chain = "kernel"
_forced_splits = 0
_stable_metadata = False
_workspaces: Dict[object, torch.Tensor] = {}
_superseded: List[torch.Tensor] = []   # earlier, smaller workspaces: captured graphs may still point into them


def set_quantizer_chain(chain: str) -> None:
    """"kernel": coefficient/residual in rotated coordinates like the reference's CUDA quantizer (default).
    "calibration": in original coordinates with bf16 prediction/target like the reference's PyTorch statement."""
    global _chain
    if chain not in _lib.CHAINS:
        raise ValueError("chain must be 'kernel' or 'calibration'")
    _chain = chain


def set_attention_splits(splits: int) -> None:
    """Force the number of KV partitions per query row (0 = library default)."""
    global _forced_splits
    _forced_splits = int(splits)


def set_stable_metadata(stable: bool) -> None:
    """Promise (or withdraw the promise) that the kernel launched immediately before an `attention` call on its stream
    never writes that call's `query_start_loc`, `seq_lens`, `block_table` or cached tokens (RQ_FLAG_STABLE_METADATA of
    include/rq_b200.h).  A serving engine that builds its metadata once per step, like the reference's vLLM builder
    (packed_backend.py:140-199), can promise it; the attention kernel then looks up its work and starts fetching pages
    while the previous kernel is still running.  Off by default."""
    global _stable_metadata
    _stable_metadata = bool(stable)


def _require(condition: bool, message: str) -> None:
    if not condition:
        raise RuntimeError(message)


def _validate_bf16_token_tensor(t: torch.Tensor) -> None:
    _require(
        t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 3 and t.stride(1) == t.size(2) and t.stride(2) == 1,
        "BF16 [tokens, heads, channels] with packed trailing strides required",
    )


def _rotation_arg(rotation, device, heads: int, head_dim: int, keep: list) -> _lib.RqRotation:
    out = _lib.RqRotation()
    if rotation is None:
        out.kind = _lib.ROTATION_NONE
        return out
    structured = rotation if isinstance(rotation, SignedHadamardRotation) else None
    if structured is None:
        _require(
            rotation.device == device and rotation.is_contiguous() and rotation.dtype == torch.float16
            and rotation.dim() == 3 and tuple(rotation.shape) == (heads, head_dim, head_dim),
            "Contiguous FP16 [heads, channels, channels] rotation required",
        )
        structured = lookup(rotation)
        if structured is None:
            # an arbitrary learned rotation: the kernels rotate with the dense matrix itself (fused, no extra launch)
            _require(rotation.data_ptr() % 16 == 0, "16-byte aligned rotation required")
            keep.append(rotation)
            out.kind = _lib.ROTATION_DENSE_FP16
            out.scale = 1.0
            out.data = rotation.data_ptr()
            return out
    _require(
        structured.heads == heads and structured.head_dim == head_dim and structured.sign_masks.device == device,
        "rotation does not match the head count, channel count or device",
    )
    keep.append(structured.sign_masks)
    out.kind = _lib.ROTATION_SIGNED_HADAMARD
    out.scale = structured.scale
    out.data = structured.sign_masks.data_ptr()
    return out


def _workspace(device: torch.device, nbytes: int, pairs: int) -> Tuple[torch.Tensor, bool]:
    """(scratch buffer of at least `nbytes`, True when it was created for this one call during graph capture).
    `pairs` = rows x heads: calls beyond 16384 pairs lay the buffer out differently and get buffers of their own."""
    key = (device.index or 0) if pairs <= 16384 else ((device.index or 0), (pairs - 1).bit_length())
    buf = _workspaces.get(key)
    if buf is not None and buf.numel() >= nbytes:
        return buf, False
    stream = torch.cuda.current_stream(device).cuda_stream
    if torch.cuda.is_current_stream_capturing():
        # graph-private memory: lives as long as the graph, zeroed by a memset node in front of the kernel
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _lib.check(_lib.load().rq_attention_workspace_init(buf.data_ptr(), nbytes, stream))
        return buf, True
    size = max(nbytes, 1 << 20, 2 * buf.numel() if buf is not None else 0)
    fresh = torch.empty(size, dtype=torch.uint8, device=device)
    _lib.check(_lib.load().rq_attention_workspace_init(fresh.data_ptr(), size, stream))
    if buf is not None:
        _superseded.append(buf)
    _workspaces[key] = fresh
    return fresh, False


def quantize(
    key_value_pairs: Sequence[Tuple[torch.Tensor, torch.Tensor]],
    kv_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    key_rotation,
    value_rotation,
    key_mean: Optional[torch.Tensor],
    records: Sequence[Sequence[int]],
    reference_mode: str,
    anchor_index: int,
    coefficient_method: str,
) -> None:
    """Rotate, quantize and pack the K/V rows of a whole KV group into the paged cache
    (reference: plugins/residual_quantization/csrc/common/api.h:22-31, quantize/api.cpp:8-95)."""
    lib = _lib.load()
    records = [list(r) for r in records]
    _require(len(records) > 0 and len(key_value_pairs) == len(records), "A nonempty group with one K/V input per record required")
    _require(
        kv_cache.is_cuda and kv_cache.dtype == torch.uint8 and kv_cache.is_contiguous() and kv_cache.dim() == 5
        and kv_cache.size(0) == 2,
        "Contiguous CUDA UINT8 [2, blocks, heads, page tokens, page width] cache required",
    )
    heads = kv_cache.size(2)
    head_dim = key_value_pairs[0][0].size(-1)
    _require(
        slot_mapping.device == kv_cache.device and slot_mapping.dtype == torch.int64 and slot_mapping.dim() == 1
        and slot_mapping.is_contiguous(),
        "Contiguous INT64 slot mapping on the cache device required",
    )
    for k, v in key_value_pairs:
        for t in (k, v):
            _validate_bf16_token_tensor(t)
            _require(
                t.device == kv_cache.device and t.size(1) == heads and t.size(2) == head_dim,
                "K/V must match the cache device/head count and logical channel count",
            )
            _require(t.size(0) >= slot_mapping.numel(), "Input has fewer rows than slot mapping")
    if key_mean is not None:
        _require(
            key_mean.device == kv_cache.device and key_mean.dtype == torch.float32 and key_mean.is_contiguous()
            and key_mean.dim() == 3 and tuple(key_mean.shape) == (len(records), heads, head_dim),
            "Contiguous FP32 [records, heads, channels] key mean required",
        )
    _require(coefficient_method in _lib.COEFFICIENTS, "Unsupported coefficient")

    args = _lib.RqQuantizeArgs()
    args.spec = _lib.make_spec(records, reference_mode, anchor_index, heads, head_dim, kv_cache.size(3))
    width = lib.rq_page_width(ctypes.byref(args.spec))
    _lib.check(min(width, 0))
    _require(kv_cache.size(4) == width, "Packed cache width differs from records")
    keep: list = []
    for i, (k, v) in enumerate(key_value_pairs):
        args.key[i] = k.data_ptr()
        args.value[i] = v.data_ptr()
        args.key_stride[i] = k.stride(0)
        args.value_stride[i] = v.stride(0)
    args.kv_cache = kv_cache.data_ptr()
    args.num_blocks = kv_cache.size(1)
    args.plane_stride = kv_cache.stride(0)
    args.slot_mapping = slot_mapping.data_ptr()
    args.num_tokens = slot_mapping.numel()
    args.key_rotation = _rotation_arg(key_rotation, kv_cache.device, heads, head_dim, keep)
    args.value_rotation = _rotation_arg(value_rotation, kv_cache.device, heads, head_dim, keep)
    args.key_mean = key_mean.data_ptr() if key_mean is not None else None
    args.coefficient = _lib.COEFFICIENTS[coefficient_method]
    args.chain = _lib.CHAINS[_chain]
    with torch.cuda.device(kv_cache.device):
        args.stream = torch.cuda.current_stream(kv_cache.device).cuda_stream
        _lib.check(lib.rq_quantize(ctypes.byref(args)))


def attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    kv_cache: torch.Tensor,
    output: torch.Tensor,
    query_start_loc: torch.Tensor,
    seq_lens: torch.Tensor,
    block_table: torch.Tensor,
    key_rotation,
    value_rotation,
    key_mean: Optional[torch.Tensor],
    records: Sequence[Sequence[int]],
    reference_mode: str,
    anchor_index: int,
    loop_index: int,
    *,
    gather=None,
    gather_buffer: int = 0,
) -> None:
    """Decode attention of one loop over the packed pages plus the live token; writes `output` in place
    (reference: plugins/residual_quantization/csrc/common/api.h:11-20, attention/api.cpp:8-115).

    `gather` (not part of the reference signature) is a `sharding.HeadGather`: when the KV heads are sharded over the
    GPUs of a node, the kernel also stores every finished row into buffer `gather_buffer` of every GPU's gathered
    output; call `gather.barrier()` afterwards, before anything reads the gathered rows (a no-op for
    `HeadGather(complete=True)`, where the call itself ends only when every rank's rows have arrived)."""
    lib = _lib.load()
    records = [list(r) for r in records]
    _validate_bf16_token_tensor(query)
    heads, head_dim = query.size(1), query.size(2)
    for t in (key, value, output):
        _validate_bf16_token_tensor(t)
        _require(t.device == query.device and t.shape == query.shape, "Q/K/V/output must have matching shapes and devices")
    for t in (query, key):
        _require(t.data_ptr() % 8 == 0 and t.stride(0) % 4 == 0, "Q/K addresses and token strides must be 8-byte aligned")
    _require(
        kv_cache.device == query.device and kv_cache.dtype == torch.uint8 and kv_cache.is_contiguous()
        and kv_cache.dim() == 5 and kv_cache.size(0) == 2 and kv_cache.size(2) == heads,
        "Contiguous UINT8 KV cache on the query device required",
    )
    if key_mean is not None:
        _require(
            key_mean.device == query.device and key_mean.dtype == torch.float32 and key_mean.is_contiguous()
            and key_mean.data_ptr() % 16 == 0 and key_mean.numel() == len(records) * heads * head_dim,
            "16-byte aligned contiguous FP32 key mean with matching dimensions required",
        )
    _require(
        query_start_loc.device == query.device and query_start_loc.dtype == torch.int32 and query_start_loc.dim() == 1
        and query_start_loc.is_contiguous() and query_start_loc.numel() == seq_lens.numel() + 1,
        "Contiguous INT32 query starts with one final boundary required",
    )
    _require(
        seq_lens.device == query.device and seq_lens.dtype == torch.int32 and seq_lens.dim() == 1 and seq_lens.is_contiguous(),
        "Contiguous INT32 sequence lengths required",
    )
    _require(
        block_table.device == query.device and block_table.dtype == torch.int32 and block_table.dim() == 2
        and block_table.stride(1) == 1 and block_table.size(0) >= seq_lens.numel(),
        "INT32 page table with packed rows required",
    )
    _require(0 <= loop_index < len(records), "Invalid loop index")
    rows = query.size(0)
    if rows == 0:
        return

    args = _lib.RqAttentionArgs()
    args.spec = _lib.make_spec(records, reference_mode, anchor_index, heads, head_dim, kv_cache.size(3))
    width = lib.rq_page_width(ctypes.byref(args.spec))
    _lib.check(min(width, 0))
    _require(kv_cache.size(4) == width, "Packed cache width differs from records")
    keep: list = []
    args.query, args.key, args.value, args.output = query.data_ptr(), key.data_ptr(), value.data_ptr(), output.data_ptr()
    args.query_stride, args.key_stride = query.stride(0), key.stride(0)
    args.value_stride, args.output_stride = value.stride(0), output.stride(0)
    args.num_query_rows = rows
    args.kv_cache = kv_cache.data_ptr()
    args.num_blocks = kv_cache.size(1)
    args.plane_stride = kv_cache.stride(0)
    args.query_start_loc = query_start_loc.data_ptr()
    args.seq_lens = seq_lens.data_ptr()
    args.block_table = block_table.data_ptr()
    args.num_requests = seq_lens.numel()
    args.block_table_stride = block_table.stride(0)
    args.max_blocks_per_request = block_table.size(1)
    args.key_rotation = _rotation_arg(key_rotation, query.device, heads, head_dim, keep)
    args.value_rotation = _rotation_arg(value_rotation, query.device, heads, head_dim, keep)
    args.key_mean = key_mean.data_ptr() if key_mean is not None else None
    args.loop_index = loop_index
    gather_flags = 0
    if gather is not None:
        _require(gather.rows >= rows and gather.local_heads == heads and gather.head_dim == head_dim,
                 "gathered output buffers do not match the query shape")
        pointers = gather.peer_pointers(gather_buffer)
        args.num_peers = len(pointers)
        for i, pointer in enumerate(pointers):
            args.peer_output[i] = pointer
        args.gather_head_offset = gather.head_offset
        args.gather_stride = gather.heads * head_dim
        complete, signalled = getattr(gather, "complete", False), getattr(gather, "signalled", False)
        if complete or signalled:
            # no barrier kernel between calls.  complete: the call itself ends only when every rank's rows have arrived.
            # signalled: this call publishes its completion and first waits for the previous one's
            for i, pointer in enumerate(gather.flag_pointers()):
                args.peer_flags[i] = pointer
            args.gather_state = gather.state.data_ptr()
            args.gather_rank = gather.rank
            args.gather_timeout_ns = int(getattr(gather, "timeout_ns", 0))   # 0: the library's 2 s
            if complete:
                gather_flags = _lib.FLAG_GATHER_COMPLETE
            else:
                gather_flags = ((_lib.FLAG_GATHER_PUBLISH if getattr(gather, "publish", True) else 0)
                                | (_lib.FLAG_GATHER_WAIT if getattr(gather, "wait", True) else 0))
    with torch.cuda.device(query.device):
        # 0: the kernel cuts every row into partitions in proportion to its own length, read on the device
        args.num_splits = _forced_splits
        nbytes = lib.rq_attention_workspace_bytes(rows, heads, head_dim, _forced_splits)
        workspace, one_call = _workspace(query.device, nbytes, rows * heads)
        keep.append(workspace)
        args.workspace = workspace.data_ptr()
        args.workspace_bytes = workspace.numel()
        if one_call:
            args.flags = _lib.FLAG_SERIAL_LAUNCH   # the kernel follows the memset of its own counters
        elif _stable_metadata:
            args.flags = _lib.FLAG_STABLE_METADATA
        args.flags |= gather_flags
        args.stream = torch.cuda.current_stream(query.device).cuda_stream
        _lib.check(lib.rq_attention(ctypes.byref(args)))


def attention_status(device=None) -> None:
    """Synchronize and raise if a bounded wait inside an attention kernel ever gave up on this device."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        for key, buf in list(_workspaces.items()):
            if (key if isinstance(key, int) else key[0]) == (device.index or 0):
                _lib.check(_lib.load().rq_attention_status(buf.data_ptr(), torch.cuda.current_stream(device).cuda_stream))
