"""ctypes view of the C ABI declared in include/rq_b200.h.  Loading fails loudly: there is no fallback."""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# RQ_B200_LIBRARY: another build of the same library (e.g. librq_b200_timeline.so, see build.py)
LIBRARY_PATH = os.environ.get("RQ_B200_LIBRARY") or os.path.join(HERE, "librq_b200.so")

RQ_MAX_RECORDS = 8
RQ_MAX_PEERS = 8
RQ_PEER_HANDLE_BYTES = 64
RQ_OK = 0
FLAG_SERIAL_LAUNCH = 1
FLAG_STABLE_METADATA = 2
FLAG_GATHER_PUBLISH = 4
FLAG_GATHER_WAIT = 8
FLAG_GATHER_COMPLETE = 16
REFERENCE_MODES = {"anchor": 0, "adjacent": 1}
COEFFICIENTS = {"unit": 0, "norm": 1, "ls": 2}
CHAINS = {"kernel": 0, "calibration": 1}
ROTATION_NONE, ROTATION_SIGNED_HADAMARD, ROTATION_DENSE_FP16 = 0, 1, 2

EXPORTS = (
    "rq_page_width",
    "rq_record_offset",
    "rq_quantize",
    "rq_quantize_workspace_bytes",
    "rq_attention_default_splits",
    "rq_attention_work_capacity",
    "rq_attention_noalloc_status",
    "rq_set_programmatic_launch",
    "rq_attention_workspace_bytes",
    "rq_attention_workspace_init",
    "rq_attention",
    "rq_attention_status",
    "rq_attention_noalloc",
    "rq_peer_barrier",
    "rq_peer_barrier_status",
    "rq_peer_alloc",
    "rq_peer_free",
    "rq_peer_export",
    "rq_peer_open",
    "rq_peer_close",
    "rq_last_error",
    "rq_version",
)


class RqRotation(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("scale", ctypes.c_float), ("data", ctypes.c_void_p)]


class RqGroupSpec(ctypes.Structure):
    _fields_ = [
        ("num_records", ctypes.c_int32),
        ("bits", ctypes.c_int32 * RQ_MAX_RECORDS),
        ("group_size", ctypes.c_int32 * RQ_MAX_RECORDS),
        ("anchor_index", ctypes.c_int32),
        ("reference_mode", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("page_tokens", ctypes.c_int32),
    ]


class RqQuantizeArgs(ctypes.Structure):
    _fields_ = [
        ("spec", RqGroupSpec),
        ("key", ctypes.c_void_p * RQ_MAX_RECORDS),
        ("value", ctypes.c_void_p * RQ_MAX_RECORDS),
        ("key_stride", ctypes.c_int64 * RQ_MAX_RECORDS),
        ("value_stride", ctypes.c_int64 * RQ_MAX_RECORDS),
        ("kv_cache", ctypes.c_void_p),
        ("num_blocks", ctypes.c_int64),
        ("plane_stride", ctypes.c_int64),
        ("slot_mapping", ctypes.c_void_p),
        ("num_tokens", ctypes.c_int64),
        ("key_rotation", RqRotation),
        ("value_rotation", RqRotation),
        ("key_mean", ctypes.c_void_p),
        ("coefficient", ctypes.c_int32),
        ("chain", ctypes.c_int32),
        ("stream", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("flags", ctypes.c_int32),
    ]


class RqAttentionArgs(ctypes.Structure):
    _fields_ = [
        ("spec", RqGroupSpec),
        ("query", ctypes.c_void_p),
        ("key", ctypes.c_void_p),
        ("value", ctypes.c_void_p),
        ("output", ctypes.c_void_p),
        ("query_stride", ctypes.c_int64),
        ("key_stride", ctypes.c_int64),
        ("value_stride", ctypes.c_int64),
        ("output_stride", ctypes.c_int64),
        ("num_query_rows", ctypes.c_int32),
        ("kv_cache", ctypes.c_void_p),
        ("num_blocks", ctypes.c_int64),
        ("plane_stride", ctypes.c_int64),
        ("query_start_loc", ctypes.c_void_p),
        ("seq_lens", ctypes.c_void_p),
        ("block_table", ctypes.c_void_p),
        ("num_requests", ctypes.c_int32),
        ("block_table_stride", ctypes.c_int32),
        ("max_blocks_per_request", ctypes.c_int32),
        ("key_rotation", RqRotation),
        ("value_rotation", RqRotation),
        ("key_mean", ctypes.c_void_p),
        ("loop_index", ctypes.c_int32),
        ("num_splits", ctypes.c_int32),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("stream", ctypes.c_void_p),
        ("num_peers", ctypes.c_int32),
        ("gather_head_offset", ctypes.c_int32),
        ("gather_stride", ctypes.c_int64),
        ("peer_output", ctypes.c_void_p * RQ_MAX_PEERS),
        ("flags", ctypes.c_int32),
        ("peer_flags", ctypes.c_void_p * RQ_MAX_PEERS),
        ("gather_state", ctypes.c_void_p),
        ("gather_rank", ctypes.c_int32),
        ("gather_timeout_ns", ctypes.c_uint64),
    ]


class RqPeerBarrierArgs(ctypes.Structure):
    _fields_ = [
        ("world", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("flags", ctypes.c_void_p * RQ_MAX_PEERS),
        ("state", ctypes.c_void_p),
        ("timeout_ns", ctypes.c_uint64),
        ("stream", ctypes.c_void_p),
        ("wait_only", ctypes.c_int32),
    ]


_lib = None


def load() -> ctypes.CDLL:
    """Load librq_b200.so (built by `python -m residualquant_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise RuntimeError(
            f"{LIBRARY_PATH} is missing: build the CUDA kernels with `python -m residualquant_b200.build`. "
            "There is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIBRARY_PATH)
    lib.rq_page_width.argtypes = [ctypes.POINTER(RqGroupSpec)]
    lib.rq_page_width.restype = ctypes.c_int32
    lib.rq_record_offset.argtypes = [ctypes.POINTER(RqGroupSpec), ctypes.c_int32]
    lib.rq_record_offset.restype = ctypes.c_int32
    lib.rq_quantize_workspace_bytes.argtypes = [ctypes.POINTER(RqGroupSpec), ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]
    lib.rq_quantize_workspace_bytes.restype = ctypes.c_size_t
    lib.rq_quantize.argtypes = [ctypes.POINTER(RqQuantizeArgs)]
    lib.rq_quantize.restype = ctypes.c_int32
    lib.rq_attention_default_splits.argtypes = [ctypes.c_int32] * 4
    lib.rq_attention_default_splits.restype = ctypes.c_int32
    lib.rq_attention_work_capacity.argtypes = [ctypes.c_int32] * 2
    lib.rq_attention_work_capacity.restype = ctypes.c_int32
    lib.rq_attention_noalloc_status.argtypes = [ctypes.c_void_p]
    lib.rq_attention_noalloc_status.restype = ctypes.c_int32
    lib.rq_set_programmatic_launch.argtypes = [ctypes.c_int32]
    lib.rq_set_programmatic_launch.restype = None
    lib.rq_attention_workspace_bytes.argtypes = [ctypes.c_int32] * 4
    lib.rq_attention_workspace_bytes.restype = ctypes.c_size_t
    lib.rq_attention_workspace_init.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]
    lib.rq_attention_workspace_init.restype = ctypes.c_int32
    lib.rq_attention.argtypes = [ctypes.POINTER(RqAttentionArgs)]
    lib.rq_attention.restype = ctypes.c_int32
    lib.rq_attention_noalloc.argtypes = [ctypes.POINTER(RqAttentionArgs)]
    lib.rq_attention_noalloc.restype = ctypes.c_int32
    lib.rq_attention_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.rq_attention_status.restype = ctypes.c_int32
    lib.rq_peer_barrier.argtypes = [ctypes.POINTER(RqPeerBarrierArgs)]
    lib.rq_peer_barrier.restype = ctypes.c_int32
    lib.rq_peer_barrier_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.rq_peer_barrier_status.restype = ctypes.c_int32
    lib.rq_peer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)]
    lib.rq_peer_alloc.restype = ctypes.c_int32
    lib.rq_peer_free.argtypes = [ctypes.c_void_p]
    lib.rq_peer_free.restype = ctypes.c_int32
    lib.rq_peer_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    lib.rq_peer_export.restype = ctypes.c_int32
    lib.rq_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.rq_peer_open.restype = ctypes.c_int32
    lib.rq_peer_close.argtypes = [ctypes.c_void_p]
    lib.rq_peer_close.restype = ctypes.c_int32
    lib.rq_last_error.argtypes = []
    lib.rq_last_error.restype = ctypes.c_char_p
    lib.rq_version.argtypes = []
    lib.rq_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def make_spec(records, reference_mode: str, anchor_index: int, heads: int, head_dim: int, page_tokens: int) -> RqGroupSpec:
    if reference_mode not in REFERENCE_MODES:
        raise RuntimeError(f"Unknown packed reference mode: {reference_mode}")
    records = [tuple(int(v) for v in record) for record in records]
    if not records or len(records) > RQ_MAX_RECORDS or any(len(record) != 2 for record in records):
        raise RuntimeError(f"A nonempty group of at most {RQ_MAX_RECORDS} [bits, group] records required")
    spec = RqGroupSpec()
    spec.num_records = len(records)
    for i, (bits, group) in enumerate(records):
        spec.bits[i] = bits
        spec.group_size[i] = group
    spec.anchor_index = int(anchor_index)
    spec.reference_mode = REFERENCE_MODES[reference_mode]
    spec.heads = int(heads)
    spec.head_dim = int(head_dim)
    spec.page_tokens = int(page_tokens)
    return spec


def check(status: int) -> None:
    if status != RQ_OK:
        raise RuntimeError(load().rq_last_error().decode() or f"rq_b200 error {status}")
