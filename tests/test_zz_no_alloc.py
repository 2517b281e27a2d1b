"""The allocation-free attention entry point against the regular one, through the C ABI.

Some callers may not allocate device memory at all: a serving loop whose framework has already frozen its
memory pool, a plugin that only receives tensors, code that must never trigger the device-wide synchronization a
cudaMalloc can cause.  `rq_attention_noalloc` serves them from a scratch buffer compiled into the library.  This
test runs last (file name) so that a run stopping at the first failure has already seen every other test; it
passes alone in a fresh process too.
"""

import ctypes

import numpy as np
import pytest
import torch

from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu


def _args(case, cache, q, k, v, out, qsl, seq, table, kr, vr, loop, splits):
    from residualquant_b200 import _lib

    L = case.layout
    a = _lib.RqAttentionArgs()
    a.spec = _lib.make_spec([list(r) for r in L.records], L.reference_mode, L.anchor_index, case.heads, L.head_dim,
                            L.page_tokens)
    a.query, a.key, a.value, a.output = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.query_stride, a.key_stride, a.value_stride, a.output_stride = q.stride(0), k.stride(0), v.stride(0), out.stride(0)
    a.num_query_rows = q.size(0)
    a.kv_cache, a.num_blocks, a.plane_stride = cache.data_ptr(), cache.size(1), cache.stride(0)
    a.query_start_loc, a.seq_lens, a.block_table = qsl.data_ptr(), seq.data_ptr(), table.data_ptr()
    a.num_requests, a.block_table_stride, a.max_blocks_per_request = seq.numel(), table.stride(0), table.size(1)
    for rot, field in ((kr, a.key_rotation), (vr, a.value_rotation)):
        field.kind = _lib.ROTATION_SIGNED_HADAMARD
        field.scale = rot.scale
        field.data = rot.sign_masks.data_ptr()
    a.key_mean = None
    a.loop_index = loop
    a.num_splits = splits
    a.stream = torch.cuda.current_stream().cuda_stream
    return a


@pytest.mark.parametrize("splits", [3, 1, 0])
def test_noalloc_entry_matches_regular_entry_twice(splits):
    from residualquant_b200 import _lib

    lib = _lib.load()
    case = helpers.make_case(77, 128, 4, [400, 1, 57], 32, 16)
    cache_np = helpers.oracle_cache(case)
    cache = torch.from_numpy(cache_np).cuda()
    kr, vr = G.device_rotations(case)
    rows = len(case.seq_lens)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    q = G.bf16(case.query)
    for loop in (0, 3):
        k = G.bf16(case.keys[loop][case.live_rows])
        v = G.bf16(case.values[loop][case.live_rows])
        want = helpers.oracle_attention(case, cache_np, loop)
        # regular entry point with a caller-owned workspace
        nbytes = lib.rq_attention_workspace_bytes(rows, case.heads, 128, splits)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.rq_attention_workspace_init(workspace.data_ptr(), nbytes, stream))
        regular = torch.zeros_like(q)
        a = _args(case, cache, q, k, v, regular, qsl, seq, table, kr, vr, loop, splits)
        a.workspace, a.workspace_bytes = workspace.data_ptr(), nbytes
        _lib.check(lib.rq_attention(ctypes.byref(a)))
        torch.cuda.synchronize()
        # The documented set-up: the first call on a device looks up the built-in buffer's address, which also makes
        # the driver materialise the library's device data (8 MiB, once per device and process).
        setup = _args(case, cache, q, k, v, torch.zeros_like(q), qsl, seq, table, kr, vr, loop, splits)
        _lib.check(lib.rq_attention_noalloc(ctypes.byref(setup)))
        # allocation-free entry point, two calls in a row on the shared built-in scratch
        for attempt in range(2):
            out = torch.zeros_like(q)
            b = _args(case, cache, q, k, v, out, qsl, seq, table, kr, vr, loop, splits)
            # free device memory as the driver sees it: a raw cudaMalloc inside the call would show here
            # (torch's own counters only see torch's allocator)
            torch.cuda.synchronize()
            before = torch.cuda.mem_get_info()[0]
            _lib.check(lib.rq_attention_noalloc(ctypes.byref(b)))
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == before
            assert lib.rq_attention_noalloc_status(torch.cuda.current_stream().cuda_stream) == 0
            got, ref = out.float().cpu().numpy(), regular.float().cpu().numpy()
            assert np.all(np.abs(got - ref) <= 2e-2 + 1e-2 * np.abs(ref)), f"attempt {attempt}: differs from rq_attention"
            assert np.all(np.abs(got - want) <= 2e-2 + 1e-2 * np.abs(want)), f"attempt {attempt}: differs from the oracle"


def test_noalloc_entry_rejects_shapes_beyond_its_buffer():
    from residualquant_b200 import _lib

    lib = _lib.load()
    case = helpers.make_case(78, 128, 4, [40], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    kr, vr = G.device_rotations(case)
    big_rows = 512                                   # 512 rows x 4 heads x 64 splits x 130 floats > 8 MiB
    q = torch.zeros(big_rows, 4, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    qsl = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    a = _args(case, cache, q, q, q, out, qsl, seq, table, kr, vr, 0, 64)
    assert lib.rq_attention_noalloc(ctypes.byref(a)) == -3
    assert b"built-in buffer" in lib.rq_last_error()


def test_noalloc_entry_reports_a_bad_spec_as_such():
    from residualquant_b200 import _lib

    lib = _lib.load()
    case = helpers.make_case(78, 128, 4, [40], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    kr, vr = G.device_rotations(case)
    q = G.bf16(case.query)
    qsl = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    a = _args(case, cache, q, q, q, torch.zeros_like(q), qsl, seq, table, kr, vr, 0, 0)
    a.spec.heads = 0
    assert lib.rq_attention_noalloc(ctypes.byref(a)) == -1          # RQ_ERR_INVALID_ARGUMENT, not a workspace error
    a.spec.heads = 4
    a.num_splits = -100000
    assert lib.rq_attention_noalloc(ctypes.byref(a)) == -1


def test_noalloc_entry_with_a_dense_key_rotation():
    """A dense (learned) key rotation: the query row is rotated inside the attention kernel, no extra scratch."""
    from residualquant_b200 import _lib

    lib = _lib.load()
    case = helpers.make_case(79, 128, 4, [260, 33], 32, 16)
    cache_np = helpers.oracle_cache(case)
    cache = torch.from_numpy(cache_np).cuda()
    kr, vr = G.device_rotations(case)
    dense = kr.dense().contiguous()
    rows = len(case.seq_lens)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    q = G.bf16(case.query)
    k, v = G.bf16(case.keys[1][case.live_rows]), G.bf16(case.values[1][case.live_rows])
    want = helpers.oracle_attention(case, cache_np, 1)
    for attempt in range(2):
        out = torch.zeros_like(q)
        a = _args(case, cache, q, k, v, out, qsl, seq, table, kr, vr, 1, 0)
        a.key_rotation.kind = _lib.ROTATION_DENSE_FP16
        a.key_rotation.scale = 1.0
        a.key_rotation.data = dense.data_ptr()
        _lib.check(lib.rq_attention_noalloc(ctypes.byref(a)))
        torch.cuda.synchronize()
        got = out.float().cpu().numpy()
        assert np.all(np.abs(got - want) <= 2e-2 + 1e-2 * np.abs(want)), f"attempt {attempt}"
