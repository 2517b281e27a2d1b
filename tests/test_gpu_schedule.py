"""Length-aware KV partitioning on the device, programmatic dependent launch and workspace lifetime.

The attention kernel cuts every query row into partitions in proportion to the row's own length, read from
`seq_lens` on the device (the reference builds the same kind of schedule in a separate kernel:
plugins/residual_quantization/csrc/attention/prepare.cuh:237-386).  These tests compare that path with the oracle on
ragged batches, with forced uniform partitions, and with plain stream-ordered launches.

Tolerance (stated by the task for bf16 outputs): |got - want| <= 2e-2 + 1e-2 * |want| on every element."""

import numpy as np
import pytest
import torch

from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-2, 1e-2


def _inside(got, want):
    return np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want))


def test_ragged_batch_of_64_rows():
    """One 8192-token row among 63 rows of 17..600 tokens, the batch the partition schedule exists for.  The cache is
    written by the GPU quantizer (bit-exact with the oracle's, see test_gpu_quantize.py); the oracle reads those bytes."""
    rng = np.random.default_rng(5)
    lengths = [8192] + [int(v) for v in rng.integers(17, 601, size=63)]
    case = helpers.make_case(41, 128, 4, lengths, 32, 16)
    cache = G.gpu_cache(case)
    cache_np = cache.cpu().numpy()
    for loop in (0, 3):
        got = G.gpu_attention(case, cache, loop).float().cpu().numpy()
        want = helpers.oracle_attention(case, cache_np, loop)
        assert _inside(got, want), f"loop {loop}: {np.abs(got - want).max()}"


@pytest.mark.parametrize("head_dim,heads,page", [(128, 16, 16), (96, 5, 32), (128, 1, 16)])
def test_device_schedule_agrees_with_forced_partitions(head_dim, heads, page):
    """Same outputs (within the tolerance) whether the kernel picks the partitions or every row gets a forced count;
    more than 32 requests (two passes of the warp-wide scan), rows without history, padding rows at the end."""
    from residualquant_b200 import _cuda

    rng = np.random.default_rng(6)
    lengths = [int(v) for v in rng.integers(1, 400, size=45)] + [1500, 1, 2]
    case = helpers.make_case(42, head_dim, heads, lengths, 32, page)
    cache = G.gpu_cache(case)
    cache_np = cache.cpu().numpy()
    want = helpers.oracle_attention(case, cache_np, 1)
    chosen = G.gpu_attention(case, cache, 1, pad_rows=5).float().cpu().numpy()
    assert np.all(chosen[len(lengths):] == 768.0), "padding rows must stay untouched"
    assert _inside(chosen[:len(lengths)], want)
    _cuda.set_attention_splits(3)
    try:
        forced = G.gpu_attention(case, cache, 1).float().cpu().numpy()
    finally:
        _cuda.set_attention_splits(0)
    assert _inside(forced, want)


def test_serial_and_programmatic_launches_agree():
    """The kernels are launched as programmatic dependents by default; switching that off must not change a byte of
    the cache nor (beyond run-to-run identical arithmetic) the attention output."""
    from residualquant_b200 import _lib

    lib = _lib.load()
    case = helpers.make_case(43, 128, 3, [700, 40, 1, 333], 16, 16)
    outputs = {}
    for mode in (1, 0):
        lib.rq_set_programmatic_launch(mode)
        try:
            cache = G.gpu_cache(case)
            outputs[mode] = (cache.cpu().numpy(), [G.gpu_attention(case, cache, loop).float().cpu().numpy() for loop in range(4)])
        finally:
            lib.rq_set_programmatic_launch(1)
    assert np.array_equal(outputs[0][0], outputs[1][0])
    assert np.array_equal(outputs[0][0], helpers.oracle_cache(case))
    for a, b in zip(outputs[0][1], outputs[1][1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("stable_metadata", [False, True])
def test_back_to_back_calls_share_the_workspace_safely(stable_metadata):
    """Many attention calls in a row on one stream with no host synchronization in between (the decode step's pattern):
    each call's partial results and counters live in the same scratch as its predecessor's, and a programmatic
    dependent is scheduled before its predecessor has finished.  With the caller's promise of stable metadata the
    work lookup and the first page copies of a call also run before its predecessor has finished."""
    from residualquant_b200 import _cuda

    case = helpers.make_case(44, 128, 8, [2000, 1100, 64, 3], 32, 16)
    L = case.layout
    cache = G.gpu_cache(case)
    cache_np = cache.cpu().numpy()
    kr, vr = G.device_rotations(case)
    rows = len(case.seq_lens)
    q = G.bf16(case.query)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    live = [(G.bf16(case.keys[loop][case.live_rows]), G.bf16(case.values[loop][case.live_rows])) for loop in range(4)]
    outs = [torch.zeros_like(q) for _ in range(24)]
    torch.cuda.synchronize()
    _cuda.set_stable_metadata(stable_metadata)
    try:
        for i, out in enumerate(outs):
            k, v = live[i % 4]
            _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, [list(r) for r in L.records], "anchor", 3, i % 4)
    finally:
        _cuda.set_stable_metadata(False)
    torch.cuda.synchronize()
    for loop in range(4):
        want = helpers.oracle_attention(case, cache_np, loop)
        for i in range(loop, 24, 4):
            assert _inside(outs[i].float().cpu().numpy(), want), f"call {i}"
            assert torch.equal(outs[i], outs[loop]), f"call {i} differs from call {loop}"


def test_graph_keeps_its_workspace_when_a_larger_call_follows():
    """A CUDA graph captured at a small batch holds the address of the scratch buffer of that time.  A later, larger eager
    call makes the library move to a bigger buffer; the old one must stay alive, and the graph's replay stay correct."""
    from residualquant_b200 import _cuda

    small = helpers.make_case(45, 128, 2, [300, 90], 32, 16)
    cache = G.gpu_cache(small)
    want = helpers.oracle_attention(small, cache.cpu().numpy(), 0)
    L = small.layout
    records = [list(r) for r in L.records]
    kr, vr = G.device_rotations(small)
    q = G.bf16(small.query)
    k, v = G.bf16(small.keys[0][small.live_rows]), G.bf16(small.values[0][small.live_rows])
    out = torch.zeros_like(q)
    qsl = torch.arange(3, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(small.seq_lens).cuda()
    table = torch.from_numpy(small.block_table).cuda()

    def call():
        _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, records, "anchor", 3, 0)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        call()
    # a much larger call: enough rows to need more scratch than any call before it in this process
    from residualquant_b200 import _lib

    held = _cuda._workspaces[torch.cuda.current_device()]
    rows = 3000
    while _lib.load().rq_attention_workspace_bytes(rows, 2, 128, 0) <= held.numel():
        rows *= 2
    big_q = torch.zeros(rows, 2, 128, dtype=torch.bfloat16, device="cuda")
    big_out = torch.zeros_like(big_q)
    big_qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    big_seq = torch.full((rows,), 40, dtype=torch.int32, device="cuda")
    big_table = torch.from_numpy(small.block_table[:1]).cuda().repeat(rows, 1)
    _cuda.attention(big_q, big_q, big_q, cache, big_out, big_qsl, big_seq, big_table, kr, vr, None, records, "anchor", 3, 0)
    torch.cuda.synchronize()
    assert _cuda._workspaces[torch.cuda.current_device()] is not held, "the larger call should have needed a new buffer"
    garbage = [torch.full((1 << 20,), 0x7F, dtype=torch.uint8, device="cuda") for _ in range(8)]   # would land in freed scratch
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert _inside(out.float().cpu().numpy(), want)
    del garbage


def test_config0_one_layer_end_to_end():
    """BASELINE's CPU-runnable case as ONE test: 4 loops, 16 heads x 128, batch 1, context 2048.  The 2047 cached tokens
    are quantized on the GPU and compared byte for byte with the oracle's cache, then the four loops' decode attentions
    are compared with the oracle."""
    case = helpers.make_case(46, 128, 16, [2048], 32, 16)
    cache = G.gpu_cache(case)
    cache_np = helpers.oracle_cache(case)
    assert np.array_equal(cache.cpu().numpy(), cache_np), "packed cache differs from the oracle"
    for loop in range(4):
        got = G.gpu_attention(case, cache, loop).float().cpu().numpy()
        want = helpers.oracle_attention(case, cache_np, loop)
        assert _inside(got, want), f"loop {loop}: {np.abs(got - want).max()}"


def test_peer_barrier_wait_runs_out_and_reports_it():
    """A bounded wait that nothing satisfies: rank 0 of a two-rank barrier whose peer slot is a zeroed local buffer that
    nobody writes.  The kernel must return after its time limit with RQ_ERR_DEVICE_TIMEOUT in the status word, the epoch
    advanced, and the GPU context intact (a one-rank barrier afterwards completes)."""
    import ctypes

    from residualquant_b200 import _lib

    lib = _lib.load()
    flags = torch.zeros(2, _lib.RQ_MAX_PEERS, dtype=torch.int32, device="cuda")
    state = torch.zeros(64, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    a = _lib.RqPeerBarrierArgs()
    a.world, a.rank = 2, 0
    a.flags[0], a.flags[1] = flags[0].data_ptr(), flags[1].data_ptr()
    a.state = state.data_ptr()
    a.timeout_ns = 1_000_000            # one millisecond
    a.stream = torch.cuda.current_stream().cuda_stream
    assert lib.rq_peer_barrier(ctypes.byref(a)) == 0
    assert lib.rq_peer_barrier_status(state.data_ptr(), a.stream) == -5
    assert b"did not reach barrier" in lib.rq_last_error()
    assert state[0].item() == 1 and flags[1, 0].item() == 1          # the epoch advanced and was published
    state[1] = 0
    b = _lib.RqPeerBarrierArgs()
    b.world, b.rank = 1, 0
    b.flags[0] = flags[0].data_ptr()
    b.state = state.data_ptr()
    b.stream = a.stream
    assert lib.rq_peer_barrier(ctypes.byref(b)) == 0
    assert lib.rq_peer_barrier_status(state.data_ptr(), b.stream) == 0
    assert state[0].item() == 2


def test_early_start_is_withdrawn_right_after_a_write_to_the_same_cache():
    """quantize then attention on the SAME cache, back to back on one stream with the stable-metadata promise given: the
    library must notice that the pages were just written and keep the attention kernel behind the quantizer."""
    from residualquant_b200 import _cuda

    case = helpers.make_case(47, 128, 4, [900, 31], 32, 16)
    L = case.layout
    records = [list(r) for r in L.records]
    kr, vr = G.device_rotations(case)
    cache_np = helpers.oracle_cache(case)
    want = helpers.oracle_attention(case, cache_np, 2)
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    slots = torch.from_numpy(case.slots).cuda()
    rows = len(case.seq_lens)
    q = G.bf16(case.query)
    k, v = G.bf16(case.keys[2][case.live_rows]), G.bf16(case.values[2][case.live_rows])
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    cache = torch.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), 0xFF, dtype=torch.uint8, device="cuda")
    out = torch.zeros_like(q)
    torch.cuda.synchronize()
    _cuda.set_stable_metadata(True)
    try:
        _cuda.quantize(pairs, cache, slots, kr, vr, None, records, "anchor", 3, "ls")
        _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, records, "anchor", 3, 2)
    finally:
        _cuda.set_stable_metadata(False)
    torch.cuda.synchronize()
    assert _inside(out.float().cpu().numpy(), want)


def test_one_workspace_serves_calls_of_different_shapes():
    """Partial results that a small call leaves behind must never sit where a later, larger call keeps its arrival
    counters (which have to read zero): alternate a few-row call that splits every row with a many-row call."""
    from residualquant_b200 import _cuda

    small = helpers.make_case(48, 128, 2, [700, 40, 333], 32, 16)
    rng = np.random.default_rng(9)
    large = helpers.make_case(49, 128, 8, [int(v) for v in rng.integers(2, 300, size=96)], 32, 16)
    caches = {}
    for name, case in (("small", small), ("large", large)):
        cache = G.gpu_cache(case)
        caches[name] = (cache, helpers.oracle_attention(case, cache.cpu().numpy(), 0))
    for round_ in range(2):
        _cuda.set_attention_splits(7)
        try:
            got = G.gpu_attention(small, caches["small"][0], 0).float().cpu().numpy()
        finally:
            _cuda.set_attention_splits(0)
        assert _inside(got, caches["small"][1]), f"small call, round {round_}"
        got = G.gpu_attention(large, caches["large"][0], 0).float().cpu().numpy()
        assert _inside(got, caches["large"][1]), f"large call, round {round_}"


@pytest.mark.parametrize("seed,requests,equal", [(1, 7, False), (2, 70, False), (3, 150, False), (4, 33, True), (5, 130, True)])
def test_random_batches_with_several_rows_per_request(seed, requests, equal):
    """The work lookup on batches the other tests do not reach: 0 to 3 query rows per request (a request without rows must
    cost no work item, several rows share their request's history), more than 64 and more than 128 requests (second and
    third sweep of the lookup), and batches of equal lengths (the partition count is then chosen without sums over the
    requests).  Every row must come out as with one forced partition per row, which the other tests pin to the oracle."""
    from residualquant_b200 import _cuda

    rng = np.random.default_rng(100 + seed)
    if equal:
        lengths = [int(rng.integers(40, 900))] * requests
    else:
        lengths = [int(v) for v in rng.integers(1, 500, size=requests)]
        lengths[int(rng.integers(requests))] = 3000
    case = helpers.make_case(60 + seed, 128, 2, lengths, 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    rows_of = rng.integers(0, 4, size=requests) if not equal else np.full(requests, 2)
    rows_of[0] = max(rows_of[0], 1)
    starts = np.concatenate([[0], np.cumsum(rows_of)]).astype(np.int32)
    total = int(starts[-1])
    L = case.layout
    kr, vr = G.device_rotations(case)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(total, 2, 128, device="cuda", generator=gen).bfloat16()
    k = torch.randn(total, 2, 128, device="cuda", generator=gen).bfloat16()
    v = torch.randn(total, 2, 128, device="cuda", generator=gen).bfloat16()
    qsl = torch.from_numpy(starts).cuda()
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    outputs = {}
    for splits in (0, 1, -8):
        _cuda.set_attention_splits(splits)
        try:
            out = torch.full_like(q, 768.0)
            _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, [list(r) for r in L.records],
                            L.reference_mode, L.anchor_index, 1)
            torch.cuda.synchronize()
            _cuda.attention_status("cuda")
            outputs[splits] = out.float().cpu().numpy()
        finally:
            _cuda.set_attention_splits(0)
    want = outputs[1]
    assert np.all(np.abs(want) < 700.0), "every row was written"
    for splits in (0, -8):
        assert _inside(outputs[splits], want), f"num_splits {splits}: {np.abs(outputs[splits] - want).max()}"
