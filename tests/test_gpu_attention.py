"""Packed paged decode attention on the GPU against the CPU oracle.

Tolerance (stated by the task for bf16 outputs): |got - want| <= 2e-2 + 1e-2 * |want| on every element."""

import numpy as np
import pytest
import torch

from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-2, 1e-2


def _check(case, cache_np, loop, splits=0, pad_rows=0):
    from residualquant_b200 import _cuda

    cache = torch.from_numpy(cache_np).cuda()
    _cuda.set_attention_splits(splits)
    try:
        got = G.gpu_attention(case, cache, loop, pad_rows=pad_rows).float().cpu().numpy()
    finally:
        _cuda.set_attention_splits(0)
    want = helpers.oracle_attention(case, cache_np, loop)
    rows = len(case.seq_lens)
    err = np.abs(got[:rows] - want)
    bound = ATOL + RTOL * np.abs(want)
    assert np.all(err <= bound), f"loop {loop} splits {splits}: max err {err.max():.4f}, worst excess {np.max(err - bound):.4f}"
    if pad_rows:
        assert np.all(got[rows:] == 768.0), "padding rows must stay untouched"
    return err.max()


@pytest.mark.parametrize("head_dim,group,page", [(128, 32, 16), (128, 16, 16), (128, 32, 32), (128, 16, 32),
                                                 (96, 32, 16), (96, 16, 16), (96, 32, 32)])
def test_all_loops_match_oracle(head_dim, group, page):
    case = helpers.make_case(31, head_dim, 3, [300, 1, 2, 17, 64, 129], group, page)
    cache = helpers.oracle_cache(case)
    for loop in range(4):
        _check(case, cache, loop)


@pytest.mark.parametrize("splits", [1, 2, 3, 7, 16])
def test_partition_counts(splits):
    case = helpers.make_case(32, 128, 2, [700, 40, 1, 333], 32, 16)
    cache = helpers.oracle_cache(case)
    for loop in (1, 3):
        _check(case, cache, loop, splits=splits)


@pytest.mark.parametrize("head_dim", [128, 96])
def test_with_key_mean(head_dim):
    case = helpers.make_case(33, head_dim, 2, [150, 31], 32, 16, with_mean=True)
    cache = helpers.oracle_cache(case)
    for loop in range(4):
        _check(case, cache, loop, splits=2)


def test_rotation_variants():
    # value rotation absorbed by the model's weights (None), or no rotation at all
    for rk, rv in ((True, False), (False, False)):
        case = helpers.make_case(34, 128, 2, [90, 200], 32, 16, rotate_keys=rk, rotate_values=rv)
        cache = helpers.oracle_cache(case)
        for loop in (0, 3):
            _check(case, cache, loop)


def test_padding_rows_are_left_untouched():
    case = helpers.make_case(35, 128, 2, [60, 75], 32, 16)
    cache = helpers.oracle_cache(case)
    _check(case, cache, 2, pad_rows=3)
    _check(case, cache, 2, splits=4, pad_rows=3)


def test_long_context_full_shape():
    """BASELINE shape of one layer: 16 heads x 128, block 16, context 2048 (config 0) for every loop."""
    case = helpers.make_case(36, 128, 16, [2048], 32, 16)
    cache = helpers.oracle_cache(case)
    for loop in range(4):
        _check(case, cache, loop)


def test_gpu_written_cache_feeds_attention():
    """quantize -> attention end to end on the device, against the oracle fed the same raw rows."""
    case = helpers.make_case(37, 128, 4, [513, 77], 16, 16)
    cache_gpu = G.gpu_cache(case)
    cache_np = helpers.oracle_cache(case)
    assert np.array_equal(cache_gpu.cpu().numpy(), cache_np)
    for loop in range(4):
        got = G.gpu_attention(case, cache_gpu, loop).float().cpu().numpy()
        want = helpers.oracle_attention(case, cache_np, loop)
        assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want))


def test_cuda_graph_replay_follows_changed_metadata():
    """One captured decode step (attention of 4 loops + the group's quantize) replayed after the sequence
    lengths, block table and slot mapping changed on the device (reference: FULL_DECODE_ONLY capture,
    experiments/kv_memory_latency/measure.py:249-253)."""
    from residualquant_b200 import _cuda

    case = helpers.make_case(38, 128, 4, [200, 90], 32, 16)
    L = case.layout
    records = [list(r) for r in L.records]
    kr, vr = G.device_rotations(case)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    r = len(case.seq_lens)
    q = G.bf16(case.query)
    live_k = [G.bf16(k[case.live_rows]) for k in case.keys]
    live_v = [G.bf16(v[case.live_rows]) for v in case.values]
    outs = [torch.zeros_like(q) for _ in range(4)]
    qsl = torch.arange(r + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    live_slots = torch.tensor(
        [int(case.block_table[i, (case.seq_lens[i] - 1) // 16]) * 16 + (case.seq_lens[i] - 1) % 16 for i in range(r)],
        dtype=torch.int64, device="cuda")

    def step():
        for loop in range(4):
            _cuda.attention(q, live_k[loop], live_v[loop], cache, outs[loop], qsl, seq, table, kr, vr, None,
                            records, "anchor", 3, loop)
        _cuda.quantize(list(zip(live_k, live_v)), cache, live_slots, kr, vr, None, records, "anchor", 3, "ls")

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())   # the inputs were created on the default stream
    with torch.cuda.stream(side):
        step()                                   # warm-up: creates the workspace outside capture
    side.synchronize()
    cache.copy_(torch.from_numpy(helpers.oracle_cache(case)).cuda())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    graph.replay()
    torch.cuda.synchronize()
    cache_np = helpers.oracle_cache(case)
    for loop in range(4):
        want = helpers.oracle_attention(case, cache_np, loop)
        got = outs[loop].float().cpu().numpy()
        assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want))
    # the step wrote the live token into the cache: now it is history.  Advance every request by one token.
    from oracle import rq_oracle as O
    okr, ovr = helpers.oracle_rotations(case)
    O.quantize([(k[case.live_rows], v[case.live_rows]) for k, v in zip(case.keys, case.values)], cache_np,
               live_slots.cpu().numpy(), L, okr, ovr, None)
    assert np.array_equal(cache.cpu().numpy(), cache_np)
    seq += 1
    new_slots = []
    for i in range(r):
        pos = int(case.seq_lens[i])              # position of the new live token
        new_slots.append(int(case.block_table[i, pos // 16]) * 16 + pos % 16)
    live_slots.copy_(torch.tensor(new_slots, dtype=torch.int64))
    graph.replay()
    torch.cuda.synchronize()
    grown = helpers.make_case(38, 128, 4, [200, 90], 32, 16)
    grown.seq_lens = case.seq_lens + 1
    for loop in range(4):
        want = O.attention(case.query, case.keys[loop][case.live_rows], case.values[loop][case.live_rows], cache_np,
                           np.arange(r + 1, dtype=np.int32), grown.seq_lens, case.block_table, L, loop, okr, ovr, None)
        got = outs[loop].float().cpu().numpy()
        assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want))
    _cuda.attention_status()


def test_argument_errors_raise_runtime_error():
    from residualquant_b200 import _cuda

    case = helpers.make_case(39, 128, 2, [20], 32, 16)
    L = case.layout
    records = [list(r) for r in L.records]
    kr, vr = G.device_rotations(case)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    q = G.bf16(case.query)
    out = torch.zeros_like(q)
    qsl = torch.arange(2, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    ok = (q, q, q, cache, out, qsl, seq, table, kr, vr, None, records, "anchor", 3, 0)

    def call(**changes):
        names = ["query", "key", "value", "kv_cache", "output", "query_start_loc", "seq_lens", "block_table",
                 "key_rotation", "value_rotation", "key_mean", "records", "reference_mode", "anchor_index", "loop_index"]
        kwargs = dict(zip(names, ok))
        kwargs.update(changes)
        _cuda.attention(**kwargs)

    call()
    with pytest.raises(RuntimeError, match="Invalid loop index"):
        call(loop_index=4)
    with pytest.raises(RuntimeError, match="matching shapes"):
        call(key=q[:, :1].contiguous())
    with pytest.raises(RuntimeError, match="INT32 sequence lengths"):
        call(seq_lens=seq.long())
    with pytest.raises(RuntimeError, match="query starts"):
        call(query_start_loc=qsl[:1])
    with pytest.raises(RuntimeError, match="page table"):
        call(block_table=table.long())
    five = torch.zeros((2, case.num_blocks, case.heads, 16, 5 * 42), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="more than 4 records"):
        call(records=[[2, 32]] * 5, anchor_index=0, reference_mode="adjacent", loop_index=1, kv_cache=five)
    other = torch.zeros((2, case.num_blocks, case.heads, 16, 328), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError, match="No compiled packed CUDA kernel"):
        call(records=[[4, 16]] * 4, loop_index=0, kv_cache=other)


def test_large_value_magnitudes_stay_accurate_and_finite():
    """V four times larger than the benchmark distribution (group ranges of ~100) stays inside the half2
    accumulation range: the error scales with the data, so the absolute part of the tolerance is scaled by the same
    factor.  Absurd magnitudes (FP8 parameters saturated) must at least give finite outputs."""
    case = helpers.make_case(40, 128, 2, [260, 33], 32, 16)
    for rows in case.values:
        rows *= 4.0                                    # bf16-exact scaling; ranges of ~100 in outlier groups
    cache = helpers.oracle_cache(case)
    for loop in (0, 3):
        cache_t = torch.from_numpy(cache).cuda()
        got = G.gpu_attention(case, cache_t, loop).float().cpu().numpy()
        want = helpers.oracle_attention(case, cache, loop)
        assert np.all(np.abs(got - want) <= 4.0 * ATOL + RTOL * np.abs(want))
    huge = helpers.make_case(41, 128, 2, [70], 32, 16)
    for rows in huge.values:
        rows *= 256.0
    cache = helpers.oracle_cache(huge)
    out = G.gpu_attention(huge, torch.from_numpy(cache).cuda(), 0).float()
    assert torch.isfinite(out).all()


def test_decode_step_through_the_group_mirror():
    """Four loop slots of one group: attention per loop, K/V held back, one quantize on the last loop
    (reference: packed_backend.py:28-137, install_model.py:40-52)."""
    from oracle import rq_oracle as O
    from residualquant_b200.group import DeferredKVGroup, PackedDecodeAttention

    case = helpers.make_case(42, 128, 4, [150, 47], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    group = DeferredKVGroup(L.records, L.page_tokens)
    slots = [PackedDecodeAttention(group, i, kr, vr) for i in range(4)]
    cache_np = helpers.oracle_cache(case)
    cache = torch.from_numpy(cache_np).cuda()
    r = len(case.seq_lens)
    qsl = torch.arange(r + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    live_slots = torch.tensor(
        [int(case.block_table[i, (case.seq_lens[i] - 1) // 16]) * 16 + (case.seq_lens[i] - 1) % 16 for i in range(r)],
        dtype=torch.int64, device="cuda")
    q = G.bf16(case.query)
    for loop in range(4):
        k = G.bf16(case.keys[loop][case.live_rows])
        v = G.bf16(case.values[loop][case.live_rows])
        out = slots[loop].forward(q, k, v, cache, qsl, seq, table, live_slots, torch.zeros_like(q))
        torch.cuda.synchronize()
        want = helpers.oracle_attention(case, cache_np, loop)
        assert np.all(np.abs(out.float().cpu().numpy() - want) <= ATOL + RTOL * np.abs(want))
        assert len(group.pending) == (loop + 1) % 4
    okr, ovr = helpers.oracle_rotations(case)
    O.quantize([(k[case.live_rows], v[case.live_rows]) for k, v in zip(case.keys, case.values)], cache_np,
               live_slots.cpu().numpy(), L, okr, ovr, None)
    assert np.array_equal(cache.cpu().numpy(), cache_np)


@pytest.mark.parametrize("records,anchor", [
    (((4, 32), (4, 32), (4, 32), (4, 32)), 3),      # "4444"
    (((2, 32), (2, 32), (2, 32), (2, 32)), 3),      # "2222" g32
    (((2, 16), (2, 16), (2, 16), (2, 16)), 0),      # "2222" g16, anchor first
    (((4, 32), (2, 32), (2, 32), (2, 32)), 0),      # "4222", anchor first
    (((4, 32), (2, 16), (2, 16), (2, 16)), 0),
    (((4, 32),), 0),
    (((2, 32),), 0),
    (((4, 32), (2, 32), (2, 32), (2, 32)), 3),      # "4222" with the anchor last: INT2 anchor, INT4 first loop
    (((4, 32), (2, 16), (2, 16), (2, 16)), 3),
    (((2, 32), (2, 32), (2, 32), (4, 32)), 0),      # "2224" with the anchor first
])
@pytest.mark.parametrize("head_dim", [128, 96])
def test_other_schedules_of_the_registry(records, anchor, head_dim):
    """Every (anchor record, loop record) pair of the reference's anchor-mode schedule lists
    (dispatch/decode_*_anchor_{0,3}_g{16,32}.cu)."""
    case = helpers.make_case(43, head_dim, 2, [170, 18], records=records, anchor_index=anchor, with_mean=(head_dim == 96))
    cache = helpers.oracle_cache(case)
    for loop in range(len(records)):
        _check(case, cache, loop, splits=2 if loop % 2 else 0)


@pytest.mark.parametrize("records", [
    ((2, 32), (2, 32), (2, 32), (2, 32)),
    ((4, 32), (2, 16), (2, 16), (2, 16)),
    ((2, 32), (2, 32), (2, 32), (4, 32)),
    ((4, 32), (4, 32), (4, 32), (4, 32)),
])
@pytest.mark.parametrize("head_dim,page", [(128, 16), (96, 32)])
def test_adjacent_reference_mode(records, head_dim, page):
    """Adjacent mode: loop r is restored as alpha_r * (loop r-1) + residual_r, a chain over records 0..r
    (reference: attention/compute.cuh:123-197, dispatch/decode_*_adjacent_0_g{16,32}.cu)."""
    case = helpers.make_case(44, head_dim, 2, [140, 35, 1], page_tokens=page, records=records, anchor_index=0,
                             reference_mode="adjacent", with_mean=(head_dim == 128))
    cache = helpers.oracle_cache(case)
    for loop in range(4):
        _check(case, cache, loop, splits=3 if loop == 2 else 0)


@pytest.mark.parametrize("fill", [0xFF, 0x7F, 0xA5])
@pytest.mark.parametrize("head_dim,page,mode", [(128, 16, "anchor"), (96, 32, "anchor"), (128, 16, "adjacent"), (96, 16, "adjacent")])
def test_unwritten_bytes_of_the_last_page_are_ignored(fill, head_dim, page, mode):
    """Tokens beyond the history share the last page with real ones; their bytes were never written and may decode to
    NaN (FP8 0x7F / 0xFF, bf16 0xFFFF) or huge values.  They must not reach the output."""
    if mode == "anchor":
        case = helpers.make_case(51, head_dim, 2, [45, 3, 130, 1], 32, page)
    else:
        case = helpers.make_case(52, head_dim, 2, [45, 3, 130, 1], page_tokens=page, anchor_index=0,
                                 records=((4, 32), (2, 16), (2, 32), (2, 32)), reference_mode="adjacent")
    cache = helpers.oracle_cache(case, fill=fill)
    for loop in range(4):
        _check(case, cache, loop, splits=2 if loop == 1 else 0)


@pytest.mark.parametrize("sharpness", [3.0, 8.0])
def test_sharp_queries(sharpness):
    """Queries with a large norm: the softmax concentrates on a few tokens and the score range grows."""
    import dataclasses

    case = helpers.make_case(53, 128, 2, [600, 90], 32, 16)
    query = (case.query.astype(np.float32) * sharpness)
    from residualquant_b200 import synth
    case = dataclasses.replace(case, query=synth.to_bf16_f32(query))
    cache = helpers.oracle_cache(case)
    for loop in range(4):
        _check(case, cache, loop, splits=2 if loop == 0 else 0)


@pytest.mark.parametrize("offload_chunk", [0, 8])
def test_mixed_batch_of_decodes_and_a_full_prompt(offload_chunk):
    """Two decode requests followed by a 21-token prompt in one batch (the reordered batch of the reference's metadata
    builder, packed_backend.py:153-199): decode rows go through the packed kernel, the prompt through the prefill
    attention, and the group's quantize writes the new K/V of all 23 tokens -- directly, or with the held-back loops
    parked in pinned host memory and streamed back 8 tokens at a time (prefill_offload.py of the reference)."""
    from oracle import rq_oracle as O
    from residualquant_b200 import synth
    from residualquant_b200.group import DeferredKVGroup, PackedAttention

    case = helpers.make_case(45, 128, 4, [150, 47], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    from residualquant_b200.prefill_offload import PrefillHostStage

    stage = PrefillHostStage(offload_chunk) if offload_chunk else None
    group = DeferredKVGroup(L.records, L.page_tokens, prefill_offload=stage)
    slots = [PackedAttention(group, i, kr, vr) for i in range(4)]
    # room for the prompt: three fresh blocks after the case's own
    prompt = 21
    extra = 3
    cache_np = np.concatenate([helpers.oracle_cache(case),
                               np.zeros((2, extra) + helpers.oracle_cache(case).shape[2:], np.uint8)], axis=1)
    cache = torch.from_numpy(cache_np).cuda()
    first_new = case.num_blocks
    table_np = np.zeros((3, case.block_table.shape[1]), np.int32)
    table_np[:2] = case.block_table
    table_np[2, :extra] = np.arange(first_new, first_new + extra)
    table = torch.from_numpy(table_np).cuda()
    seq_np = np.array([case.seq_lens[0], case.seq_lens[1], prompt], np.int32)
    starts_np = np.array([0, 1, 2, 2 + prompt], np.int32)
    live = [int(case.block_table[i, (case.seq_lens[i] - 1) // 16]) * 16 + (case.seq_lens[i] - 1) % 16 for i in range(2)]
    prompt_slots = [int(table_np[2, t // 16]) * 16 + t % 16 for t in range(prompt)]
    slot_mapping = torch.tensor(live + prompt_slots, dtype=torch.int64, device="cuda")

    rng = np.random.default_rng(9)
    prompt_q = synth.to_bf16_f32(rng.standard_normal((prompt, 4, 128)).astype(np.float32))
    prompt_k = [synth.to_bf16_f32(rng.standard_normal((prompt, 4, 128)).astype(np.float32)) for _ in range(4)]
    prompt_v = [synth.to_bf16_f32(rng.standard_normal((prompt, 4, 128)).astype(np.float32)) for _ in range(4)]
    q = torch.cat([G.bf16(case.query), G.bf16(prompt_q)])
    all_k, all_v = [], []
    for loop in range(4):
        k = torch.cat([G.bf16(case.keys[loop][case.live_rows]), G.bf16(prompt_k[loop])])
        v = torch.cat([G.bf16(case.values[loop][case.live_rows]), G.bf16(prompt_v[loop])])
        all_k.append(k)
        all_v.append(v)
        out = slots[loop].forward_batch(q, k, v, cache, torch.from_numpy(starts_np).cuda(), torch.from_numpy(seq_np).cuda(),
                                        table, slot_mapping, torch.zeros_like(q), starts_np.tolist(), seq_np.tolist())
        torch.cuda.synchronize()
        want = helpers.oracle_attention(case, cache_np[:, :case.num_blocks], loop)
        got = out.float().cpu().numpy()
        assert np.all(np.abs(got[:2] - want) <= ATOL + RTOL * np.abs(want))
        # the prompt rows are plain causal attention over the raw rows
        scores = np.einsum("thd,shd->hts", prompt_q, prompt_k[loop]) / np.sqrt(128.0)
        scores = np.where(np.triu(np.ones((prompt, prompt), bool), 1)[None], -np.inf, scores)
        p = np.exp(scores - scores.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        ref = np.einsum("hts,shd->thd", p, prompt_v[loop])
        assert np.all(np.abs(got[2:] - ref) <= ATOL + RTOL * np.abs(ref))
        if stage is not None and loop < 3:
            assert not group.pending[loop][0].is_cuda and group.pending[loop][0].is_pinned()
    okr, ovr = helpers.oracle_rotations(case)
    pairs = [(k.float().cpu().numpy(), v.float().cpu().numpy()) for k, v in zip(all_k, all_v)]
    O.quantize(pairs, cache_np, slot_mapping.cpu().numpy(), L, okr, ovr, None)
    assert np.array_equal(cache.cpu().numpy(), cache_np)
