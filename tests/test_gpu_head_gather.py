"""Fused head gather on one GPU: the attention kernel stores its rows into a gathered buffer at a head offset and the
barrier kernel of a one-rank world completes; the barrier-free forms, in which the kernel publishes its own completion
and either the next call waits for it or the call itself stays until every rank has published.  (Several ranks: tests/test_gpu_head_gather_multi.py, which needs two GPUs.)"""

import numpy as np
import pytest
import torch

from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu


class _OffsetGather:
    """A HeadGather whose local heads sit in the middle of wider gathered rows, as on rank 1 of 3."""

    def __init__(self, inner, heads_before, heads_after):
        from residualquant_b200 import sharding

        self.inner = inner
        self.rows, self.head_dim = inner.rows, inner.head_dim
        self.local_heads = inner.heads - heads_before - heads_after
        self.heads = inner.heads
        self.head_offset = heads_before
        assert sharding.shard_counts(self.heads, 1) == [self.heads]

    def peer_pointers(self, buffer):
        return self.inner.peer_pointers(buffer)


def test_rows_land_in_the_gathered_buffer_and_barrier_completes():
    from residualquant_b200 import _cuda, sharding

    case = helpers.make_case(71, 128, 2, [90, 33, 1], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    rows = len(case.seq_lens)
    gather = sharding.HeadGather(rows, case.heads + 3, 128, "cuda", buffers=2)
    try:
        view = _OffsetGather(gather, heads_before=2, heads_after=1)
        L = case.layout
        kr, vr = G.device_rotations(case)
        for loop, buffer in ((1, 0), (3, 1)):
            q = G.bf16(case.query)
            k = G.bf16(case.keys[loop][case.live_rows])
            v = G.bf16(case.values[loop][case.live_rows])
            out = torch.zeros_like(q)
            _cuda.attention(q, k, v, cache, out, torch.arange(rows + 1, dtype=torch.int32, device="cuda"),
                            torch.from_numpy(case.seq_lens).cuda(), torch.from_numpy(case.block_table).cuda(),
                            kr, vr, None, [list(r) for r in L.records], L.reference_mode, L.anchor_index, loop,
                            gather=view, gather_buffer=buffer)
            gather.barrier()
            gather.check()
            _cuda.attention_status("cuda")
            full = gather.gathered(buffer)
            assert torch.equal(full[:, 2:2 + case.heads], out)
            assert torch.count_nonzero(full[:, :2]) == 0 and torch.count_nonzero(full[:, 2 + case.heads:]) == 0
            want = helpers.oracle_attention(case, cache.cpu().numpy(), loop)
            err = np.abs(out.float().cpu().numpy() - want)
            assert np.all(err <= 2e-2 + 1e-2 * np.abs(want))
        # the epoch advanced once per barrier and no wait timed out
        assert gather.state[:2].tolist() == [2, 0]
    finally:
        gather.close()


def test_gather_arguments_are_checked():
    from residualquant_b200 import _cuda, sharding

    case = helpers.make_case(72, 128, 1, [20], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    gather = sharding.HeadGather(1, case.heads + 1, 128, "cuda", buffers=1)   # one rank, but one head too many
    try:
        q = G.bf16(case.query)
        with pytest.raises(RuntimeError, match="gathered output"):
            _cuda.attention(q, q, q, cache, torch.zeros_like(q), torch.arange(2, dtype=torch.int32, device="cuda"),
                            torch.from_numpy(case.seq_lens).cuda(), torch.from_numpy(case.block_table).cuda(),
                            None, None, None, [list(r) for r in case.layout.records], "anchor", 3, 0, gather=gather)
        with pytest.raises(ValueError):
            gather.peer_pointers(1)
    finally:
        gather.close()


def test_kernel_published_completion_replaces_the_barrier():
    """Signalled gather: no barrier kernel between calls.  Every call advances the epoch from inside the kernel (last CTA)
    and publishes it; the following call waits for it before reading its inputs; the consumer-side wait at the end
    finds the last epoch in place."""
    from residualquant_b200 import _cuda, sharding

    case = helpers.make_case(73, 128, 3, [300, 33, 1, 90], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    rows = len(case.seq_lens)
    gather = sharding.HeadGather(rows, case.heads, 128, "cuda", buffers=2, signalled=True)
    try:
        L = case.layout
        kr, vr = G.device_rotations(case)
        q = G.bf16(case.query)
        qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
        seq = torch.from_numpy(case.seq_lens).cuda()
        table = torch.from_numpy(case.block_table).cuda()
        outs = []
        for call, loop in enumerate((0, 1, 2, 3, 0, 3)):
            k = G.bf16(case.keys[loop][case.live_rows])
            v = G.bf16(case.values[loop][case.live_rows])
            out = torch.zeros_like(q)
            _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, [list(r) for r in L.records],
                            L.reference_mode, L.anchor_index, loop, gather=gather, gather_buffer=call % 2)
            outs.append((loop, call % 2, out))
        gather.barrier()         # wait only
        gather.check()
        torch.cuda.synchronize()
        assert gather.state[:3].tolist() == [6, 0, 0]          # six epochs published, no timeout, counter back at zero
        flags = gather._bytes[gather.flag_offset: gather.flag_offset + 4].view(torch.int32)
        assert int(flags[0]) == 6
        for loop, buffer, out in outs[-2:]:
            assert torch.equal(gather.gathered(buffer), out)
            want = helpers.oracle_attention(case, cache.cpu().numpy(), loop)
            assert np.all(np.abs(out.float().cpu().numpy() - want) <= 2e-2 + 1e-2 * np.abs(want))
    finally:
        gather.close()


def _run_calls(case, cache, gather, loops, after_each=None):
    from residualquant_b200 import _cuda

    rows = len(case.seq_lens)
    L = case.layout
    kr, vr = G.device_rotations(case)
    q = G.bf16(case.query)
    qsl = torch.arange(rows + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    outs = []
    for call, loop in enumerate(loops):
        k = G.bf16(case.keys[loop][case.live_rows])
        v = G.bf16(case.values[loop][case.live_rows])
        out = torch.zeros_like(q)
        _cuda.attention(q, k, v, cache, out, qsl, seq, table, kr, vr, None, [list(r) for r in L.records],
                        L.reference_mode, L.anchor_index, loop, gather=gather, gather_buffer=call % 2)
        if after_each is not None:
            after_each(call)
        outs.append((loop, call % 2, out))
    return outs


def test_call_ends_only_when_the_gathered_rows_are_complete():
    """Complete form: no barrier and no wait in the next call.  Whatever follows a call on the stream reads the complete
    gathered buffer: here a plain copy queued right behind every call, compared with that call's own output."""
    from residualquant_b200 import sharding

    case = helpers.make_case(74, 128, 3, [300, 33, 1, 90], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    rows = len(case.seq_lens)
    gather = sharding.HeadGather(rows, case.heads, 128, "cuda", buffers=2, complete=True)
    try:
        snapshots = []
        outs = _run_calls(case, cache, gather, (0, 1, 2, 3, 0, 3),
                          after_each=lambda call: snapshots.append(gather.gathered(call % 2).clone()))
        gather.barrier()         # nothing to launch in this form
        gather.check()
        torch.cuda.synchronize()
        assert gather.state[:3].tolist() == [6, 0, 0]          # six epochs, no timeout, ticket counter back at zero
        for (loop, _, out), seen in zip(outs, snapshots):
            assert torch.equal(seen, out)
            want = helpers.oracle_attention(case, cache.cpu().numpy(), loop)
            assert np.all(np.abs(out.float().cpu().numpy() - want) <= 2e-2 + 1e-2 * np.abs(want))
    finally:
        gather.close()


class _AbsentPeer:
    """A complete-form gather that claims a second rank which never publishes: both "ranks" are this GPU's own
    allocation, slot 1 of the flag array is written by nobody."""

    complete, signalled, rank = True, False, 0
    timeout_ns = 20_000_000   # 20 ms

    def __init__(self, inner):
        self.inner = inner
        self.rows, self.heads, self.head_dim = inner.rows, inner.heads, inner.head_dim
        self.local_heads, self.head_offset, self.state = inner.heads, 0, inner.state

    def peer_pointers(self, buffer):
        return self.inner.peer_pointers(buffer) * 2

    def flag_pointers(self):
        return self.inner.flag_pointers() * 2


def test_wait_for_an_absent_rank_runs_out_and_reports():
    """The wait at the end of a complete-form call is bounded: with a peer that never publishes the kernel gives up after
    its limit, the call still returns its rows, and the state block holds the timeout status for the host to read."""
    from residualquant_b200 import sharding

    case = helpers.make_case(75, 128, 2, [40, 17], 32, 16)
    cache = torch.from_numpy(helpers.oracle_cache(case)).cuda()
    gather = sharding.HeadGather(len(case.seq_lens), case.heads, 128, "cuda", buffers=2, complete=True)
    try:
        (loop, buffer, out), = _run_calls(case, cache, _AbsentPeer(gather), (0,))
        torch.cuda.synchronize()
        assert torch.equal(gather.gathered(buffer), out)
        assert gather.state[:3].tolist() == [1, -5, 0]             # RQ_ERR_DEVICE_TIMEOUT
        with pytest.raises(RuntimeError):
            gather.check()
    finally:
        gather.close()
