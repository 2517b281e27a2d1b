"""Fused head gather on one GPU: the attention kernel stores its rows into a gathered buffer at a head offset and the
barrier kernel of a one-rank world completes (the multi-rank form needs several GPUs and is exercised by
`bench.py --shard heads` under torchrun)."""

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
