"""Arbitrary learned (dense fp16) rotations: rows are rotated on the tensor cores (TF32 products, fp32 sums) in
front of the quantizer and the attention kernel.  The oracle rotates in float64; the summation order of the hardware
differs, so a code sitting on a rounding boundary may land on either side: packed bytes must agree almost everywhere
and attention must stay inside the usual tolerance (reference: common/api.h:42-55, quantize/rotation.cuh:25-150,
attention/prepare.cuh:61-145, merge.cuh:74-79)."""

import numpy as np
import pytest
import torch

from oracle import rq_oracle as O
from residualquant_b200 import _cuda
from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu


def _random_rotations(rng, heads, dim):
    mats = []
    for _ in range(heads):
        q, _ = np.linalg.qr(rng.standard_normal((dim, dim)))
        mats.append(q)
    return np.stack(mats).astype(np.float16)          # what a calibrated artifact holds: fp16 [heads, D, D]


@pytest.mark.parametrize("head_dim,group", [(128, 32), (96, 16)])
def test_dense_rotation_quantize_and_attention(head_dim, group):
    rng = np.random.default_rng(5)
    case = helpers.make_case(51, head_dim, 3, [130, 41, 1], group, 16, rotate_keys=False, rotate_values=False)
    L = case.layout
    rk, rv = _random_rotations(rng, case.heads, head_dim), _random_rotations(rng, case.heads, head_dim)
    want = np.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), 0xA5, dtype=np.uint8)
    O.quantize(list(zip(case.keys, case.values)), want, case.slots, L, rk.astype(np.float32), rv.astype(np.float32), None)

    records = [list(r) for r in L.records]
    rk_t, rv_t = torch.from_numpy(rk).cuda(), torch.from_numpy(rv).cuda()
    cache = torch.full(want.shape, 0xA5, dtype=torch.uint8, device="cuda")
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    _cuda.quantize(pairs, cache, torch.from_numpy(case.slots).cuda(), rk_t, rv_t, None, records, "anchor", 3, "ls")
    torch.cuda.synchronize()
    got = cache.cpu().numpy()
    assert np.mean(got != want) < 0.01, f"{np.mean(got != want):.4f} of the packed bytes differ"
    # untouched bytes (padding slots, other pages) keep the fill pattern in both
    assert np.array_equal(got == 0xA5, want == 0xA5) or np.mean((got == 0xA5) != (want == 0xA5)) < 0.01

    # attention over the ORACLE's cache with the dense key rotation and the explicit dense value rotation
    r = len(case.seq_lens)
    qsl = torch.arange(r + 1, dtype=torch.int32, device="cuda")
    seq = torch.from_numpy(case.seq_lens).cuda()
    table = torch.from_numpy(case.block_table).cuda()
    cache_t = torch.from_numpy(want).cuda()
    q = G.bf16(case.query)
    for loop in range(4):
        k = G.bf16(case.keys[loop][case.live_rows])
        v = G.bf16(case.values[loop][case.live_rows])
        for splits in (0, 3):
            _cuda.set_attention_splits(splits)
            try:
                out = torch.zeros_like(q)
                _cuda.attention(q, k, v, cache_t, out, qsl, seq, table, rk_t, rv_t, None, records, "anchor", 3, loop)
                torch.cuda.synchronize()
            finally:
                _cuda.set_attention_splits(0)
            ref = O.attention(case.query, case.keys[loop][case.live_rows], case.values[loop][case.live_rows], want,
                              np.arange(r + 1, dtype=np.int32), case.seq_lens, case.block_table, L, loop,
                              rk.astype(np.float32), rv.astype(np.float32), None)
            err = np.abs(out.float().cpu().numpy() - ref)
            assert np.all(err <= 2e-2 + 1e-2 * np.abs(ref)), f"loop {loop} splits {splits}: max err {err.max():.4f}"


def test_dense_copy_of_a_hadamard_rotation_matches_the_fused_path():
    """The same rotation given densely (unregistered) or as sign masks must produce (almost) the same cache."""
    case = helpers.make_case(52, 128, 2, [90], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    fused = G.gpu_cache(case, fill=0xA5).cpu().numpy()
    records = [list(r) for r in L.records]
    cache = torch.full(fused.shape, 0xA5, dtype=torch.uint8, device="cuda")
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    _cuda.quantize(pairs, cache, torch.from_numpy(case.slots).cuda(), kr.dense(), vr.dense(), None, records, "anchor", 3, "ls")
    torch.cuda.synchronize()
    assert np.mean(cache.cpu().numpy() != fused) < 0.01
