"""Page layout, packing and cache round trips of the oracle (CPU), including property tests."""

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import rq_oracle as O
from tests import helpers


def test_page_widths_match_the_reference_formula():
    # D*bits/8 + 2*D/group + 2 per record (reference: common/cache.cuh:14-17, install_model.py:34-38)
    assert O.PackedLayout(128, ((2, 32),) * 3 + ((4, 32),), 16, 3).page_width == 200
    assert O.PackedLayout(128, ((2, 16),) * 3 + ((4, 32),), 16, 3).page_width == 224
    assert O.PackedLayout(96, ((2, 32),) * 3 + ((4, 32),), 16, 3).page_width == 152
    assert O.PackedLayout(96, ((2, 16),) * 3 + ((4, 32),), 16, 3).page_width == 170
    lay = O.PackedLayout(128, ((2, 32),) * 3 + ((4, 32),), 16, 3)
    assert [lay.record_offset(i) for i in range(5)] == [0, 42, 84, 126, 200]
    assert [lay.record_bytes(i) for i in range(4)] == [42, 42, 42, 74]


def test_invalid_layouts_are_rejected():
    with pytest.raises(ValueError):
        O.PackedLayout(100, ((2, 32),), 16, 0)
    with pytest.raises(ValueError):
        O.PackedLayout(128, ((3, 32),), 16, 0)
    with pytest.raises(ValueError):
        O.PackedLayout(128, ((2, 32), (2, 32)), 16, 1, "adjacent")


@settings(max_examples=60, deadline=None)
@given(bits=st.sampled_from([2, 4]), seed=st.integers(0, 2**32 - 1), rows=st.integers(1, 5),
       dim=st.sampled_from([32, 96, 128]))
def test_pack_unpack_round_trip(bits, seed, rows, dim):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 1 << bits, size=(rows, dim)).astype(np.uint8)
    packed = O.pack_codes(codes, bits)
    assert packed.shape == (rows, dim * bits // 8)
    assert np.array_equal(O.unpack_codes(packed, bits, dim), codes)
    # channel c sits at bit (c%4)*bits of storage word c//4 (uint8 / little-endian uint16)
    c = int(rng.integers(0, dim))
    if bits == 2:
        assert (packed[0, c // 4] >> (2 * (c % 4))) & 3 == codes[0, c]
    else:
        word = packed[0, 2 * (c // 4)].astype(np.uint16) | (packed[0, 2 * (c // 4) + 1].astype(np.uint16) << 8)
        assert (word >> (4 * (c % 4))) & 15 == codes[0, c]


@settings(max_examples=40, deadline=None)
@given(seed=st.integers(0, 2**32 - 1), bits=st.sampled_from([2, 4]), group=st.sampled_from([16, 32]))
def test_group_quantizer_properties(seed, bits, group):
    rng = np.random.default_rng(seed)
    z = (rng.standard_normal((4, 2, 128)) * rng.uniform(0.01, 20)).astype(np.float32)
    codes, s8, o8 = O.group_quantize(z, bits, group)
    assert codes.max() <= (1 << bits) - 1
    scale = O.e4m3_decode(s8)
    assert np.all(scale >= 0)
    # decoding stays within about one step of the clipped input (fp8 parameters are coarse: 1/16 relative)
    dec = O.dequantize_group(codes, s8, o8, group)
    g = z.reshape(4, 2, 128 // group, group)
    lo, hi = g.min(-1, keepdims=True), g.max(-1, keepdims=True)
    step = np.maximum(scale[..., None], 1e-6)
    err = np.abs(dec.reshape(g.shape) - g)
    assert np.all(err <= 1.2 * step + 0.15 * (hi - lo))
    # constant groups store scale 0 and code 0
    flat = np.full((1, 1, 128), 0.75, dtype=np.float32)
    c2, s2, o2 = O.group_quantize(flat, bits, group)
    assert np.all(c2 == 0) and np.all(s2 == 0) and np.all(O.e4m3_decode(o2) == 0.75)
    zero = np.zeros((1, 1, 128), dtype=np.float32)
    zero[0, 0, ::2] = -0.0
    c3, s3, o3 = O.group_quantize(zero, bits, group)
    assert np.all(c3 == 0) and np.all(s3 == 0) and np.all(o3 == 0)


@pytest.mark.parametrize("head_dim,group,page", [(128, 32, 16), (128, 16, 32), (96, 32, 16)])
def test_cache_write_read_round_trip(head_dim, group, page):
    case = helpers.make_case(5, head_dim, 2, [37, 1, 18], group, page)
    cache = helpers.oracle_cache(case, fill=0xAB)
    kr, _ = helpers.oracle_rotations(case)
    fields = O.quantize_plane([k for k in case.keys], case.layout, kr, None)
    keep = case.slots >= 0
    for r in range(4):
        back = O.read_record(cache, 0, r, case.slots[keep], case.layout)
        assert np.array_equal(back.codes, fields[r].codes[keep])
        assert np.array_equal(back.scale8, fields[r].scale8[keep])
        assert np.array_equal(back.offset8, fields[r].offset8[keep])
        assert np.array_equal(back.alpha_bits, fields[r].alpha_bits[keep])
    assert np.all(O.read_record(cache, 0, 3, case.slots[keep], case.layout).alpha_bits == 0x3F80)
    # bytes of slots that were never written keep the fill pattern: negative slots are skipped
    P, W = case.layout.page_tokens, case.layout.page_width
    written = np.zeros(case.num_blocks * P, dtype=bool)
    written[case.slots[keep]] = True
    pages = cache.reshape(2, case.num_blocks, case.heads, P * W)
    lay = case.layout
    for block in range(case.num_blocks):
        for tok in range(P):
            if written[block * P + tok]:
                continue
            cb = lay.code_bytes(0)
            assert np.all(pages[:, block, :, tok * cb:(tok + 1) * cb] == 0xAB)


def test_attention_oracle_equals_dense_softmax():
    case = helpers.make_case(9, 128, 2, [33, 5], 32, 16)
    cache = helpers.oracle_cache(case)
    kr, vr = helpers.oracle_rotations(case)
    for loop in (0, 3):
        out = helpers.oracle_attention(case, cache, loop)
        cursor = 0
        for r, length in enumerate(case.seq_lens):
            hist = int(length) - 1
            slots = case.slots[cursor:cursor + hist]
            k_rot = O.restore_rotated(cache, 0, loop, slots, case.layout)
            v_rot = O.restore_rotated(cache, 1, loop, slots, case.layout)
            k_orig = np.einsum("the,hde->thd", k_rot, kr.dense().astype(np.float64))
            v_orig = np.einsum("the,hde->thd", v_rot, vr.dense().astype(np.float64))
            live = cursor + hist
            k_all = np.concatenate([k_orig, case.keys[loop][live:live + 1].astype(np.float64)])
            v_all = np.concatenate([v_orig, case.values[loop][live:live + 1].astype(np.float64)])
            logits = np.einsum("hd,thd->ht", case.query[r].astype(np.float64), k_all) / np.sqrt(128.0)
            p = np.exp(logits - logits.max(1, keepdims=True))
            p /= p.sum(1, keepdims=True)
            ref = np.einsum("ht,thd->hd", p, v_all)
            # the fp16-rounded rotation scale makes R R^T = (1 +- 2^-11) I: allow that much
            assert np.abs(out[r] - ref).max() < 5e-3 * max(1.0, np.abs(ref).max())
            cursor += int(length)
