"""The oracle against outputs of the reference's own PyTorch code (fixtures in tests/golden, CPU).

Inputs are regenerated from the seeds of tests/golden/make_golden.py; the fixtures hold only what the
reference computed.
"""

import os
import sys

import numpy as np
import pytest

from oracle import rq_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)
import make_golden as MG  # noqa: E402  (only its seeded input builders are used; the reference is not imported)


@pytest.mark.parametrize("dim", [128, 96])
@pytest.mark.parametrize("bits,group", [(2, 16), (2, 32), (4, 32)])
def test_group_quantizer_is_bit_exact_against_affine_qdq(dim, bits, group):
    """Reference: scripts/calibration/quantization.py:31-61 with an identity rotation."""
    fx = np.load(os.path.join(GOLDEN, f"gq_d{dim}.npz"))
    x, mean = MG.gq_inputs(dim)
    codes, s8, o8 = O.group_quantize(x, bits, group)
    mine = O.bf16_bits(O.bf16_round_from_f64(O.dequantize_group(codes, s8, o8, group)))
    assert np.array_equal(mine, fx[f"plain_{bits}_{group}"])
    z = (x - mean[None]).astype(np.float32)
    codes, s8, o8 = O.group_quantize(z, bits, group)
    restored = (O.dequantize_group(codes, s8, o8, group).astype(np.float32) + mean[None]).astype(np.float32)
    assert np.array_equal(O.bf16_bits(restored), fx[f"mean_{bits}_{group}"])


def _chain_case(dim, group, chain):
    fx = np.load(os.path.join(GOLDEN, f"chain_d{dim}_g{group}.npz"))
    k, v, signs, q = MG.chain_inputs(dim, group)
    tokens, heads = k[0].shape[:2]
    rot = O.SignedHadamard(signs, fx["rscale"])
    page = 8
    layout = O.PackedLayout(dim, ((2, group),) * 3 + ((4, 32),), page, 3)
    cache = np.zeros((2, tokens // page, heads, page, layout.page_width), dtype=np.uint8)
    O.quantize(list(zip(k, v)), cache, np.arange(tokens), layout, rot, rot, None, chain=chain)
    return fx, k, v, q, rot, layout, cache, tokens, heads


@pytest.mark.parametrize("dim,group", [(128, 32), (128, 16), (96, 32), (96, 16)])
def test_calibration_chain_tracks_fp32chain_reconstruct(dim, group):
    """Reference: scripts/calibration/rotation_training.py:46-62 (FP32Chain.reconstruct).  Not bit-comparable:
    the reference rotates with an fp32 matmul, this code with butterflies, so a code sitting on a rounding
    boundary can land on either side (one step of one rotated channel, spread over the row by the inverse
    rotation).  Everything else must agree."""
    fx, k, v, q, rot, layout, cache, tokens, heads = _chain_case(dim, group, "calibration")
    dense = rot.dense().astype(np.float64)
    for plane, rows, name in ((0, k, "k_hat"), (1, v, "v_hat")):
        for loop in range(4):
            mine = np.einsum("the,hde->thd", O.restore_rotated(cache, plane, loop, np.arange(tokens), layout), dense)
            ref = O.bf16_to_f32(fx[f"{name}_{loop}"]).astype(np.float64)
            diff = np.abs(mine - ref)
            assert np.mean(diff > 0.03) < 0.03, (plane, loop, np.mean(diff > 0.03))
            assert np.mean(diff) < 6e-3
            truth = rows[loop].astype(np.float64)
            assert abs(np.sqrt(np.mean((mine - truth) ** 2)) / np.sqrt(np.mean((ref - truth) ** 2)) - 1) < 0.02


@pytest.mark.parametrize("dim,group", [(128, 32), (128, 16), (96, 32), (96, 16)])
def test_kernel_chain_is_an_equally_good_quantizer(dim, group):
    """The CUDA-style chain forms the coefficient in rotated coordinates (kernel.cuh:76-120); it is a
    different, equally valid quantization: same anchor record, same error against the true rows."""
    fx, k, v, q, rot, layout, cache, tokens, heads = _chain_case(dim, group, "kernel")
    _, _, _, _, _, _, cache_cal, _, _ = _chain_case(dim, group, "calibration")
    P, W = layout.page_tokens, layout.page_width
    anchor_lo, anchor_hi = P * layout.record_offset(3), P * W
    pages, pages_cal = cache.reshape(2, -1, heads, P * W), cache_cal.reshape(2, -1, heads, P * W)
    assert np.array_equal(pages[..., anchor_lo:anchor_hi], pages_cal[..., anchor_lo:anchor_hi])
    dense = rot.dense().astype(np.float64)
    for loop in range(3):
        mine = np.einsum("the,hde->thd", O.restore_rotated(cache, 0, loop, np.arange(tokens), layout), dense)
        ref = O.bf16_to_f32(fx[f"k_hat_{loop}"]).astype(np.float64)
        truth = k[loop].astype(np.float64)
        assert abs(np.sqrt(np.mean((mine - truth) ** 2)) / np.sqrt(np.mean((ref - truth) ** 2)) - 1) < 0.03


@pytest.mark.parametrize("dim,group", [(128, 32), (128, 16), (96, 32), (96, 16)])
def test_decode_attention_tracks_reference_attention(dim, group):
    """Reference: rotation_math.py:44-49 (`probabilities`) followed by p @ V over the reconstructed rows, last
    token live.  With only 39 cached tokens one flipped code moves the output visibly, so the bound is the
    documented 2e-2 + 1e-2*|ref| on at least 97% of the outputs and 0.12 absolute everywhere."""
    fx, k, v, q, rot, layout, cache, tokens, heads = _chain_case(dim, group, "calibration")
    table = np.arange(tokens // layout.page_tokens, dtype=np.int32)[None]
    for loop in range(4):
        out = O.attention(q, k[loop][tokens - 1:], v[loop][tokens - 1:], cache, np.array([0, 1]), np.array([tokens]),
                          table, layout, loop, rot, rot, None)[0]
        ref = fx[f"attn_{loop}"].astype(np.float64)
        diff = np.abs(out - ref)
        assert np.mean(diff <= 2e-2 + 1e-2 * np.abs(ref)) > 0.97
        assert diff.max() < 0.12
