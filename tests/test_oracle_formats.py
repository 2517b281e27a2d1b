"""Number formats of the oracle against PyTorch's own casts (CPU)."""

import numpy as np
import torch

from oracle import rq_oracle as O


def _values(n=100000):
    rng = np.random.default_rng(0)
    x = rng.standard_normal(n).astype(np.float32) * (10.0 ** rng.uniform(-4, 3, n)).astype(np.float32)
    special = np.array([0.0, -0.0, 448, 449, 464, 465, 1e9, -1e9, 2**-9, 2**-10, 1.5 * 2**-10, 2.5 * 2**-9, 2**-6],
                       dtype=np.float32)
    return np.concatenate([x, special, -special])


def test_e4m3_encode_matches_torch():
    x = _values()
    ref = torch.from_numpy(x).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(O.e4m3_encode(x), ref)


def test_e4m3_decode_matches_torch():
    codes = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    mine = O.e4m3_decode(codes)
    finite = np.isfinite(ref)
    assert np.array_equal(mine[finite], ref[finite]) and np.all(np.isnan(mine[~finite]))


def test_bf16_rounding_matches_torch():
    x = _values()
    ref = torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.bf16_bits(x), ref)
    x64 = np.random.default_rng(2).standard_normal(50000) * 3
    ref64 = torch.from_numpy(x64).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.bf16_bits(O.bf16_round_from_f64(x64)), ref64)


def test_signed_hadamard_matches_dense_matrix():
    rng = np.random.default_rng(3)
    for dim in (128, 96):
        signs = (rng.integers(0, 2, (3, dim)) * 2 - 1).astype(np.int8)
        rot = O.SignedHadamard(signs, np.float32(np.float16(dim ** -0.5)))
        x = rng.standard_normal((5, 3, dim)).astype(np.float32)
        dense = rot.dense().astype(np.float64)
        ref = np.einsum("thd,hde->the", x.astype(np.float64), dense)
        fast = O.rotate_signed_hadamard(x, rot)
        assert np.abs(fast - ref).max() < 2e-5
        back = O.rotate_signed_hadamard(fast, rot, inverse=True)
        assert np.abs(back - x).max() < 5e-3          # fp16-rounded scale: R R^T = (1 +- 2^-11) I
        ref_back = np.einsum("the,hde->thd", fast.astype(np.float64), dense)
        assert np.abs(back - ref_back).max() < 2e-5
        # orthogonality of the +-1 matrix
        h = O.hadamard_unnormalized(dim)
        assert np.array_equal(h @ h.T, dim * np.eye(dim, dtype=np.float32))
