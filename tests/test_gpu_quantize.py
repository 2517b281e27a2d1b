"""KV-write quantizer on the GPU against the CPU oracle: the whole packed cache must be bit-identical."""

import numpy as np
import pytest
import torch

from residualquant_b200 import synth
from tests import gpu_helpers as G
from tests import helpers

pytestmark = pytest.mark.gpu


def _compare(case, coefficient="ls", chain="kernel"):
    from residualquant_b200 import _cuda

    _cuda.set_quantizer_chain(chain)
    try:
        got = G.gpu_cache(case, coefficient, fill=0xA5).cpu().numpy()
    finally:
        _cuda.set_quantizer_chain("kernel")
    want = helpers.oracle_cache(case, coefficient, chain, fill=0xA5)
    if not np.array_equal(got, want):
        bad = np.argwhere(got != want)
        raise AssertionError(f"{len(bad)} of {got.size} bytes differ; first at {bad[0]} (got {got[tuple(bad[0])]}, want {want[tuple(bad[0])]})")


@pytest.mark.parametrize("head_dim,group,page", [(128, 32, 16), (128, 16, 16), (128, 32, 32), (128, 16, 32),
                                                 (96, 32, 16), (96, 16, 32)])
def test_packed_bytes_bit_exact(head_dim, group, page):
    _compare(helpers.make_case(11, head_dim, 3, [70, 1, 33, 16], group, page))


@pytest.mark.parametrize("head_dim,group,mean", [(128, 32, False), (128, 16, True), (96, 32, True), (96, 16, False)])
def test_prefill_sized_write_bit_exact(head_dim, group, mean):
    """More than 256 tokens in one call: the kernel that walks the records of a row one after another (smaller calls
    of the headline schedule take the one-warp-per-token kernel, which the other cases of this file cover)."""
    _compare(helpers.make_case(15, head_dim, 2, [300, 41, 130], group, 16, with_mean=mean))


@pytest.mark.parametrize("head_dim", [128, 96])
def test_with_key_mean(head_dim):
    _compare(helpers.make_case(12, head_dim, 2, [45, 20], 32, 16, with_mean=True))


def test_without_rotation():
    _compare(helpers.make_case(13, 128, 2, [40], 16, 16, rotate_keys=False, rotate_values=False))
    _compare(helpers.make_case(14, 128, 2, [40], 32, 16, rotate_keys=True, rotate_values=False))


@pytest.mark.parametrize("coefficient", ["unit", "norm", "ls"])
def test_coefficient_methods(coefficient):
    _compare(helpers.make_case(15, 128, 2, [50, 9], 32, 16), coefficient)


@pytest.mark.parametrize("head_dim", [128, 96])
def test_calibration_chain(head_dim):
    _compare(helpers.make_case(16, head_dim, 2, [60, 30], 32, 16, with_mean=(head_dim == 128)), chain="calibration")


@pytest.mark.parametrize("records,anchor,mode", [
    (((4, 32), (2, 32), (2, 32), (2, 32)), 0, "anchor"),
    (((4, 32), (2, 32), (2, 32), (2, 32)), 0, "adjacent"),
    (((2, 16), (2, 16), (2, 16), (2, 16)), 0, "adjacent"),
    (((4, 32), (4, 32), (4, 32), (4, 32)), 3, "anchor"),
    (((4, 32),), 0, "anchor"),
    (((2, 32),), 0, "adjacent"),
])
def test_other_schedules(records, anchor, mode):
    _compare(helpers.make_case(17, 128, 2, [44, 21], records=records, anchor_index=anchor, reference_mode=mode,
                               with_mean=(mode == "adjacent")))


def test_extreme_values_and_zero_rows():
    case = helpers.make_case(18, 128, 2, [40], 32, 16)
    for rows in (case.keys, case.values):
        rows[3][3] = 0.0                     # an all-zero anchor row: scale 0, code 0, alpha 0/eps
        rows[0][5] = 0.0
        rows[3][7] = synth.to_bf16_f32(rows[3][7] * 300.0)   # saturates the FP8 scale/offset
        rows[1][9] = rows[3][9]              # residual equal to its anchor
        rows[2][11, :, ::2] = -0.0
    _compare(case)


def test_unaligned_rows_take_the_scalar_load_path():
    from residualquant_b200 import _cuda

    case = helpers.make_case(19, 128, 2, [30], 32, 16)
    L = case.layout
    cache = torch.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), 0xA5, dtype=torch.uint8, device="cuda")
    kr, vr = G.device_rotations(case)
    pairs = []
    for k, v in zip(case.keys, case.values):
        rows = k.shape[0]
        # a [T, H*D + 4] buffer viewed as [T, H, D]: row stride 260 elements (not a multiple of 8)
        def skew(x):
            buf = torch.zeros(rows, case.heads * 128 + 4, dtype=torch.bfloat16, device="cuda")
            buf[:, : case.heads * 128] = G.bf16(x).reshape(rows, -1)
            return buf[:, : case.heads * 128].unflatten(1, (case.heads, 128))
        pairs.append((skew(k), skew(v)))
    _cuda.quantize(pairs, cache, torch.from_numpy(case.slots).cuda(), kr, vr, None,
                   [list(r) for r in L.records], "anchor", 3, "ls")
    torch.cuda.synchronize()
    assert np.array_equal(cache.cpu().numpy(), helpers.oracle_cache(case, fill=0xA5))


def test_more_rows_than_slots_and_empty_call():
    from residualquant_b200 import _cuda

    case = helpers.make_case(20, 128, 2, [25], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    slots = torch.from_numpy(case.slots[:10]).cuda()
    cache = torch.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), 0xA5, dtype=torch.uint8, device="cuda")
    _cuda.quantize(pairs, cache, slots, kr, vr, None, [list(r) for r in L.records], "anchor", 3, "ls")
    want = np.full(cache.shape, 0xA5, dtype=np.uint8)
    from oracle import rq_oracle as O
    okr, ovr = helpers.oracle_rotations(case)
    O.quantize(list(zip(case.keys, case.values)), want, case.slots[:10], L, okr, ovr, None)
    assert np.array_equal(cache.cpu().numpy(), want)
    before = cache.clone()
    _cuda.quantize(pairs, cache, slots[:0], kr, vr, None, [list(r) for r in L.records], "anchor", 3, "ls")
    assert torch.equal(before, cache)


def test_argument_errors_raise_runtime_error():
    from residualquant_b200 import _cuda

    case = helpers.make_case(21, 128, 2, [20], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    slots = torch.from_numpy(case.slots).cuda()
    cache = torch.zeros((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), dtype=torch.uint8, device="cuda")
    records = [list(r) for r in L.records]
    with pytest.raises(RuntimeError, match="one K/V input per record"):
        _cuda.quantize(pairs[:3], cache, slots, kr, vr, None, records, "anchor", 3, "ls")
    with pytest.raises(RuntimeError, match="cache width"):
        _cuda.quantize(pairs, cache[..., :-2].contiguous(), slots, kr, vr, None, records, "anchor", 3, "ls")
    with pytest.raises(RuntimeError, match="INT64 slot mapping"):
        _cuda.quantize(pairs, cache, slots.int(), kr, vr, None, records, "anchor", 3, "ls")
    with pytest.raises(RuntimeError, match="Unsupported coefficient"):
        _cuda.quantize(pairs, cache, slots, kr, vr, None, records, "anchor", 3, "median")
    with pytest.raises(RuntimeError, match="reference mode"):
        _cuda.quantize(pairs, cache, slots, kr, vr, None, records, "sideways", 3, "ls")
    with pytest.raises(RuntimeError, match="BF16"):
        _cuda.quantize([(k.float(), v) for k, v in pairs], cache, slots, kr, vr, None, records, "anchor", 3, "ls")
    with pytest.raises(RuntimeError, match="FP16"):
        _cuda.quantize(pairs, cache, slots, torch.eye(128, device="cuda").expand(2, 128, 128).contiguous(), None, None,
                       records, "anchor", 3, "ls")


def test_dense_rotation_tensor_is_recognised_after_registration():
    """The reference API hands over a dense fp16 [heads, D, D] matrix (common/api.h:42-55)."""
    from residualquant_b200 import _cuda, rotation

    case = helpers.make_case(22, 128, 2, [30], 32, 16)
    L = case.layout
    kr, vr = G.device_rotations(case)
    dense_k, dense_v = kr.dense(), vr.dense()
    assert rotation.register_rotation(dense_k) is not None and rotation.register_rotation(dense_v) is not None
    assert rotation.register_rotation(torch.randn(2, 128, 128, device="cuda").half()) is None
    cache = torch.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), 0xA5, dtype=torch.uint8, device="cuda")
    pairs = [(G.bf16(k), G.bf16(v)) for k, v in zip(case.keys, case.values)]
    _cuda.quantize(pairs, cache, torch.from_numpy(case.slots).cuda(), dense_k, dense_v, None,
                   [list(r) for r in L.records], "anchor", 3, "ls")
    torch.cuda.synchronize()
    assert np.array_equal(cache.cpu().numpy(), helpers.oracle_cache(case, fill=0xA5))
    rotation.forget(dense_k)
    rotation.forget(dense_v)
