"""Pool sizing arithmetic (no GPU)."""

import pytest

from residualquant_b200 import cache_plan as cp
from residualquant_b200.group import DeferredKVGroup

G32 = ((2, 32), (2, 32), (2, 32), (4, 32))
G16 = ((2, 16), (2, 16), (2, 16), (4, 32))


def test_page_widths_match_the_layout_and_the_group_mirror():
    assert cp.page_width(G32, 128) == 200 and cp.page_width(G16, 128) == 224
    assert cp.page_width(G32, 96) == 152 and cp.page_width(G16, 96) == 170
    for records, dim in ((G32, 128), (G16, 96)):
        assert DeferredKVGroup(records, 16).page_width(dim) == cp.page_width(records, dim)
    with pytest.raises(ValueError):
        cp.page_width(((3, 32),), 128)
    with pytest.raises(ValueError):
        cp.page_width(((2, 32),), 100)


def test_ouro_shaped_pool_on_one_b200():
    owners = cp.looped_model_owners(layers=24, groups_per_layer=1, records=G32, heads=16, head_dim=128)
    plan = cp.plan_cache(owners, budget_bytes=150 * 10**9, max_model_len=8192 + 128)
    assert plan.bytes_per_block == 24 * 2 * 16 * 16 * 200
    assert plan.num_blocks == 150 * 10**9 // plan.bytes_per_block
    assert plan.total_bytes <= 150 * 10**9
    # 64 sequences of 8k context fit with room to spare; bf16 KV for the same 4 loops would need 2.47x the bytes
    assert plan.tokens >= 64 * (8192 + 128)
    spec = owners["layers.0.group.0"]
    assert spec.cache_shape(10) == (2, 10, 16, 16, 200)
    native = cp.OwnerSpec(16, 128, 16)
    assert 4 * native.page_bytes / spec.page_bytes == pytest.approx(4 * 256 / 200)


def test_mixed_owners_share_one_block_space():
    owners = {"packed": cp.OwnerSpec(55, 96, 16, G32), "native": cp.OwnerSpec(55, 96, 16)}
    plan = cp.plan_cache(owners, 10**9, 4096)
    assert plan.bytes_per_block == 2 * 55 * 16 * (152 + 192)
    assert plan.owner_bytes["native"] * 152 == plan.owner_bytes["packed"] * 192
    with pytest.raises(ValueError, match="null block"):
        cp.plan_cache(owners, plan.bytes_per_block * 256, 4096)
    with pytest.raises(ValueError, match="block sizes differ"):
        cp.plan_cache({"a": cp.OwnerSpec(8, 128, 16, G32), "b": cp.OwnerSpec(8, 128, 32, G32)}, 10**9, 128)


def test_kv_footprint_per_token():
    """The figures of the reference's capacity experiment for the Ouro-1.4B geometry (24 layers x 4 loops, 16 x 128)."""
    geometry = dict(layers=24, loops=4, heads=16, head_dim=128)
    assert cp.kv_footprint([], **geometry) == 786432                     # native bf16 KV
    packed = cp.kv_footprint([[[2, 32]] * 3 + [[4, 32]]], **geometry)
    assert packed == 2 * 24 * 16 * 200 == 153600 and 786432 / packed == pytest.approx(5.12)
    assert cp.kv_footprint([[[2, 16]] * 3 + [[4, 32]]], **geometry) == 2 * 24 * 16 * 224
    with pytest.raises(ValueError):
        cp.kv_footprint([[[2, 32]] * 3], **geometry)                    # a loop without a record
    with pytest.raises(ValueError):
        cp.kv_footprint([[[3, 32]] * 4], **geometry)
    # 100 GB of KV at context 8192: 79 sequences packed against 15 native
    assert cp.sequences_that_fit(100 * 10**9, 8192, packed) == 79
    assert cp.sequences_that_fit(100 * 10**9, 8192, 786432) == 15
