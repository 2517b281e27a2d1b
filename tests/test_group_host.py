"""Host logic of the deferred KV group (CPU): staging order, copies and the page-width formula."""

import pytest
import torch

from residualquant_b200.group import DeferredKVGroup


def test_page_width_and_cache_shape():
    g = DeferredKVGroup([[2, 32]] * 3 + [[4, 32]], 16)
    assert g.anchor_index == 3 and g.page_width(128) == 200 and g.page_width(96) == 152
    assert DeferredKVGroup([[2, 16]] * 3 + [[4, 32]], 32).page_width(128) == 224
    assert g.cache_shape(10, 16, 128) == (2, 10, 16, 16, 200)


def test_stage_holds_copies_until_the_last_loop():
    g = DeferredKVGroup([[2, 32]] * 3 + [[4, 32]], 16)
    keys = [torch.full((2, 1, 4), float(i)) for i in range(4)]
    for i in range(3):
        assert g.stage(keys[i], keys[i] + 10) is None
        keys[i].fill_(-1.0)                       # the group must have cloned: later writes do not leak in
    out = g.stage(keys[3], keys[3] + 10)
    assert len(out) == 4 and g.pending == []
    for i in range(3):
        assert torch.all(out[i][0] == float(i)) and torch.all(out[i][1] == float(i) + 10)
    assert out[3][0] is keys[3]                   # the completing call borrows its input
    single = DeferredKVGroup([[4, 32]], 16, anchor_index=0)
    k = torch.zeros(1, 1, 4)
    assert single.stage(k, k)[0][0] is k


def test_invalid_configurations_raise():
    with pytest.raises(ValueError):
        DeferredKVGroup([], 16)
    with pytest.raises(ValueError):
        DeferredKVGroup([[2, 32], [2, 32]], 16, reference_mode="adjacent", anchor_index=1)
    with pytest.raises(ValueError):
        DeferredKVGroup([[2, 32]], 16, coefficient_method="median")
    with pytest.raises(ValueError):
        DeferredKVGroup([[2, 32]], 16, reference_mode="sideways")
