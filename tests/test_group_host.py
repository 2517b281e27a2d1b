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


def test_batch_slices_split_decodes_from_full_prompts():
    from residualquant_b200.group import BatchSlice, batch_slices, causal_prefill

    assert batch_slices([0], []) == []
    assert batch_slices([0, 1, 2, 3], [9, 4, 700]) == [BatchSlice(0, 3, 0, 3, True)]
    # two decodes, then prompts of 5 and 3 tokens
    assert batch_slices([0, 1, 2, 7, 10], [40, 12, 5, 3]) == [BatchSlice(0, 2, 0, 2, True), BatchSlice(2, 4, 2, 10, False)]
    assert batch_slices([0, 6], [6]) == [BatchSlice(0, 1, 0, 6, False)]
    with pytest.raises(ValueError, match="partial prefill"):
        batch_slices([0, 1, 5], [8, 9])            # 4 query tokens of a 9-token sequence: a chunked prefill
    with pytest.raises(ValueError, match="precede"):
        batch_slices([0, 4, 5], [4, 30])           # a decode after a prompt: the batch was not reordered
    # the default prefill is causal per prompt and keeps prompts independent
    torch.manual_seed(0)
    q, k, v = (torch.randn(8, 2, 16) for _ in range(3))
    out = torch.zeros_like(q)
    causal_prefill(q, k, v, out, [0, 5, 8])
    scores = torch.einsum("thd,shd->hts", q[5:8], k[5:8]) / 4.0
    scores = scores.masked_fill(torch.triu(torch.ones(3, 3, dtype=torch.bool), 1), float("-inf"))
    want = torch.einsum("hts,shd->thd", scores.softmax(-1), v[5:8])
    assert torch.allclose(out[5:8], want, atol=1e-5)
    assert torch.allclose(out[0], v[0], atol=1e-6)  # a prompt's first token attends to itself only
