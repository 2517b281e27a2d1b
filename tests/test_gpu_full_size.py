"""Size-independent properties at the full shapes of the BASELINE configurations (no CPU oracle at this size).

One sequence's K/V rows are quantized into every sequence's own (randomly permuted) pages, so all rows of the batch
see the same content through different block tables:

* paging invariance: with the same query the outputs of all rows are bit-identical, whatever pages hold the data;
* partition invariance: 1 partition and several partitions agree within the attention tolerance;
* softmax normalisation: when every cached V row and the live V row are the same vector, the output does not depend
  on the query (the probabilities sum to one whatever the scores are);
* idempotence of the write: quantizing the same rows into the same slots again leaves every cache byte unchanged.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-2, 1e-2


def _rows(tokens, heads, dim, seed, device="cuda"):
    g = torch.Generator(device=device).manual_seed(seed)
    scale = torch.exp(0.5 * torch.randn(heads, dim, generator=g, device=device))
    anchor = torch.randn(tokens, heads, dim, generator=g, device=device) * scale
    rows = [(0.9 * anchor + 0.3 * torch.randn(tokens, heads, dim, generator=g, device=device)).bfloat16() for _ in range(3)]
    return rows + [anchor.bfloat16()]


@pytest.mark.parametrize("batch,context,heads,dim,group", [
    (64, 8192, 16, 128, 32),    # kernel sweep corner / Ouro-1.4B-shaped layer
    (64, 8192, 16, 128, 16),    # Ouro-2.6B-shaped layer (INT2 g16 residuals)
    (16, 4096, 55, 96, 32),     # Huginn-shaped group
])
def test_full_size_properties(batch, context, heads, dim, group):
    from residualquant_b200 import _cuda, rotation, synth
    from residualquant_b200.cache_plan import page_width

    device = "cuda"
    page = 16
    records = [[2, group], [2, group], [2, group], [4, 32]]
    width = page_width(records, dim)
    pages_per_sequence = (context + page - 1) // page
    num_blocks = batch * pages_per_sequence + 1
    g = torch.Generator(device="cpu").manual_seed(7)
    order = torch.randperm(num_blocks - 1, generator=g) + 1            # block 0 stays unused (vLLM's null block)
    block_table = order.view(batch, pages_per_sequence).to(torch.int32).to(device)
    cache = torch.zeros(2, num_blocks, heads, page, width, dtype=torch.uint8, device=device)

    import numpy as np
    signs = synth.signs(np.random.default_rng(3), heads, dim)
    key_rot = rotation.signed_hadamard(signs, float(synth.fp16_rsqrt(dim)), device)

    history = context - 1
    keys = _rows(history, heads, dim, 11)
    values = _rows(history, heads, dim, 12)
    same_v = values[3][:1].expand(history, heads, dim).contiguous()     # every cached V row of loop 3 is one vector
    values[3] = same_v
    positions = torch.arange(history, device=device)
    pairs = list(zip(keys, values))
    for b in range(batch):
        slots = block_table[b, positions // page].long() * page + positions % page
        _cuda.quantize(pairs, cache, slots, key_rot, None, None, records, "anchor", 3, "ls")
    torch.cuda.synchronize()

    # idempotence of the write
    before = cache.clone()
    slots = block_table[batch - 1, positions // page].long() * page + positions % page
    _cuda.quantize(pairs, cache, slots, key_rot, None, None, records, "anchor", 3, "ls")
    torch.cuda.synchronize()
    assert torch.equal(cache, before)
    del before

    gq = torch.Generator(device=device).manual_seed(21)
    q_one = torch.randn(1, heads, dim, generator=gq, device=device).bfloat16()
    q = q_one.expand(batch, heads, dim).contiguous()
    qsl = torch.arange(batch + 1, dtype=torch.int32, device=device)
    seq_lens = torch.full((batch,), context, dtype=torch.int32, device=device)

    def run(loop, splits, v_live, query=None, k_live=None):
        query = q if query is None else query
        if k_live is None:
            k_live = keys[loop][-1:].expand(batch, heads, dim).contiguous()
        out = torch.zeros_like(query)
        _cuda.set_attention_splits(splits)
        try:
            _cuda.attention(query, k_live, v_live, cache, out, qsl, seq_lens, block_table, key_rot, None, None, records,
                            "anchor", 3, loop)
        finally:
            _cuda.set_attention_splits(0)
        torch.cuda.synchronize()
        _cuda.attention_status(device)
        return out

    for loop in (0, 3):
        v_live = values[loop][-1:].expand(batch, heads, dim).contiguous()
        one = run(loop, 1, v_live)
        assert torch.isfinite(one.float()).all()
        # paging invariance: same content behind different block tables
        assert torch.equal(one, one[:1].expand_as(one))
        # partition invariance
        several = run(loop, 4, v_live)
        assert torch.equal(several, several[:1].expand_as(several))
        diff = (one.float() - several.float()).abs()
        assert bool((diff <= ATOL + RTOL * one.float().abs()).all()), float(diff.max())

    # softmax normalisation: loop 3 (the anchor) holds one V vector everywhere, so the query must not matter
    v0 = same_v[:1].expand(batch, heads, dim).contiguous()
    other = (3.0 * torch.randn(batch, heads, dim, generator=gq, device=device)).bfloat16()   # sharper, row-dependent scores
    # (a zero live key keeps the live token, whose V is the unquantized vector, at a weight near 1/context)
    no_key = torch.zeros_like(q)
    first, second = run(3, 0, v0, None, no_key).float(), run(3, 0, v0, other, no_key).float()
    diff = (first - second).abs()
    assert bool((diff <= ATOL + RTOL * first.abs()).all()), float(diff.max())
    # and the common value is the stored vector up to its INT4 quantization error (a loose sanity bound)
    spread = v0.float().view(batch, heads, dim // 32, 32)
    width_of_group = (spread.amax(-1) - spread.amin(-1)).unsqueeze(-1).expand_as(spread).reshape(batch, heads, dim)
    assert bool(((first - v0.float()).abs() <= 0.15 * width_of_group + 0.05).all())
