"""Shared scaffolding of the parity tests: seeded cases that the oracle and the CUDA path both consume."""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import numpy as np

from oracle import rq_oracle as O
from residualquant_b200 import synth


@dataclass
class Case:
    layout: O.PackedLayout
    heads: int
    seq_lens: np.ndarray            # [R] including the live token
    block_table: np.ndarray         # int32 [R, max_blocks]
    num_blocks: int
    keys: List[np.ndarray]          # per record: [T_total, H, D] rows of all requests back to back (history + live)
    values: List[np.ndarray]
    slots: np.ndarray               # int64 [T_total]; the live token of every request has slot -1 (never written)
    live_rows: np.ndarray           # index into keys/values of every request's live token
    query: np.ndarray               # [R, H, D]
    key_signs: Optional[np.ndarray]
    value_signs: Optional[np.ndarray]
    rscale: np.float32
    key_mean: Optional[np.ndarray]  # [n, H, D] rotated coordinates


def make_case(seed, head_dim, heads, seq_lens, residual_group=32, page_tokens=16, records=None, anchor_index=3,
              rotate_keys=True, rotate_values=True, with_mean=False, reference_mode="anchor") -> Case:
    rng = np.random.default_rng(seed)
    if records is None:
        records = ((2, residual_group),) * 3 + ((4, 32),)
    layout = O.PackedLayout(head_dim, tuple(tuple(r) for r in records), page_tokens, anchor_index, reference_mode)
    n = len(layout.records)
    seq_lens = np.asarray(seq_lens, dtype=np.int32)
    block_table, num_blocks = synth.paging(rng, seq_lens, page_tokens)
    total = int(seq_lens.sum())
    loops = synth.loop_rows(rng, total, heads, head_dim, loops=max(n, 2))
    vloops = synth.loop_rows(rng, total, heads, head_dim, loops=max(n, 2))
    # loop_rows puts its anchor last; move it to anchor_index
    order = list(range(len(loops) - 1))
    order.insert(anchor_index, len(loops) - 1)
    keys = [loops[i] for i in order][:n]
    values = [vloops[i] for i in order][:n]
    slots = np.full(total, -1, dtype=np.int64)
    live_rows = np.zeros(len(seq_lens), dtype=np.int64)
    cursor = 0
    for r, length in enumerate(seq_lens):
        hist = int(length) - 1
        if hist > 0:
            slots[cursor:cursor + hist] = synth.slots_for(block_table, r, np.arange(hist), page_tokens)
        live_rows[r] = cursor + max(hist, 0)
        cursor += int(length)
    query = synth.to_bf16_f32(rng.standard_normal((len(seq_lens), heads, head_dim)).astype(np.float32))
    key_signs = synth.signs(rng, heads, head_dim) if rotate_keys else None
    value_signs = synth.signs(rng, heads, head_dim) if rotate_values else None
    key_mean = (0.25 * rng.standard_normal((n, heads, head_dim))).astype(np.float32) if with_mean else None
    return Case(layout, heads, seq_lens, block_table, num_blocks, keys, values, slots, live_rows, query,
                key_signs, value_signs, synth.fp16_rsqrt(head_dim), key_mean)


def oracle_rotations(case: Case):
    kr = O.SignedHadamard(case.key_signs, case.rscale) if case.key_signs is not None else None
    vr = O.SignedHadamard(case.value_signs, case.rscale) if case.value_signs is not None else None
    return kr, vr


def oracle_cache(case: Case, coefficient="ls", chain="kernel", fill=0) -> np.ndarray:
    L = case.layout
    cache = np.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), fill, dtype=np.uint8)
    kr, vr = oracle_rotations(case)
    O.quantize(list(zip(case.keys, case.values)), cache, case.slots, L, kr, vr, case.key_mean, coefficient, chain)
    return cache


def oracle_attention(case: Case, cache: np.ndarray, loop_index: int) -> np.ndarray:
    kr, vr = oracle_rotations(case)
    r = len(case.seq_lens)
    return O.attention(
        case.query, case.keys[loop_index][case.live_rows], case.values[loop_index][case.live_rows], cache,
        np.arange(r + 1, dtype=np.int32), case.seq_lens, case.block_table, case.layout, loop_index, kr, vr,
        case.key_mean,
    )
