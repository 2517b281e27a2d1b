"""Seeded synthetic K/V, rotations and paging metadata with the value distributions of the
benchmark configurations (numpy, CPU; small and medium sizes).

Distributions: the last-loop anchor is N(0,1) times a per-channel log-normal(0, 0.5) scale with four
outlier channels per head scaled by 8; every earlier loop is 0.9*anchor + 0.3*N(0,1); everything is
rounded to bfloat16.  The rotation is diag(+-1) times the normalized Hadamard matrix of the head
dimension.  Block tables are a random permutation of a page pool.
"""

from __future__ import annotations

import numpy as np


def to_bf16_f32(x: np.ndarray) -> np.ndarray:
    """Round binary32 to the nearest bfloat16 (ties to even); returned as binary32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32)


def loop_rows(rng: np.random.Generator, tokens: int, heads: int, dim: int, loops: int = 4):
    """One plane (K or V) for `loops` loops, anchor last: list of [tokens, heads, dim] bf16-valued float32."""
    channel_scale = np.exp(0.5 * rng.standard_normal((heads, dim))).astype(np.float32)
    anchor = rng.standard_normal((tokens, heads, dim)).astype(np.float32) * channel_scale
    for h in range(heads):
        anchor[:, h, rng.permutation(dim)[:4]] *= 8.0
    rows = [
        to_bf16_f32(0.9 * anchor + 0.3 * rng.standard_normal((tokens, heads, dim)).astype(np.float32))
        for _ in range(loops - 1)
    ]
    rows.append(to_bf16_f32(anchor))
    return rows


def signs(rng: np.random.Generator, heads: int, dim: int) -> np.ndarray:
    return (rng.integers(0, 2, size=(heads, dim)) * 2 - 1).astype(np.int8)


def fp16_rsqrt(dim: int) -> np.float32:
    """Magnitude of the entries of an fp16 copy of H_D / sqrt(D)."""
    return np.float32(np.float16(1.0 / np.sqrt(float(dim))))


def paging(rng: np.random.Generator, seq_lens, page_tokens: int, spare_blocks: int = 3):
    """Random block tables over a shared pool.  Returns (block_table int32 [R, max_blocks], num_blocks)."""
    seq_lens = [int(s) for s in seq_lens]
    need = [(s + page_tokens - 1) // page_tokens for s in seq_lens]
    max_blocks = max(need + [1])
    total = sum(need) + spare_blocks
    pool = rng.permutation(total)
    table = np.zeros((len(seq_lens), max_blocks), dtype=np.int32)
    cursor = 0
    for r, n in enumerate(need):
        table[r, :n] = pool[cursor:cursor + n]
        cursor += n
    return table, total


def slots_for(block_table: np.ndarray, request: int, positions: np.ndarray, page_tokens: int) -> np.ndarray:
    positions = np.asarray(positions, dtype=np.int64)
    return block_table[request, positions // page_tokens].astype(np.int64) * page_tokens + positions % page_tokens
