"""Moves a `helpers.Case` onto the GPU and calls the product through its reference-shaped API."""

from __future__ import annotations

import numpy as np
import torch

from residualquant_b200 import _cuda, rotation


def bf16(x: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).to(device).to(torch.bfloat16)


def device_rotations(case, device="cuda"):
    kr = rotation.signed_hadamard(case.key_signs, float(case.rscale), device) if case.key_signs is not None else None
    vr = rotation.signed_hadamard(case.value_signs, float(case.rscale), device) if case.value_signs is not None else None
    return kr, vr


def gpu_cache(case, coefficient="ls", fill=0, device="cuda") -> torch.Tensor:
    L = case.layout
    cache = torch.full((2, case.num_blocks, case.heads, L.page_tokens, L.page_width), fill, dtype=torch.uint8, device=device)
    kr, vr = device_rotations(case, device)
    pairs = [(bf16(k, device), bf16(v, device)) for k, v in zip(case.keys, case.values)]
    mean = torch.from_numpy(case.key_mean).to(device) if case.key_mean is not None else None
    _cuda.quantize(pairs, cache, torch.from_numpy(case.slots).to(device), kr, vr, mean,
                   [list(r) for r in L.records], L.reference_mode, L.anchor_index, coefficient)
    torch.cuda.synchronize()
    return cache


def gpu_attention(case, cache: torch.Tensor, loop_index: int, device="cuda", pad_rows=0) -> torch.Tensor:
    L = case.layout
    r = len(case.seq_lens)
    kr, vr = device_rotations(case, device)
    q = bf16(case.query, device)
    k = bf16(case.keys[loop_index][case.live_rows], device)
    v = bf16(case.values[loop_index][case.live_rows], device)
    if pad_rows:
        pad = torch.zeros((pad_rows,) + tuple(q.shape[1:]), dtype=q.dtype, device=device)
        q, k, v = torch.cat([q, pad]), torch.cat([k, pad]), torch.cat([v, pad])
    out = torch.full_like(q, 768.0)
    mean = torch.from_numpy(case.key_mean).to(device) if case.key_mean is not None else None
    _cuda.attention(
        q, k, v, cache, out,
        torch.arange(r + 1, dtype=torch.int32, device=device),
        torch.from_numpy(case.seq_lens).to(device),
        torch.from_numpy(case.block_table).to(device),
        kr, vr, mean, [list(rec) for rec in L.records], L.reference_mode, L.anchor_index, loop_index,
    )
    torch.cuda.synchronize()
    _cuda.attention_status(device)
    return out
