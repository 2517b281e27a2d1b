"""Host-side sharding logic with two CPU ranks over gloo (the multi-GPU path without GPUs)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from residualquant_b200 import sharding


def test_shard_counts_cover_everything():
    assert sharding.shard_counts(55, 8) == [7, 7, 7, 7, 7, 7, 7, 6]
    assert sharding.shard_counts(64, 8) == [8] * 8
    assert sharding.shard_counts(3, 4) == [1, 1, 1, 0]
    covered = []
    for rank in range(8):
        begin, end = sharding.shard_range(55, 8, rank)
        covered.extend(range(begin, end))
    assert covered == list(range(55))
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)
    assert sharding.gather_heads(torch.ones(2, 4, 8), 4).shape == (2, 4, 8)   # single process: identity
    assert sharding.max_over_ranks(3.5, "cpu") == 3.5


def test_gather_layout_is_aligned_and_disjoint():
    one, flags, total = sharding.gather_layout(rows=16, heads=55, head_dim=96, buffers=2)
    assert one % 256 == 0 and one >= 16 * 55 * 96 * 2
    assert flags == 2 * one and total == flags + 256
    one, flags, total = sharding.gather_layout(rows=1, heads=1, head_dim=96, buffers=1)
    assert (one, flags, total) == (256, 256, 512)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        begin, end = sharding.shard_range(heads, world, rank)
        full = torch.arange(3 * heads * 4, dtype=torch.float32).reshape(3, heads, 4)
        gathered = sharding.gather_heads(full[:, begin:end].contiguous(), heads)
        slowest = sharding.max_over_ranks(10.0 + rank, "cpu")
        results[rank] = (bool(torch.equal(gathered, full)), slowest)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [5, 16])
def test_head_gather_and_max_over_two_ranks(heads):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), heads, results), nprocs=world, join=True)
    assert dict(results) == {0: (True, 11.0), 1: (True, 11.0)}
