"""The N > 1 path on CPU: two gloo ranks shard a global batch, and the whole-job throughput is
the sum of units over the maximum time."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from torch_mojo_backend.sharding import aggregate_throughput, shard_range


def test_shard_range_partitions_the_batch():
    for batch, world in ((64, 1), (64, 2), (64, 8), (10, 4), (3, 8)):
        spans = [shard_range(batch, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == batch
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [e - s for s, e in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def test_aggregate_without_process_group():
    out = aggregate_throughput(100.0, 5.0)
    assert out == {"units": 100.0, "ms": 5.0, "per_rank_ms": [5.0]}


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, end = shard_range(64, rank, world)
        ids = torch.arange(64 * 4).view(64, 4)[start:end]  # this rank's slice of the global batch
        tokens = float(ids.numel())
        elapsed = 10.0 * (rank + 1)  # rank 1 is the slow one
        dist.barrier()
        agg = aggregate_throughput(tokens, elapsed)
        results[rank] = (start, end, int(ids.sum()), agg)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_aggregate():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert results[0][:2] == (0, 32) and results[1][:2] == (32, 64)
    total = int(torch.arange(64 * 4).sum())
    assert results[0][2] + results[1][2] == total, "the shards cover the batch exactly once"
    for rank in (0, 1):
        agg = results[rank][3]
        assert agg["units"] == 256.0 and agg["ms"] == 20.0 and agg["per_rank_ms"] == [10.0, 20.0]
