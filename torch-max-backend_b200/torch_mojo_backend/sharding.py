"""Batch sharding of the forward over the GPUs of one box.

The forward has no cross-sample dependency (GEMM rows, LayerNorm/softmax rows and per-(batch,
head) attention are all independent), so it shards by batch with the weights replicated and no
collective on the data path. The reference has no multi-device code (its
docs/multi_gpu_training_plan.md is a proposal); the process group is used only to line the ranks up
before timing and to gather a few scalars afterwards.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(global_batch: int, rank: int, world_size: int) -> tuple[int, int]:
    """[start, end) of the samples rank `rank` owns; the first `global_batch % world_size` ranks
    take one extra sample."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def aggregate_throughput(units: float, elapsed_ms: float, device: torch.device | str = "cpu", group=None) -> dict:
    """Whole-job figures from per-rank ones: units are summed over ranks, time is the maximum
    over ranks. Works without an initialised process group (single process)."""
    if not (dist.is_available() and dist.is_initialized()):
        return {"units": units, "ms": elapsed_ms, "per_rank_ms": [elapsed_ms]}
    world = dist.get_world_size(group)
    mine = torch.tensor([units, elapsed_ms], dtype=torch.float64, device=device)
    gathered = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    per_rank = [g.cpu() for g in gathered]
    return {
        "units": float(sum(g[0].item() for g in per_rank)),
        "ms": float(max(g[1].item() for g in per_rank)),
        "per_rank_ms": [float(g[1].item()) for g in per_rank],
    }
