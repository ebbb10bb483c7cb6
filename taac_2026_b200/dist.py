"""Multi-GPU plumbing of the inference path: batch sharding and the one exchange step.

Samples are independent and weights / tables are read-only, so the job shards by batch: one process
per GPU, a full replica of the model on each, rank ``r`` scores rows ``[r * B / W, (r + 1) * B / W)``.
The only communication is an ``all_gather`` of the per-rank score vectors (NCCL over NVLink on GPUs,
gloo in the CPU tests).  The reference itself is single-process
(`evaluation/workflow.py:246-293` loops over batches on one device); this is the data-parallel form of
that loop.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced row range of `rank` (earlier ranks take the remainder)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_scores(local_scores: torch.Tensor, total: int | None = None, group=None) -> torch.Tensor:
    """All ranks' score vectors in rank order -> ``float32[total]`` on every rank.

    Equal shard sizes use one ``all_gather_into_tensor``; ragged shards (total not divisible by the
    world size) are padded to the largest shard and trimmed afterwards."""
    if not dist.is_available() or not dist.is_initialized():
        return local_scores
    world = dist.get_world_size(group)
    scores = local_scores.contiguous().float()
    if total is None or total % world == 0:
        out = torch.empty(world * scores.shape[0], dtype=torch.float32, device=scores.device)
        dist.all_gather_into_tensor(out, scores, group=group)
        return out
    sizes = [shard_bounds(total, r, world) for r in range(world)]
    longest = max(hi - lo for lo, hi in sizes)
    padded = torch.zeros(longest, dtype=torch.float32, device=scores.device)
    padded[: scores.shape[0]] = scores
    out = torch.empty(world * longest, dtype=torch.float32, device=scores.device)
    dist.all_gather_into_tensor(out, padded, group=group)
    return torch.cat([out[r * longest : r * longest + (hi - lo)] for r, (lo, hi) in enumerate(sizes)])


__all__ = ["gather_scores", "shard_bounds"]
