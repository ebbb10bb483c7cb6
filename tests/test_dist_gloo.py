"""Multi-process path on CPU (gloo, world size 2): batch sharding and the scores gather."""

from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from taac_2026_b200.dist import gather_scores, shard_bounds


def test_shard_bounds_cover_the_batch():
    for total in (0, 1, 7, 8, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= 1
    with pytest.raises(ValueError):
        shard_bounds(10, 2, 2)


def _worker(rank: int, world: int, port: int, total: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(total, dtype=torch.float32) * 0.5  # stands for the single-process result
        lo, hi = shard_bounds(total, rank, world)
        got = gather_scores(full[lo:hi], total)
        assert torch.equal(got, full), (rank, got, full)
        torch.save(got, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [16, 17])
def test_gather_scores_world_size_2(tmp_path, total):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, total, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "rank0.pt"), torch.load(tmp_path / "rank1.pt")
    assert torch.equal(a, b) and a.shape == (total,)


def test_gather_is_identity_without_a_process_group():
    x = torch.ones(5)
    assert gather_scores(x) is x
