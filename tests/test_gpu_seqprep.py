"""GPU parity of the one-kernel sequence preprocessing (duplicate removal + statistics): bit-exact
against the reference's golden outputs and against the CPU oracle on random and edge cases."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import gpu_ready
from oracle import reference_ops as R
from taac_2026_b200 import ops

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _apply(values, timestamps, src):
    keep = src.clamp_min(0).long()
    gone = src < 0
    new_values = values.gather(2, keep[:, None, :].expand(-1, values.shape[1], -1)).masked_fill(gone[:, None, :], 0)
    return new_values, timestamps.gather(1, keep).masked_fill(gone, 0)


def _check(values, lengths, ts, req):
    new_len, src, stats = ops.sequence_prepare(values.cuda(), lengths.cuda(), ts.cuda(), req.cuda())
    got_v, got_t = _apply(values, ts, src.cpu())
    want_v, want_l, want_t = R.deduplicate_sequence_events(values.numpy(), lengths.numpy(), ts.numpy())
    assert np.array_equal(new_len.cpu().numpy(), want_l)
    assert np.array_equal(got_v.numpy(), want_v)
    assert np.array_equal(got_t.numpy(), want_t)
    assert np.array_equal(stats.cpu().numpy(), R.sequence_stats(values.numpy(), lengths.numpy(), ts.numpy(), req.numpy()))


def test_reference_golden(ops_golden):
    g = {k: torch.from_numpy(v.copy()) for k, v in ops_golden.items() if k.startswith(("seq_", "dedup_"))}
    new_len, src, stats = ops.sequence_prepare(g["seq_values"].cuda(), g["seq_lengths"].cuda(), g["seq_ts"].cuda(), g["seq_req"].cuda())
    got_v, got_t = _apply(g["seq_values"], g["seq_ts"], src.cpu())
    assert torch.equal(new_len.cpu(), g["dedup_lengths"])
    assert torch.equal(got_v, g["dedup_values"]) and torch.equal(got_t, g["dedup_ts"])
    assert torch.equal(stats.cpu(), g["seq_stats"])


@pytest.mark.parametrize("seed", range(8))
def test_random_rows_match_oracle(seed):
    gen = torch.Generator().manual_seed(seed)
    B, F, L = 37, 1 + seed % 3, [1, 2, 7, 64, 255, 256, 257, 300][seed]
    values = torch.randint(-1, 6, (B, F, L), generator=gen)
    lengths = torch.randint(-2, L + 4, (B,), generator=gen)
    ts = torch.randint(0, 3, (B, L), generator=gen) * torch.randint(1, 4 * 10**7, (B, L), generator=gen)
    req = torch.randint(10**7, 5 * 10**7, (B,), generator=gen)
    _check(values, lengths, ts, req)


def test_full_length_zipf_rows():
    """1024 positions of heavy-tailed ids (many duplicates) and an all-distinct row (hash table at its fullest)."""
    from taac_2026_b200.inputs import zipf_ids

    gen = torch.Generator().manual_seed(3)
    B, L = 24, 1024
    values = zipf_ids(B * L, 1_000_000, 1.1, gen).view(B, 1, L)
    values[0, 0] = torch.randperm(L, generator=gen) + 1  # every event distinct
    values[1, 0] = 7                                        # every event the same
    lengths = torch.randint(0, L + 1, (B,), generator=gen)
    lengths[0] = lengths[1] = L
    _check(values, lengths, torch.zeros(B, L, dtype=torch.long), torch.full((B,), 1000))
