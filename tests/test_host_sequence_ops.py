"""The integer preprocessing of the inference engine (duplicate removal, statistics, gap buckets,
id hashing, pyramid schedule) is plain tensor code that also runs on CPU tensors: checked bit-exactly
against the reference's golden outputs and against the oracle on random cases."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import onetrans as oracle_model
from oracle import reference_ops as R
from taac_2026_b200 import onetrans as M

EDGES = torch.tensor(M._BUCKET_EDGES, dtype=torch.long)


def test_bucket_edges_match_oracle_table():
    assert np.array_equal(EDGES.numpy(), R.BUCKET_BOUNDARIES)


def test_golden_integer_ops(ops_golden):
    g = {k: torch.from_numpy(v.copy()) for k, v in ops_golden.items() if k.startswith(("seq_", "dedup_", "hash_", "bucket_"))}
    v, l, t = M.deduplicate_sequence_events(g["seq_values"], g["seq_lengths"], g["seq_ts"])
    assert torch.equal(v, g["dedup_values"]) and torch.equal(l, g["dedup_lengths"]) and torch.equal(t, g["dedup_ts"])
    assert torch.equal(M.sequence_time_buckets(g["seq_ts"], g["seq_req"], EDGES), g["seq_buckets"])
    edge = M.sequence_time_buckets(10**11 - g["bucket_edge_gaps"], torch.tensor([10**11]), EDGES)
    assert torch.equal(edge, g["bucket_edge_out"])
    stats = M.sequence_stats(g["seq_values"], g["seq_lengths"], g["seq_ts"], g["seq_req"], EDGES)
    assert torch.equal(stats, g["seq_stats"])
    assert torch.equal(M.hash_compress_ids(g["hash_in"], 7), g["hash_out_7"])
    assert torch.equal(M.hash_compress_ids(g["hash_in"], 0), g["hash_out_0"])


@pytest.mark.parametrize("seed", range(12))
def test_random_sequences_match_oracle(seed):
    gen = torch.Generator().manual_seed(seed)
    B, F, L = 7, 1 + seed % 3, 5 + 3 * seed
    values = torch.randint(0, 5, (B, F, L), generator=gen)
    lengths = torch.randint(-1, L + 3, (B,), generator=gen)
    ts = torch.randint(0, 3, (B, L), generator=gen) * torch.randint(1, 10**7, (B, L), generator=gen)
    req = torch.randint(10**7, 2 * 10**7, (B,), generator=gen)
    v, l, t = M.deduplicate_sequence_events(values, lengths, ts)
    rv, rl, rt = R.deduplicate_sequence_events(values.numpy(), lengths.numpy(), ts.numpy())
    assert np.array_equal(v.numpy(), rv) and np.array_equal(l.numpy(), rl) and np.array_equal(t.numpy(), rt)
    stats = M.sequence_stats(values, lengths, ts, req, EDGES)
    assert np.array_equal(stats.numpy(), R.sequence_stats(values.numpy(), lengths.numpy(), ts.numpy(), req.numpy()))


def test_empty_and_degenerate_sequences():
    values = torch.zeros(3, 2, 0, dtype=torch.long)
    lengths = torch.zeros(3, dtype=torch.long)
    ts = torch.zeros(3, 0, dtype=torch.long)
    v, l, t = M.deduplicate_sequence_events(values, lengths, ts)
    assert v.shape == values.shape and torch.equal(l, lengths) and t.shape == ts.shape
    assert M.sequence_time_buckets(ts, torch.zeros(3, dtype=torch.long), EDGES).shape == (3, 0)


def test_pyramid_schedule_matches_oracle():
    for seq, layers, ns in ((1024, 8, 9), (256, 2, 9), (40, 2, 9), (5, 3, 9), (14 + 1 + 6, 3, 8)):
        s = seq
        for layer in range(layers):
            assert M.pyramid_keep_count(s, layer, layers, ns) == oracle_model.pyramid_keep_count(s, layer, layers, ns)
            s = M.pyramid_keep_count(s, layer, layers, ns)
    # the schedule quoted for the full-scale configuration: 1024 sequence tokens, 9 NS tokens, 8 layers
    s, seen = 1024, []
    for layer in range(8):
        s = M.pyramid_keep_count(s, layer, 8, 9)
        seen.append(s)
    assert seen == [567, 314, 174, 97, 54, 30, 17, 9]
