"""The compact 32-bit host format of the behaviour sequences: the library's host packers against a numpy restatement
of the reference converter's rules (`pad_list_offsets_values`, `_fill_sequence`, `_clip_sequence_vocab`,
src/taac2026/infrastructure/data/batch_converter.py:68-103, :503-538, :594-650).  Host code only: no GPU needed."""
import numpy as np
import pytest
import torch

from taac_2026_b200 import ops
from taac_2026_b200.inputs import OneTransSpec, compact_model_input, synthetic_batch

NONE = -2**31


def _pad(offsets, values, rows, width):
    """numpy restatement of pad_list_offsets_values (first `width` values of every row, zero fill)."""
    out = np.zeros((rows, width), dtype=np.int64)
    lengths = np.zeros(rows, dtype=np.int64)
    for r in range(rows):
        n = min(max(int(offsets[r + 1]) - int(offsets[r]), 0), width)
        out[r, :n] = values[int(offsets[r]):int(offsets[r]) + n]
        lengths[r] = n
    return out, lengths


def _unpack(cu, ids, gaps, request_ts, max_len):
    """The padded record a compact one stands for (what the device kernel rebuilds)."""
    rows, feats = cu.shape[0] - 1, ids.shape[0]
    values = np.zeros((rows, feats, max_len), dtype=np.int64)
    ts = np.zeros((rows, max_len), dtype=np.int64)
    for r in range(rows):
        lo, hi = int(cu[r]), int(cu[r + 1])
        values[r, :, :hi - lo] = ids[:, lo:hi]
        if gaps is not None:
            g = gaps[lo:hi].astype(np.int64)
            ts[r, :hi - lo] = np.where(g == NONE, 0, request_ts[r] - g)
    return values, np.diff(cu.astype(np.int64)), ts


@pytest.mark.parametrize("threads", [1, 3])
def test_padded_record_round_trip(threads):
    g = torch.Generator().manual_seed(5)
    rows, feats, max_len = 700, 3, 48
    lengths = torch.randint(0, max_len + 1, (rows,), generator=g)
    lengths[:3] = torch.tensor([0, max_len, 1])
    valid = torch.arange(max_len)[None, :] < lengths[:, None]
    values = torch.randint(0, 2**31 - 1, (rows, feats, max_len), generator=g) * valid[:, None, :]
    now = torch.randint(1_600_000_000, 1_700_000_000, (rows,), generator=g)
    ts = (now[:, None] - torch.randint(-5, 10**9, (rows, max_len), generator=g)) * valid
    ts[torch.rand(rows, max_len, generator=g) < 0.2] = 0            # missing timestamps inside the prefix
    cu, ids, gaps = ops.compact_sequence_host(values, lengths, ts, now, threads=threads)
    assert cu.dtype == ids.dtype == gaps.dtype == torch.int32 and int(cu[-1]) == int(lengths.sum())
    got_values, got_len, got_ts = _unpack(cu.numpy(), ids.numpy(), gaps.numpy(), now.numpy(), max_len)
    assert np.array_equal(got_values, values.numpy()) and np.array_equal(got_len, lengths.numpy())
    assert np.array_equal(got_ts, (ts * valid).numpy())


def test_values_beyond_32_bits_are_refused_not_truncated():
    values = torch.zeros(300, 1, 8, dtype=torch.int64)
    lengths = torch.full((300,), 8)
    values[299, 0, 7] = 2**31
    with pytest.raises(OverflowError):
        ops.compact_sequence_host(values, lengths, None, None)
    values[299, 0, 7] = 2**31 - 1
    ts = torch.ones(300, 8, dtype=torch.int64)
    now = torch.full((300,), 2**33)                               # gap needs 34 bits
    with pytest.raises(OverflowError):
        ops.compact_sequence_host(values, lengths, ts, now)
    values[0, 0, 0] = 5
    lengths[0] = 0                                                 # beyond the length: never looked at
    cu, ids, gaps = ops.compact_sequence_host(values, lengths, None, None)
    assert gaps is None and int(cu[1]) == 0


@pytest.mark.parametrize("wide_offsets", [False, True])
def test_list_columns_follow_the_converter_rules(wide_offsets):
    rng = np.random.default_rng(9)
    rows, feats, max_len = 400, 3, 20
    off_dtype = np.int64 if wide_offsets else np.int32
    vocab = [50, 0, 1000]                                          # column 1 has no vocabulary: all zeros
    columns, padded, col_lengths = [], [], []
    for f in range(feats):
        counts = rng.integers(0, 2 * max_len, rows)
        counts[:4] = [0, max_len, max_len + 7, 1]
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(off_dtype)
        values = rng.integers(-3, 80, int(offsets[-1])).astype(np.int64)
        columns.append((offsets, values))
        p, n = _pad(offsets, values, rows, max_len)
        padded.append(p)
        col_lengths.append(n)
    t_counts = rng.integers(0, 2 * max_len, rows)
    t_off = np.concatenate([[0], np.cumsum(t_counts)]).astype(off_dtype)
    now = rng.integers(1_600_000_000, 1_700_000_000, rows).astype(np.int64)
    t_val = (now.repeat(t_counts) - rng.integers(0, 10**8, int(t_off[-1]))).astype(np.int64)
    t_val[rng.random(t_val.shape[0]) < 0.1] = 0
    # the reference's rules on the padded buffers
    want = np.stack(padded, axis=1)
    want[want <= 0] = 0
    lengths = np.max(np.stack(col_lengths), axis=0)
    oob_want = []
    for f in range(feats):
        if vocab[f] > 0:
            oob = want[:, f, :] >= vocab[f]
            oob_want.append(int(oob.sum()))
            want[:, f, :][oob] = 0
        else:
            oob_want.append(0)
            want[:, f, :] = 0
    ts_want, _ = _pad(t_off, t_val, rows, max_len)
    ts_want *= np.arange(max_len)[None, :] < lengths[:, None]      # the compact record holds the valid prefix only

    cu, ids, gaps, oob = ops.compact_sequence_from_lists(columns, (t_off, t_val), now, max_len, vocab_sizes=vocab, threads=2)
    got_values, got_len, got_ts = _unpack(cu.numpy(), ids.numpy(), gaps.numpy(), now, max_len)
    assert np.array_equal(got_len, lengths)
    assert np.array_equal(got_values, want)
    assert np.array_equal(got_ts, ts_want)
    assert oob.tolist() == oob_want


def test_model_input_shrinks_and_keeps_everything_else():
    spec = OneTransSpec(user_int_specs=[(100, i, 1) for i in range(4)], item_int_specs=[(100, 0, 1)], user_dense_dim=4,
                        item_dense_dim=0, seq_vocab_sizes={"seq_a": [500, 30]}, d_model=64, emb_dim=32, num_blocks=1,
                        num_heads=2, seq_top_k=64)
    batch = synthetic_batch(spec, 300, seq_len=64, min_len=4, seed=1)
    compact = compact_model_input(batch, threads=2)
    assert compact.batch_size == 300 and compact.nbytes() < 0.45 * batch.nbytes()
    seq = compact.sequences["seq_a"]
    assert seq.max_len == 64 and seq.ids.shape[0] == 2 and seq.gaps is None     # synthetic timestamps are all zero
    assert compact.user is batch.user and compact.request_timestamp is batch.request_timestamp
    values, lengths, _ = _unpack(seq.cu.numpy(), seq.ids.numpy(), None, None, 64)
    assert np.array_equal(values, batch.sequences["seq_a"].values.numpy())
    assert np.array_equal(lengths, batch.sequences["seq_a"].lengths.numpy())
