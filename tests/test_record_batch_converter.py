"""`CompactRecordBatchConverter` against the reference's own `PCVRRecordBatchConverter`
(src/taac2026/infrastructure/data/batch_converter.py:203-348) on seeded Arrow record batches: entity tensors equal,
and the compact sequences, unpacked, equal the reference's padded buffers over the valid prefix — with and without
the strict time filter.  Host code only; needs the reference (a checkout or the compiled archive)."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

pa = pytest.importorskip("pyarrow")

from oracle import ref_runtime  # noqa: E402
from taac_2026_b200.converter import CompactRecordBatchConverter  # noqa: E402

pytestmark = pytest.mark.skipif(not ref_runtime.available(), reason="no reference checkout and no oracle/_ref available")

NONE = -2**31


def _schema(tmp_path):
    path = tmp_path / "schema.json"
    path.write_text(json.dumps({
        "format": "raw_parquet",
        "user_int": [[1, 50, 1], [2, 20, 3], [5, 0, 1]],
        "item_int": [[3, 30, 1]],
        "user_dense": [[4, 3]],
        "seq": {"seq_a": {"prefix": "domain_a_seq", "ts_fid": 9, "features": [[9, 128], [10, 16], [11, 40]]}},
    }))
    return path


def _lists(rng, rows, max_count, low, high, dtype):
    counts = rng.integers(0, max_count + 1, rows)
    return pa.array([rng.integers(low, high, c).astype(dtype).tolist() for c in counts], type=pa.list_(pa.from_numpy_dtype(dtype)))


def _record_batch(rows: int, seed: int):
    rng = np.random.default_rng(seed)
    now = rng.integers(1_000_000, 2_000_000, rows)
    ts_counts = rng.integers(0, 14, rows)
    ts = [np.sort(rng.integers(-5, 2_100_000, c)).tolist() for c in ts_counts]      # some <= 0, some after the request
    scalar = [None if rng.random() < 0.2 else int(v) for v in rng.integers(-2, 70, rows)]
    dense = [[float("nan") if rng.random() < 0.1 else float(v) for v in rng.normal(size=c)] for c in rng.integers(0, 5, rows)]
    arrays = [
        pa.array(now, type=pa.int64()), pa.array(rng.integers(0, 3, rows), type=pa.int64()),
        pa.array([f"u{i}" for i in range(rows)]),
        pa.array(scalar, type=pa.int64()), _lists(rng, rows, 5, -1, 30, np.int64), pa.array(rng.integers(0, 9, rows), type=pa.int64()),
        pa.array(rng.integers(0, 40, rows), type=pa.int64()), pa.array(dense, type=pa.list_(pa.float32())),
        pa.array(ts, type=pa.list_(pa.int64())),
        pa.array([rng.integers(-1, 25, max(0, c + int(rng.integers(-2, 3)))).tolist() for c in ts_counts], type=pa.list_(pa.int64())),
        pa.array([rng.integers(0, 60, max(0, c + int(rng.integers(-2, 3)))).tolist() for c in ts_counts], type=pa.list_(pa.int64())),
    ]
    names = ["timestamp", "label_type", "user_id", "user_int_feats_1", "user_int_feats_2", "user_int_feats_5", "item_int_feats_3",
             "user_dense_feats_4", "domain_a_seq_9", "domain_a_seq_10", "domain_a_seq_11"]
    return pa.record_batch(arrays, names=names)


def _unpack(seq, request_ts):
    cu, ids = seq.cu.numpy(), seq.ids.numpy()
    rows, feats = cu.shape[0] - 1, ids.shape[0]
    values = np.zeros((rows, feats, seq.max_len), dtype=np.int64)
    ts = np.zeros((rows, seq.max_len), dtype=np.int64)
    for r in range(rows):
        lo, hi = int(cu[r]), int(cu[r + 1])
        values[r, :, :hi - lo] = ids[:, lo:hi]
        if seq.gaps is not None:
            g = seq.gaps.numpy()[lo:hi].astype(np.int64)
            ts[r, :hi - lo] = np.where(g == NONE, 0, request_ts[r] - g)
    return values, np.diff(cu.astype(np.int64)), ts


@pytest.mark.parametrize("strict", [False, True])
@pytest.mark.parametrize("seed", [0, 1])
def test_matches_the_reference_converter(tmp_path, strict, seed):
    ref_runtime.import_reference()
    from taac2026.infrastructure.data.batch_converter import PCVRRecordBatchConverter, build_pcvr_column_plan
    from taac2026.infrastructure.data.schema_layout import load_pcvr_schema_layout

    layout = load_pcvr_schema_layout(_schema(tmp_path), {"seq_a": 8})
    batch = _record_batch(257, seed)
    plan = build_pcvr_column_plan(layout, batch.schema.names)
    want = PCVRRecordBatchConverter(layout=layout, column_plan=plan, batch_size=512, clip_vocab=True, is_training=True,
                                    strict_time_filter=strict).convert(batch)
    ours = CompactRecordBatchConverter(layout=layout, column_plan=plan, clip_vocab=True, is_training=True,
                                       strict_time_filter=strict, threads=2)
    got = ours.convert(batch)
    assert got.user_id == want.user_id and torch.equal(got.label, want.label)
    assert torch.equal(got.inputs.request_timestamp, want.inputs.request_timestamp)
    for side in ("user", "item"):
        a, b = getattr(got.inputs, side), getattr(want.inputs, side)
        assert torch.equal(a.int_values, b.int_values) and torch.equal(a.int_missing_mask, b.int_missing_mask)
        assert torch.equal(a.dense_values, b.dense_values) and torch.equal(a.dense_missing_mask, b.dense_missing_mask)
    seq_want = want.inputs.sequences["seq_a"]
    values, lengths, ts = _unpack(got.inputs.sequences["seq_a"], want.inputs.request_timestamp.numpy())
    assert np.array_equal(lengths, seq_want.lengths.numpy())
    assert np.array_equal(values, seq_want.values.numpy())
    # the compact record holds the valid prefix; the reference's non-strict fill may carry timestamps behind it
    inside = np.arange(8)[None, :] < lengths[:, None]
    assert np.array_equal(ts, seq_want.timestamps.numpy() * inside)
    assert sum(v["count"] for v in ours.oob_stats.values()) > 0       # the seeded ids do leave the vocabularies


def test_out_of_vocabulary_without_clipping_raises(tmp_path):
    ref_runtime.import_reference()
    from taac2026.infrastructure.data.batch_converter import build_pcvr_column_plan
    from taac2026.infrastructure.data.schema_layout import load_pcvr_schema_layout

    layout = load_pcvr_schema_layout(_schema(tmp_path), {"seq_a": 8})
    batch = _record_batch(64, 3)
    plan = build_pcvr_column_plan(layout, batch.schema.names)
    with pytest.raises(ValueError, match="out of range"):
        CompactRecordBatchConverter(layout=layout, column_plan=plan, clip_vocab=False).convert(batch)
