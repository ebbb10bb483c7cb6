"""Compact 32-bit host format on the GPU: `tb200_expand_sequence` rebuilds the padded int64 record bit for bit, and
the serving loop gives the same scores from compact batches as from the reference's padded ones
(application/evaluation/workflow.py:246-262 copies the padded record)."""
from __future__ import annotations

import dataclasses

import pytest
import torch

from conftest import gpu_ready, load_onetrans_fixture
from taac_2026_b200 import ops
from taac_2026_b200.inputs import (EntityInput, ModelInput, OneTransSpec, SequenceInput, compact_model_input,
                                   synthetic_batch)
from taac_2026_b200.onetrans import OneTransInference, random_state_dict, score_stream

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


@pytest.mark.parametrize("rows,feats,max_len", [(1, 1, 2), (257, 3, 50), (2000, 2, 1024), (64, 1, 8192)])
@pytest.mark.parametrize("with_time", [False, True])
def test_expand_rebuilds_the_padded_record(rows, feats, max_len, with_time):
    g = torch.Generator().manual_seed(rows + max_len)
    lengths = torch.randint(0, max_len + 1, (rows,), generator=g)
    lengths[0] = max_len
    valid = torch.arange(max_len)[None, :] < lengths[:, None]
    values = torch.randint(0, 2**31 - 1, (rows, feats, max_len), generator=g) * valid[:, None, :]
    now = torch.randint(1_600_000_000, 1_700_000_000, (rows,), generator=g)
    ts = (now[:, None] - torch.randint(-100, 2 * 10**9, (rows, max_len), generator=g)) * valid
    ts[torch.rand(rows, max_len, generator=g) < 0.1] = 0
    cu, ids, gaps = ops.compact_sequence_host(values, lengths, ts if with_time else None, now if with_time else None)
    got_values, got_lengths, got_ts = ops.expand_sequence(cu.cuda(), ids.cuda(), None if gaps is None else gaps.cuda(),
                                                          now.cuda(), max_len)
    assert got_values.dtype == got_lengths.dtype == got_ts.dtype == torch.int64
    assert torch.equal(got_values.cpu(), values) and torch.equal(got_lengths.cpu(), lengths)
    assert torch.equal(got_ts.cpu(), ts if with_time else torch.zeros_like(ts))


def test_expand_of_strided_feature_rows_and_empty_batches():
    """ids as rows of a larger buffer (what the list-column packer returns) and a batch without a single event."""
    buf = torch.arange(1, 61, dtype=torch.int32).reshape(2, 30).cuda()
    cu = torch.tensor([0, 3, 3, 7], dtype=torch.int32).cuda()
    values, lengths, ts = ops.expand_sequence(cu, buf[:, :7], None, None, 4)
    assert lengths.tolist() == [3, 0, 4] and int(ts.abs().sum()) == 0
    assert values[0].tolist() == [[1, 2, 3, 0], [31, 32, 33, 0]] and values[2].tolist() == [[4, 5, 6, 7], [34, 35, 36, 37]]
    empty = torch.zeros(5, dtype=torch.int32).cuda()
    values, lengths, _ = ops.expand_sequence(empty, torch.zeros(1, 0, dtype=torch.int32).cuda(), None, None, 6)
    assert values.shape == (4, 1, 6) and int(values.abs().sum()) == 0 and lengths.tolist() == [0, 0, 0, 0]
    with pytest.raises(ValueError):
        ops.expand_sequence(cu, buf[:, :7], None, None, 5)          # odd max_len


def test_scores_from_compact_batches_are_bit_identical():
    spec = OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(24)], item_int_specs=[(1000, i, 1) for i in range(8)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=128, emb_dim=64,
        num_blocks=2, num_heads=4, hidden_mult=4, seq_top_k=96, user_ns_tokens=5, item_ns_tokens=2)
    model = OneTransInference(random_state_dict(spec, seed=0), spec, dtype=torch.bfloat16)
    host = [synthetic_batch(spec, 64, seq_len=96, min_len=0, seed=s).pin_memory() for s in (3, 4, 5)]
    compact = [compact_model_input(b, pin=True) for b in host]
    assert compact[0].nbytes() < host[0].nbytes()
    want = [model.scores(b.to("cuda"), micro_batch=32).clone() for b in host]
    got = [s.clone() for s in score_stream(model, compact, micro_batch=32)]
    torch.cuda.synchronize()
    assert len(got) == len(want) and all(torch.equal(a, b) for a, b in zip(got, want))


def test_time_features_survive_the_compact_format():
    """A fixture with time buckets, two domains and real timestamps: the expanded record equals the padded one and
    the logits are bit-identical."""
    sd, spec_dict, inputs, _, _ = load_onetrans_fixture("onetrans_b")
    spec = OneTransSpec(**{k: spec_dict[k] for k in OneTransSpec.__dataclass_fields__ if k in spec_dict})
    ent = lambda e: EntityInput(e.int_values, e.int_missing_mask, e.dense_values, e.dense_missing_mask)  # noqa: E731
    batch = ModelInput(ent(inputs.user), ent(inputs.item),
                       {k: SequenceInput(s.values, s.lengths, s.timestamps) for k, s in inputs.sequences.items()},
                       inputs.request_timestamp)
    # the fixture's padding may hold anything; the compact record stands for the valid prefix with zeros behind it
    clean = {}
    for name, s in batch.sequences.items():
        valid = torch.arange(s.values.shape[2])[None, :] < s.lengths[:, None]
        clean[name] = SequenceInput(s.values * valid[:, None, :], s.lengths, s.timestamps * valid)
    batch = dataclasses.replace(batch, sequences=clean)
    compact = compact_model_input(batch)
    assert any(seq.gaps is not None for seq in compact.sequences.values())
    expanded = compact.to("cuda").expand()
    for name, s in batch.sequences.items():
        assert torch.equal(expanded.sequences[name].values.cpu(), s.values)
        assert torch.equal(expanded.sequences[name].timestamps.cpu(), s.timestamps)
        assert torch.equal(expanded.sequences[name].lengths.cpu(), s.lengths)
    model = OneTransInference(sd, spec, dtype=torch.float32)
    want, _ = model.predict(batch.to("cuda"))
    got, _ = model.predict(expanded)
    assert torch.equal(got, want)


def test_prediction_loop_returns_the_reference_loops_dictionary():
    """`run_inference_prediction_loop` against plain `model.scores` per batch: same keys (str(user_id), row number
    where a batch has no ids), same probabilities bit for bit, same counters as
    `_run_inference_prediction_loop` (application/evaluation/workflow.py:246-293) reports."""
    from types import SimpleNamespace

    from taac_2026_b200.serving import run_inference_prediction_loop

    spec = OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(8)], item_int_specs=[(1000, i, 1) for i in range(4)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=128, emb_dim=64,
        num_blocks=2, num_heads=4, hidden_mult=4, seq_top_k=96, user_ns_tokens=5, item_ns_tokens=2)
    model = OneTransInference(random_state_dict(spec, seed=0), spec, dtype=torch.bfloat16)
    batches = []
    for i, rows in enumerate((64, 64, 40)):
        inputs = synthetic_batch(spec, rows, seq_len=96, min_len=0, seed=20 + i)
        ids = [f"u{i}_{r}" for r in range(rows)] if i != 1 else None
        batches.append(SimpleNamespace(inputs=inputs, user_id=ids))
    out = run_inference_prediction_loop(model, batches)
    assert out["batch_count"] == 3 and out["processed_rows"] == 168 and out["loop_elapsed_sec"] > 0
    want = {}
    for batch in batches:
        scores = model.scores(batch.inputs.to("cuda")).cpu().tolist()
        keys = batch.user_id or list(range(len(scores)))
        for key, value in zip(keys, scores):
            want[str(key)] = float(value)
    assert out["predictions"] == want
    padded = run_inference_prediction_loop(model, batches, compact=False)
    assert padded["predictions"] == want
