"""Pins the CPU oracle (``oracle/``) to outputs of the reference project's own code.

The fixtures were produced by ``tests/golden/make_golden.py`` from the unmodified reference;
these tests need no GPU and no reference checkout.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_onetrans_fixture
from oracle import onetrans as oracle_model
from oracle import reference_ops as R

NORM_CASES = [("f32_96", False), ("f32_128", False), ("f32_127", False), ("bf16_128", True), ("bf16_400", True)]


@pytest.mark.parametrize("tag,bf16", NORM_CASES)
def test_rms_norm_matches_reference(ops_golden, tag, bf16):
    load = bf16_from_bits if bf16 else (lambda a: torch.from_numpy(a.copy()))
    x, w = load(ops_golden[f"norm_{tag}_x"]), load(ops_golden[f"norm_{tag}_w"])
    ref = load(ops_golden[f"norm_{tag}_rms"])
    # the literal restatement of the torch path reproduces the reference bit for bit
    assert torch.equal(R.rms_norm_input_dtype(x, w, 1e-6), ref)
    # the fp32 form (what accelerated kernels compute) stays within the reference's own tolerance
    tol = 2e-2 if bf16 else 1e-5
    torch.testing.assert_close(R.rms_norm_fp32(x, w, 1e-6).float(), ref.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("tag,bf16", NORM_CASES)
def test_layer_norm_matches_reference(ops_golden, tag, bf16):
    load = bf16_from_bits if bf16 else (lambda a: torch.from_numpy(a.copy()))
    x, w, b = (load(ops_golden[f"norm_{tag}_{k}"]) for k in ("x", "w", "b"))
    ref = load(ops_golden[f"norm_{tag}_ln"])
    tol = 2e-2 if bf16 else 2e-5
    torch.testing.assert_close(R.layer_norm_fp32(x, w, b, 1e-6).float(), ref.float(), atol=tol, rtol=tol)


def test_bag_mean_bit_exact(ops_golden):
    table = torch.from_numpy(ops_golden["bag_table"].copy())
    for ids_key, out_key in (("bag_ids", "bag_out"), ("bag1_ids", "bag1_out")):
        ids = torch.from_numpy(ops_golden[ids_key].copy())
        got = R.embedding_bag_mean(table, ids)
        assert torch.equal(got, torch.from_numpy(ops_golden[out_key].copy())), ids_key
    # an all-padding bag is zero; a bag of one id is the row itself
    assert torch.equal(R.embedding_bag_mean(table, torch.zeros(2, 3, dtype=torch.int64)), torch.zeros(2, 16))
    assert torch.equal(R.embedding_bag_mean(table, torch.tensor([[17]])), table[17:18])


def test_attention_mask_families(ops_golden):
    q, k, v = (torch.from_numpy(ops_golden[f"attn_{n}"].copy()) for n in "qkv")
    lens = torch.from_numpy(ops_golden["attn_lens"].copy())
    B, H, T, D = q.shape
    # prefix key-padding
    m = R.structured_attention_mask(lens, T, T, causal=False, padded_query_self=False)
    torch.testing.assert_close(R.attention(q, k, v, m[:, None]), torch.from_numpy(ops_golden["attn_out_keypad"]), atol=2e-6, rtol=1e-5)
    assert np.array_equal(ops_golden["plan_keypad_lengths"], lens.numpy())
    # plain causal
    m = R.structured_attention_mask(torch.full((B,), T), T, T, causal=True, padded_query_self=False)
    torch.testing.assert_close(R.attention(q, k, v, m[:, None]), torch.from_numpy(ops_golden["attn_out_causal_nomask"]), atol=2e-6, rtol=1e-5)
    # causal + valid prefix + padded-query self fallback: both mask builders agree with the reference's
    m = R.structured_attention_mask(lens, T, T, causal=True, padded_query_self=True)
    ref_mask = torch.from_numpy(ops_golden["attn_mask_causal_valid"])
    assert torch.equal(m, ref_mask)
    assert torch.equal(R.causal_valid_attention_mask(R.make_padding_mask(lens, T)), ref_mask)
    torch.testing.assert_close(R.attention(q, k, v, m[:, None]), torch.from_numpy(ops_golden["attn_out_causal_valid"]), atol=2e-6, rtol=1e-5)
    assert np.array_equal(ops_golden["plan_causal_valid_lengths"], lens.numpy())
    assert np.array_equal(ops_golden["plan_causal_valid_self"], R.make_padding_mask(lens, T).numpy())
    # OneTrans layout: valid prefix, padding, always-valid NS suffix
    seq_lens = torch.from_numpy(ops_golden["attn_ns_seq_lens"].copy())
    m = R.structured_attention_mask(seq_lens, T, T - 5, causal=True, padded_query_self=True)
    assert torch.equal(m, torch.from_numpy(ops_golden["attn_mask_ns"]))
    torch.testing.assert_close(R.attention(q, k, v, m[:, None]), torch.from_numpy(ops_golden["attn_out_ns"]), atol=2e-6, rtol=1e-5)


def test_integer_helpers_bit_exact(ops_golden):
    g = ops_golden
    assert np.array_equal(R.hash_compress_ids(g["hash_in"], 7), g["hash_out_7"])
    assert np.array_equal(R.hash_compress_ids(g["hash_in"], 0), g["hash_out_0"])
    v, l, t = R.deduplicate_sequence_events(g["seq_values"], g["seq_lengths"], g["seq_ts"])
    assert np.array_equal(v, g["dedup_values"])
    assert np.array_equal(l, g["dedup_lengths"])
    assert np.array_equal(t, g["dedup_ts"])
    assert np.array_equal(R.sequence_time_buckets(g["seq_ts"], g["seq_req"]), g["seq_buckets"])
    edge = R.sequence_time_buckets(10**11 - g["bucket_edge_gaps"], np.array([10**11]))
    assert np.array_equal(edge, g["bucket_edge_out"])
    stats = R.sequence_stats(g["seq_values"], g["seq_lengths"], g["seq_ts"], g["seq_req"])
    assert np.array_equal(stats, g["seq_stats"])


def test_pooling_positions_auc(ops_golden):
    g = ops_golden
    got = R.masked_mean(torch.from_numpy(g["mm_tokens"].copy()), torch.from_numpy(g["mm_mask"].copy()))
    torch.testing.assert_close(got, torch.from_numpy(g["mm_out"]), atol=1e-6, rtol=1e-6)
    assert torch.equal(R.sinusoidal_positions(9, 16), torch.from_numpy(g["sinus_9_16"]))
    assert R.binary_auc(g["auc_labels"], g["auc_scores"]) == pytest.approx(float(g["auc_value"]), abs=1e-12)


@pytest.mark.parametrize("name", ["onetrans_a", "onetrans_b"])
def test_onetrans_forward_matches_reference(name):
    sd, spec, inputs, logits, embeddings = load_onetrans_fixture(name)
    got_logits, got_emb = oracle_model.predict(sd, spec, inputs)
    torch.testing.assert_close(got_emb, embeddings, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(got_logits, logits, atol=2e-5, rtol=1e-4)
    scores = oracle_model.sigmoid_scores(got_logits)
    assert np.abs(scores - torch.sigmoid(logits).numpy()).max() < 1e-5


@pytest.mark.parametrize("name", ["onetrans_a", "onetrans_b"])
def test_vectorised_cpu_port_matches_reference(name):
    """The multi-threaded CPU port that the benchmark times is held to the same golden outputs."""
    from oracle import torch_cpu

    sd, spec, inputs, logits, embeddings = load_onetrans_fixture(name)
    got_logits, got_emb = torch_cpu.predict(sd, spec, inputs)
    torch.testing.assert_close(got_emb, embeddings, atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(got_logits, logits, atol=2e-5, rtol=1e-4)
    # bf16 tables (the serving configuration) only move the result by table rounding
    sd16 = {k: (v.bfloat16() if "embeddings." in k and k.endswith(".weight") and "missing" not in k else v) for k, v in sd.items()}
    lo, _ = torch_cpu.predict(sd16, spec, inputs)
    assert (torch.sigmoid(lo) - torch.sigmoid(logits)).abs().max().item() < 5e-3
