"""End-to-end GPU parity of the OneTrans inference engine.

* against the reference's own logits / pooled embeddings (golden fixtures exported from the unmodified
  reference model), in the fp32 dense mode: sigmoid scores within 1e-3 (the task's bound);
* against the CPU oracle on a seeded synthetic batch with the baseline model shape in miniature
  (32 sparse fields, Zipf ids, ragged behaviour sequence): scores within 1e-3 and AUC equal
  to 4 decimals; the bf16 serving mode is held to 5e-3 on the same batch.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import gpu_ready, load_onetrans_fixture
from oracle import onetrans as oracle_model
from oracle import reference_ops as R
from taac_2026_b200.inputs import EntityInput, ModelInput, OneTransSpec, SequenceInput, synthetic_batch
from taac_2026_b200.onetrans import OneTransInference, random_state_dict

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _spec_from_dict(d: dict) -> OneTransSpec:
    fields = {k: d[k] for k in OneTransSpec.__dataclass_fields__ if k in d}
    return OneTransSpec(**fields)


def _to_model_input(ns) -> ModelInput:
    ent = lambda e: EntityInput(e.int_values, e.int_missing_mask, e.dense_values, e.dense_missing_mask)  # noqa: E731
    return ModelInput(ent(ns.user), ent(ns.item),
                      {k: SequenceInput(s.values, s.lengths, s.timestamps) for k, s in ns.sequences.items()},
                      ns.request_timestamp)


@pytest.mark.parametrize("packed", [True, False])
@pytest.mark.parametrize("name", ["onetrans_a", "onetrans_b"])
def test_matches_reference_golden(name, packed):
    """onetrans_a has one sequence domain (packed valid-token layout by default), onetrans_b two
    domains, time buckets, hashed tables and a tail crop (padded layout with a key-validity map)."""
    sd, spec_dict, inputs, logits, embeddings = load_onetrans_fixture(name)
    spec = _spec_from_dict(spec_dict)
    model = OneTransInference(sd, spec, dtype=torch.float32, packed=packed)
    got_logits, got_emb = model.predict(_to_model_input(inputs).to("cuda"))
    assert np.abs(torch.sigmoid(got_logits).cpu().numpy() - torch.sigmoid(logits).numpy()).max() <= 1e-3
    torch.testing.assert_close(got_emb.cpu(), embeddings, atol=2e-2, rtol=2e-2)


def _mini_spec() -> OneTransSpec:
    return OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(24)], item_int_specs=[(1000, i, 1) for i in range(8)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=128, emb_dim=64,
        num_blocks=2, num_heads=4, hidden_mult=4, seq_top_k=96, user_ns_tokens=5, item_ns_tokens=2,
    )


@pytest.mark.parametrize("packed", [True, False])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 5e-3)])
def test_matches_oracle_on_synthetic_batch(dtype, tol, packed):
    """512 samples of the baseline shape in miniature.  Labels are drawn from the oracle's own logits
    (standardised, temperature 2) so that the AUC is well away from 0.5; the AUC of the CUDA scores must
    agree to 4 decimals (|difference| < 5e-5; comparing rounded strings would fail spuriously whenever
    the two values straddle a rounding boundary)."""
    spec = _mini_spec()
    sd = random_state_dict(spec, seed=0)
    batch = synthetic_batch(spec, 512, seq_len=96, min_len=4, seed=1)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    model = OneTransInference(sd, spec, dtype=dtype, packed=packed)
    got = model.scores(batch.to("cuda")).cpu().numpy()
    want = oracle_model.sigmoid_scores(want_logits).reshape(-1)
    assert np.abs(got - want).max() <= tol
    z = (want_logits.reshape(-1) - want_logits.mean()) / want_logits.std()
    labels = (torch.rand(512, generator=torch.Generator().manual_seed(2)) < torch.sigmoid(2.0 * z)).numpy()
    auc_got, auc_want = R.binary_auc(labels, got), R.binary_auc(labels, want)
    print(f"dtype={dtype} max|dscore|={np.abs(got - want).max():.2e} auc cuda={auc_got:.6f} oracle={auc_want:.6f}")
    if dtype == torch.float32:
        assert abs(auc_got - auc_want) < 5e-5  # equal to 4 decimals (half a unit in the 4th place)
    else:
        assert abs(auc_got - auc_want) <= 2e-3


def test_scores_are_batch_independent():
    """Samples are independent: scoring a batch in two halves gives the same numbers (what lets the
    job shard by batch across GPUs)."""
    spec = _mini_spec()
    sd = random_state_dict(spec, seed=3)
    batch = synthetic_batch(spec, 64, seq_len=96, min_len=1, seed=4).to("cuda")
    model = OneTransInference(sd, spec, dtype=torch.bfloat16)
    full = model.scores(batch)
    halves = torch.cat([model.scores(batch.slice(0, 32)), model.scores(batch.slice(32, 64))])
    assert (full - halves).abs().max().item() <= 2e-3


def _wide_spec() -> OneTransSpec:
    """Small tables, serving-size backbone (d 512, 8 heads of 64, hidden 2048): the shapes the FP8 FFN
    and the head_dim-64 attention kernels are built for."""
    return OneTransSpec(
        user_int_specs=[(500, i, 1) for i in range(6)], item_int_specs=[(500, i, 1) for i in range(3)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [3000]}, d_model=512, emb_dim=128,
        num_blocks=3, num_heads=8, hidden_mult=4, seq_top_k=200, user_ns_tokens=5, item_ns_tokens=2,
    )


@pytest.mark.parametrize("ffn,tol", [("bf16", 5e-3), ("fp8", 1e-2)])
def test_serving_shape_against_oracle(ffn, tol):
    """d_model 512 with a tail crop (sequence 260 > seq_top_k 200), packed layout, bf16 and FP8 FFN."""
    spec = _wide_spec()
    sd = random_state_dict(spec, seed=5)
    batch = synthetic_batch(spec, 48, seq_len=260, min_len=0, seed=6)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    want = oracle_model.sigmoid_scores(want_logits).reshape(-1)
    model = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn=ffn)
    got = model.scores(batch.to("cuda"), micro_batch=20).cpu().numpy()
    assert np.abs(got - want).max() <= tol
    padded = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn=ffn, packed=False).scores(batch.to("cuda")).cpu().numpy()
    assert np.abs(got - padded).max() <= tol


def test_score_stream_matches_resident_scores():
    """The pipelined serving loop (copy of batch i + 1 under the kernels of batch i) returns, batch by
    batch, exactly the scores of the plain call on device-resident inputs."""
    from taac_2026_b200.onetrans import score_stream

    spec = _mini_spec()
    sd = random_state_dict(spec, seed=0)
    model = OneTransInference(sd, spec, dtype=torch.bfloat16)
    host = [synthetic_batch(spec, 64, seq_len=96, min_len=4, seed=s).pin_memory() for s in (3, 4, 5, 6)]
    got = [s.clone() for s in score_stream(model, host, micro_batch=32)]
    torch.cuda.synchronize()
    assert len(got) == len(host)
    for scores, batch in zip(got, host):
        want = model.scores(batch.to("cuda"), micro_batch=32)
        assert torch.equal(scores, want)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-3), (torch.bfloat16, 5e-3)])
def test_blocks_with_only_ns_tokens_left(dtype, tol):
    """Short behaviour sequences under a deep pyramid: from some block on no sample has a sequence token left
    and the engine switches to its token-major NS-only blocks.  Scores must still match the oracle, which
    runs the reference's padded algorithm."""
    spec = OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(12)], item_int_specs=[(1000, i, 1) for i in range(6)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=128, emb_dim=64,
        num_blocks=4, num_heads=2, hidden_mult=4, seq_top_k=96, user_ns_tokens=4, item_ns_tokens=2,
    )
    sd = random_state_dict(spec, seed=3)
    batch = synthetic_batch(spec, 96, seq_len=96, min_len=1, seed=7)
    # keep every sequence short so that the pyramid's tail crop removes all of it after the first blocks
    short = batch.sequences["seq_a"].lengths.clamp(max=6)
    batch = ModelInput(batch.user, batch.item,
                       {"seq_a": SequenceInput(batch.sequences["seq_a"].values, short, batch.sequences["seq_a"].timestamps)},
                       batch.request_timestamp)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    model = OneTransInference(sd, spec, dtype=dtype)
    calls = []
    inner = model._ns_only_blocks
    model._ns_only_blocks = lambda tokens, first_layer, b: (calls.append(first_layer), inner(tokens, first_layer, b))[1]
    got = model.scores(batch.to("cuda")).cpu().numpy()
    assert calls and 0 < calls[0] < spec.num_blocks, "the NS-only path was expected to take over after the first block"
    want = oracle_model.sigmoid_scores(want_logits).reshape(-1)
    assert np.abs(got - want).max() <= tol


def test_per_token_layers_on_the_grouped_gemm():
    """bf16, d_model 256: the per-token layers of the non-sequence tokens run on the grouped tcgen05 GEMM (bias,
    SiLU and residual in its epilogue), in the mixed blocks and in the NS-only blocks.  The scores match the
    oracle, and the same model without the fused weights (library batched GEMMs + separate passes) agrees."""
    from taac_2026_b200 import ops

    spec = OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(12)], item_int_specs=[(1000, i, 1) for i in range(6)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=256, emb_dim=64,
        num_blocks=4, num_heads=4, hidden_mult=4, seq_top_k=96, user_ns_tokens=4, item_ns_tokens=2,
    )
    sd = random_state_dict(spec, seed=4)
    batch = synthetic_batch(spec, 200, seq_len=96, min_len=1, seed=8)
    short = batch.sequences["seq_a"].lengths.clamp(max=9)
    batch = ModelInput(batch.user, batch.item,
                       {"seq_a": SequenceInput(batch.sequences["seq_a"].values, short, batch.sequences["seq_a"].timestamps)},
                       batch.request_timestamp)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    want = oracle_model.sigmoid_scores(want_logits).reshape(-1)
    model = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn="bf16")
    assert all("g_w1" in blk for blk in model.blocks)
    records: list = []
    ops.set_kernel_timing(records)
    try:
        got = model.scores(batch.to("cuda"))
    finally:
        ops.set_kernel_timing(None)
    names = [r[0] for r in records]
    assert names.count("gemm_bf16") >= 5 and "bias_act_rows" not in names
    assert np.abs(got.cpu().numpy() - want).max() <= 5e-3
    for blk in model.blocks:                      # the same weights through the unfused path
        for key in [k for k in blk if k.startswith("g_")]:
            del blk[key]
    unfused = model.scores(batch.to("cuda"))
    assert (got - unfused).abs().max().item() <= 5e-3


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-3)])
def test_early_row_selection_changes_nothing(dtype, tol):
    """Selecting the rows the pyramid keeps before the row-wise half of a block (default) or after the whole
    block (the reference's order) gives the same scores."""
    spec = _mini_spec()
    sd = random_state_dict(spec, seed=0)
    batch = synthetic_batch(spec, 128, seq_len=96, min_len=4, seed=9).to("cuda")
    early = OneTransInference(sd, spec, dtype=dtype, select_early=True).scores(batch)
    late = OneTransInference(sd, spec, dtype=dtype, select_early=False).scores(batch)
    assert (early - late).abs().max().item() <= tol


@pytest.mark.parametrize("packed", [True, False])
def test_batch_without_any_behaviour_event(packed):
    """Every sequence is empty: the forward runs on the NS tokens alone from the first block on."""
    spec = _mini_spec()
    sd = random_state_dict(spec, seed=0)
    batch = synthetic_batch(spec, 40, seq_len=96, min_len=4, seed=11)
    seq = batch.sequences["seq_a"]
    batch = ModelInput(batch.user, batch.item, {"seq_a": SequenceInput(seq.values, torch.zeros_like(seq.lengths), seq.timestamps)},
                       batch.request_timestamp)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    got = OneTransInference(sd, spec, dtype=torch.float32, packed=packed).scores(batch.to("cuda")).cpu().numpy()
    assert np.abs(got - oracle_model.sigmoid_scores(want_logits).reshape(-1)).max() <= 1e-3


def test_one_kernel_tokenizer_gives_the_same_scores():
    """`fused_tokenizer=True` replaces gather + projection + tail by `ops.token_project`: same scores to bf16 rounding."""
    spec = _wide_spec()
    sd = random_state_dict(spec, seed=5)
    batch = synthetic_batch(spec, 48, seq_len=260, min_len=0, seed=6).to("cuda")
    plain = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn="fp8")
    fused = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn="fp8", fused_tokenizer=True)
    a, b = plain.scores(batch), fused.scores(batch)
    fused.raise_if_incomplete()
    assert (a - b).abs().max().item() <= 2e-3


def test_block_scaled_ffn_mode_gives_the_same_scores_as_the_amax_scaled_one():
    """ffn="fp8_mx" (power-of-two block scales inside the block-scaled tensor-core instruction) against ffn="fp8" on
    the serving-size backbone: both are e4m3 FFNs, so the scores agree to the e4m3 noise level, and both stay within
    the bf16-mode tolerance of the oracle."""
    spec = _wide_spec()
    sd = random_state_dict(spec, seed=5)
    batch = synthetic_batch(spec, 48, seq_len=260, min_len=0, seed=6)
    want_logits, _ = oracle_model.predict(sd, spec.as_dict(), batch)
    want = oracle_model.sigmoid_scores(want_logits).reshape(-1)
    base = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn="fp8").scores(batch.to("cuda")).cpu().numpy()
    model = OneTransInference(sd, spec, dtype=torch.bfloat16, ffn="fp8_mx")
    got = model.scores(batch.to("cuda")).cpu().numpy()
    model.raise_if_incomplete()
    assert np.abs(got - want).max() <= 1e-2
    assert np.abs(got - base).max() <= 1e-2
