"""The baseline-sized configuration at its full size on the GPU: batch 512, 32 sparse fields (24 user + 8 item) of
100 000 ids and 64 columns, Zipf(1.2) ids, 16 dense features, one behaviour sequence over 1 000 000 ids
(Zipf 1.1) with lengths uniform in [16, 256] right-padded to 256, d_model 128, 4 heads, 2 blocks, hidden 4 x,
fp32 weights from seed 0.

Oracle: the reference's own ``PCVROneTrans.predict`` on the CPU (torch backend, fp32) with the parameters of its
own seed-0 initialisation, where the reference can be imported (a checkout or ``oracle/_ref``); otherwise the
vectorised port ``oracle/torch_cpu.py`` with this repository's seeded generator.  Bounds: sigmoid scores within
1e-3 and the AUC (labels ~ Bernoulli(0.1), independent of the inputs) equal to four decimals in the fp32 mode;
the bf16 serving mode is held to the same 1e-3 on the scores.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import gpu_ready
from oracle import ref_runtime, torch_cpu
from oracle import reference_ops as R
from taac_2026_b200.inputs import OneTransSpec, synthetic_batch
from taac_2026_b200.onetrans import OneTransInference, random_state_dict

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def c1_spec() -> OneTransSpec:
    return OneTransSpec(
        user_int_specs=[(100_000, i, 1) for i in range(24)], item_int_specs=[(100_000, i, 1) for i in range(8)],
        user_dense_dim=16, item_dense_dim=0, seq_vocab_sizes={"seq_a": [1_000_000]}, d_model=128, emb_dim=64,
        num_blocks=2, num_heads=4, hidden_mult=4, seq_top_k=256, user_ns_tokens=5, item_ns_tokens=2,
    )


@pytest.fixture(scope="module")
def c1_case():
    spec = c1_spec()
    batch = synthetic_batch(spec, 512, seq_len=256, min_len=16, seed=0, field_exponent=1.2, seq_exponent=1.1)
    if ref_runtime.available():
        model = ref_runtime.build_model(spec.as_dict(), seed=0)          # the reference's own seed-0 parameter stream
        sd = {name: t.detach().clone() for name, t in model.state_dict().items()}
        want_logits, _ = ref_runtime.predict(model, batch)
        source = "reference PCVROneTrans.predict"
        del model
    else:
        sd = random_state_dict(spec, seed=0)
        want_logits, _ = torch_cpu.predict(sd, spec.as_dict(), batch)
        source = "oracle/torch_cpu.py"
    want = torch.sigmoid(want_logits.reshape(-1).float()).numpy()
    labels = (torch.rand(512, generator=torch.Generator().manual_seed(1)) < 0.1).numpy()
    return spec, sd, batch, want, labels, source


@pytest.mark.parametrize("packed", [True, False])
def test_fp32_scores_and_auc(c1_case, packed):
    spec, sd, batch, want, labels, source = c1_case
    model = OneTransInference(sd, spec, dtype=torch.float32, packed=packed)
    got = model.scores(batch.to("cuda")).cpu().numpy()
    model.raise_if_incomplete()
    auc_got, auc_want = R.binary_auc(labels, got), R.binary_auc(labels, want)
    print(f"oracle={source} packed={packed} max|dscore|={np.abs(got - want).max():.2e} auc cuda={auc_got:.6f} oracle={auc_want:.6f}")
    assert np.abs(got - want).max() <= 1e-3
    assert round(auc_got, 4) == round(auc_want, 4) or abs(auc_got - auc_want) < 5e-5


def test_bf16_serving_mode_scores(c1_case):
    spec, sd, batch, want, labels, source = c1_case
    model = OneTransInference(sd, spec, dtype=torch.bfloat16)
    got = model.scores(batch.to("cuda")).cpu().numpy()
    model.raise_if_incomplete()
    auc_got, auc_want = R.binary_auc(labels, got), R.binary_auc(labels, want)
    print(f"oracle={source} bf16 max|dscore|={np.abs(got - want).max():.2e} auc cuda={auc_got:.6f} oracle={auc_want:.6f}")
    assert np.abs(got - want).max() <= 1e-3
    assert abs(auc_got - auc_want) <= 2e-3
