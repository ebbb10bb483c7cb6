"""The reference's OWN model (`PCVROneTrans`, experiments/onetrans/model.py) on the GPU with the one-line switch set
to ``cuda`` after ``install()``, against the same module on its ``torch`` backend: the drop-in claim with the real
kernels underneath.  The model is built the way `build_prediction_model` builds it
(src/taac2026/application/evaluation/workflow.py:116-129): the backends come from ``PCVRModelConfig``.

Needs the reference (a checkout, or the byte-compiled modules of ``python -m oracle.build_ref``)."""

from __future__ import annotations

import pytest
import torch

from conftest import gpu_ready
from oracle import ref_runtime
from taac_2026_b200 import _lib
from taac_2026_b200.inputs import OneTransSpec, synthetic_batch

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_runtime.available(), reason="no reference checkout and no oracle/_ref available")]


@pytest.fixture(autouse=True)
def _need_gpu():
    if not gpu_ready():
        pytest.fail("gpu tests need an sm_100 device and a built libtb200.so")


def _spec() -> OneTransSpec:
    return OneTransSpec(
        user_int_specs=[(1000, i, 1) for i in range(6)], item_int_specs=[(1000, i, 1) for i in range(3)],
        user_dense_dim=8, item_dense_dim=0, seq_vocab_sizes={"seq_a": [5000]}, d_model=128, emb_dim=64,
        num_blocks=2, num_heads=2, hidden_mult=4, seq_top_k=96, user_ns_tokens=3, item_ns_tokens=2,
    )


def test_reference_model_with_cuda_backends_matches_its_torch_backends():
    from taac_2026_b200 import install as tb

    ref_runtime.import_reference()
    spec = _spec().as_dict()
    batch = synthetic_batch(_spec(), 96, seq_len=96, min_len=4, seed=3).to("cuda")
    plain = ref_runtime.build_model(spec, seed=0, device="cuda")
    want, _ = ref_runtime.predict(plain, batch)
    weights = plain.state_dict()
    tb.install()
    try:
        switched = ref_runtime.build_model(spec, seed=None, state_dict=weights, device="cuda",
                                           rms_norm_backend="cuda", flash_attention_backend="cuda")
        assert all(m.backend == "cuda" for m in switched.modules() if type(m).__name__ == "RMSNorm")
        before = _lib.launch_count()
        got, _ = ref_runtime.predict(switched, batch)
        torch.cuda.synchronize()
        launched = _lib.launch_count() - before
    finally:
        tb.uninstall()
        from taac2026.infrastructure.modeling import normalization as m_norm
        from taac2026.infrastructure.modeling import sequence as m_seq

        m_norm.configure_rms_norm_runtime(backend="torch", block_rows=1)     # the two context-wide switches back to torch
        m_seq.configure_flash_attention_runtime(backend="torch")
    # 2 blocks x (2 norms + 1 attention) + the final norm, and the bag-mean hook of both NS tokenizers
    assert launched >= 7, f"only {launched} launches of this library: the cuda backend was not reached"
    # fp32 callers of accelerated attention are computed in bf16 and cast back (flash_attention.py:249-252)
    assert (torch.sigmoid(got) - torch.sigmoid(want)).abs().max().item() <= 1e-3
    assert (got - want).abs().max().item() <= 2e-2
