"""`install()` against a real checkout of the reference, when one is importable (set
TAAC2026_REFERENCE=/path/to/TAAC_2026 or have `taac2026` on sys.path); skipped otherwise, e.g. on
the GPU box.  The CUDA operators are replaced by recording fakes — the pattern the reference's own
tests use for backends they cannot run (tests/unit/infrastructure/accelerators/test_tilelang_ops.py:222-302)
— so the routing is checked without a GPU."""

from __future__ import annotations

import json
import os
import sys
import types
from pathlib import Path

import pytest
import torch


def _reference_root() -> Path | None:
    # the checkout named by TAAC2026_REFERENCE, else a sibling `reference/` directory of this repository
    sibling = Path(__file__).resolve().parents[2] / "reference"
    for candidate in (os.environ.get("TAAC2026_REFERENCE"), str(sibling)):
        if candidate and (Path(candidate) / "src" / "taac2026").is_dir():
            return Path(candidate)
    return None


ROOT = _reference_root()
pytestmark = pytest.mark.skipif(ROOT is None, reason="no reference checkout available")


@pytest.fixture()
def installed(monkeypatch):
    if "orjson" not in sys.modules:
        try:
            import orjson  # noqa: F401
        except ImportError:
            shim = types.ModuleType("orjson")
            shim.OPT_INDENT_2 = shim.OPT_SORT_KEYS = shim.OPT_SERIALIZE_NUMPY = shim.OPT_NON_STR_KEYS = 0
            shim.dumps = lambda obj, default=None, option=0: json.dumps(obj, default=default).encode()
            shim.loads = json.loads
            shim.JSONDecodeError = json.JSONDecodeError
            monkeypatch.setitem(sys.modules, "orjson", shim)
    for path in (ROOT / "src", ROOT):
        if str(path) not in sys.path:
            monkeypatch.syspath_prepend(str(path))
    from taac_2026_b200 import install as tb
    from taac_2026_b200 import ops

    calls: list[str] = []
    monkeypatch.setattr(ops, "rms_norm", lambda x, w, eps=1e-6, **kw: calls.append("rms_norm") or x * 2)
    monkeypatch.setattr(ops, "layer_norm", lambda x, w, b, eps=1e-5, **kw: calls.append("layer_norm") or x * 3)
    monkeypatch.setattr(ops, "flash_attention", lambda q, k, v, **kw: calls.append("flash_attention") or v)
    monkeypatch.setattr(ops, "embedding_bag_mean", lambda w, v, **kw: calls.append("embedding_bag_mean") or w[:1].expand(v.shape[0], -1))
    tb.install()
    yield tb, calls
    tb.uninstall()


def test_cuda_literal_routes_to_this_library(installed):
    tb, calls = installed
    from taac2026.infrastructure import accelerators as acc
    from taac2026.infrastructure.modeling import normalization as m_norm
    from taac2026.infrastructure.modeling import sequence as m_seq

    x, w = torch.ones(2, 4), torch.ones(4)
    assert torch.equal(acc.rms_norm(x, w, backend="cuda"), x * 2)
    assert torch.equal(acc.layer_norm(x, w, w, backend="cuda"), x * 3)
    q = torch.ones(1, 1, 2, 4)
    assert torch.equal(acc.flash_attention(q, q, q * 5, backend="cuda"), q * 5)
    assert calls == ["rms_norm", "layer_norm", "flash_attention"]
    # other backends still reach the reference's own code
    torch.testing.assert_close(acc.rms_norm(x, w, backend="torch"), x / torch.sqrt(torch.tensor(1.0 + 1e-6)))
    with pytest.raises(ValueError, match="unsupported rms_norm backend"):
        acc.rms_norm(x, w, backend="nope")
    # the one-line switch accepts the new literal; RMSNorm captures it at construction, attention reads it at call time
    m_norm.configure_rms_norm_runtime(backend="cuda", block_rows=1)
    m_seq.configure_flash_attention_runtime(backend="cuda")
    try:
        norm = m_norm.RMSNorm(4)
        assert norm.backend == "cuda"
        assert torch.equal(norm(x), x * 2)
        out = m_seq.scaled_dot_product_attention(torch.ones(1, 2, 4), torch.ones(1, 2, 4), torch.ones(1, 2, 4) * 7,
                                                 num_heads=1, attn_mask=None, dropout_p=0.0, training=False)
        assert torch.equal(out, torch.ones(1, 2, 4) * 7)
    finally:
        m_norm.configure_rms_norm_runtime(backend="torch", block_rows=1)
        m_seq.configure_flash_attention_runtime(backend="torch")
    assert m_norm.RMSNorm(4).backend == "torch"


def test_uninstall_restores_reference(installed):
    tb, _calls = installed
    from taac2026.infrastructure.modeling import normalization as m_norm

    tb.uninstall()
    with pytest.raises(ValueError, match="unsupported rms_norm backend"):
        m_norm.configure_rms_norm_runtime(backend="cuda", block_rows=1)
    tb.install()  # the fixture's teardown expects an installed state


def test_spec_from_reference_matches_fixture_spec(installed):
    tb, _ = installed
    from taac2026.domain.config import PCVRModelConfig, PCVRNSConfig
    from taac2026.domain.schema import PCVRSchema

    schema = PCVRSchema(format="raw_parquet", user_int=[[1, 40, 1], [2, 41, 2]], item_int=[[10, 30, 1]], user_dense=[[1, 4]],
                        item_dense=[], seq={"seq_a": {"prefix": "seq_a", "ts_fid": 1, "features": [[1, 0], [2, 90]]}})
    config = PCVRModelConfig(d_model=64, emb_dim=16, num_blocks=2, num_heads=2, seq_top_k=40, use_time_buckets=True,
                             ns=PCVRNSConfig(grouping_strategy="singleton", tokenizer_type="rankmixer", user_tokens=2, item_tokens=1))
    spec = tb.spec_from_reference(schema, config)
    assert spec.user_int_specs == [(40, 0, 1), (41, 1, 2)] and spec.item_int_specs == [(30, 0, 1)]
    assert spec.seq_vocab_sizes == {"seq_a": [90]} and spec.num_time_buckets == 64 and spec.user_dense_dim == 4
