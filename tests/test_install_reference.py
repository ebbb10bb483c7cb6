"""`install()` against the reference itself: a checkout named by TAAC2026_REFERENCE or lying beside this
repository, else the byte-compiled modules under oracle/_ref (`python -m oracle.build_ref`); skipped when
neither exists.  The CUDA operators are replaced by recording fakes — the pattern the reference's own
tests use for backends they cannot run (tests/unit/infrastructure/accelerators/test_tilelang_ops.py:222-302)
— so the routing is checked without a GPU."""

from __future__ import annotations

import pytest
import torch

from oracle import ref_runtime

pytestmark = pytest.mark.skipif(not ref_runtime.available(), reason="no reference checkout and no oracle/_ref available")


@pytest.fixture()
def installed(monkeypatch):
    ref_runtime.import_reference()
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


def test_config_layer_accepts_the_literal_only_while_installed(installed):
    tb, _ = installed
    from taac2026.domain import config as cfg

    made = cfg.PCVRModelConfig(rms_norm_backend="cuda", flash_attention_backend="cuda")
    assert (made.rms_norm_backend, made.flash_attention_backend) == ("cuda", "cuda")
    assert "cuda" in cfg.RMS_NORM_BACKEND_CHOICES and "cuda" in cfg.FLASH_ATTENTION_BACKEND_CHOICES
    assert cfg.PCVRModelConfig(rms_norm_backend="triton").rms_norm_backend == "triton"   # the reference's own names still pass
    with pytest.raises(Exception, match="rms_norm"):
        cfg.PCVRModelConfig(rms_norm_backend="nope")
    tb.uninstall()
    with pytest.raises(Exception):
        cfg.PCVRModelConfig(rms_norm_backend="cuda")
    assert "cuda" not in cfg.RMS_NORM_BACKEND_CHOICES
    tb.install()


def test_resolvers_answer_cuda_in_every_namespace(installed, monkeypatch):
    tb, _ = installed
    from taac2026.infrastructure import accelerators as acc
    from taac2026.infrastructure.accelerators import attention, embedding, normalization
    from taac_2026_b200 import ops

    seen = []
    for name in ("resolved_rms_norm_backend", "resolved_layer_norm_backend", "resolved_flash_attention_backend",
                 "resolved_embedding_bag_mean_backend"):
        monkeypatch.setattr(ops, name, lambda *a, _n=name, **k: seen.append((_n, a[-1] if isinstance(a[-1], str) else k)) or "cuda")
    tb.uninstall()
    tb.install()      # re-wrap with the recording resolvers in place
    x = torch.ones(2, 4)
    q = torch.ones(1, 1, 2, 4)
    ids = torch.ones(2, 3, dtype=torch.long)
    for holder in (acc, normalization):
        assert holder.resolved_rms_norm_backend(x, "cuda", eps=1e-6) == "cuda"
        assert holder.resolved_layer_norm_backend(x, backend="cuda") == "cuda"
    for holder in (acc, attention):
        assert holder.resolved_flash_attention_backend(q, q, q, "cuda", is_causal=True) == "cuda"
    for holder in (acc, embedding):
        assert holder.resolved_embedding_bag_mean_backend(x, ids, "cuda") == "cuda"
    assert len(seen) == 8
    assert acc.resolved_rms_norm_backend(x, "torch") == "torch"          # other names reach the reference's resolver
    with pytest.raises(ValueError):
        acc.resolved_rms_norm_backend(x, "nope")


def test_operator_benchmark_cli_takes_the_cuda_backend(installed, monkeypatch):
    tb, calls = installed
    from taac2026.application.benchmarking import pcvr_tilelang_ops_benchmark as bench
    from taac_2026_b200 import ops

    monkeypatch.setattr(ops, "compile_rms_norm_kernel", lambda x, w, eps=1e-6, **kw: (lambda x_, w_: bench._reference_rms_norm(x_, w_, eps)))
    monkeypatch.setattr(ops, "compile_layer_norm_kernel",
                        lambda x, w, b, eps=1e-5, **kw: (lambda x_, w_, b_: bench._reference_layer_norm(x_, w_, b_, eps)))
    for operator in ("rms_norm", "layer_norm"):
        args = bench.parse_args(["--operator", operator, "--backends", "torch,cuda", "--device", "cpu", "--rows", "16", "--cols", "32",
                                 "--steps", "2", "--warmup-steps", "1", "--repeats", "1", "--dtype", "float32"])
        assert args.backends == ("torch", "cuda")
        summary = bench.run_benchmark(args)
        by_backend = {r["backend"]: r for r in summary["results"]}
        assert by_backend["cuda"]["status"] == "ok" and by_backend["cuda"]["resolved_backend"] == "cuda", by_backend["cuda"]
    tb.uninstall()
    with pytest.raises(ValueError, match="unsupported backends"):
        bench.parse_args(["--operator", "rms_norm", "--backends", "cuda"])
    tb.install()


def test_route_all_leaves_training_calls_differentiable(installed):
    """The kernels are forward-only.  With every backend routed here wholesale, a call that needs gradients goes to
    the reference's torch path instead of silently cutting the graph; an explicit backend="cuda" is left to the
    operator, which refuses."""
    tb, calls = installed
    from taac2026.infrastructure import accelerators as acc
    from taac_2026_b200 import ops

    tb.install(route_all=True)
    x = torch.ones(2, 4, requires_grad=True)
    w = torch.ones(4, requires_grad=True)
    out = acc.rms_norm(x, w, backend="torch")
    out.sum().backward()
    assert w.grad is not None and calls == []
    with torch.no_grad():
        acc.rms_norm(x, w, backend="torch")
    assert calls == ["rms_norm"]
    with pytest.raises(RuntimeError, match="forward-only"):
        ops._refuse_autograd("rms_norm", x, w)
    with torch.no_grad():
        ops._refuse_autograd("rms_norm", x, w)      # no gradient is being recorded: nothing to refuse
    tb.install(route_all=False)
