"""Host-side behaviour of the ``cuda`` operator boundary that needs no GPU: validation order,
exception types and messages follow the reference dispatchers
(tests/unit/infrastructure/accelerators/test_tilelang_ops.py:222-302 is the model)."""

from __future__ import annotations

import pytest
import torch

from taac_2026_b200 import ops


def test_shape_errors_are_value_errors():
    with pytest.raises(ValueError, match="at least 2 dimensions"):
        ops.rms_norm(torch.ones(4), torch.ones(4))
    with pytest.raises(ValueError, match="weight must be a 1D tensor"):
        ops.rms_norm(torch.ones(2, 4), torch.ones(1, 4))
    with pytest.raises(ValueError, match="does not match weight size"):
        ops.rms_norm(torch.ones(2, 4), torch.ones(3))
    with pytest.raises(ValueError, match="bias must be a 1D tensor"):
        ops.layer_norm(torch.ones(2, 4), torch.ones(4), torch.ones(1, 4))
    with pytest.raises(ValueError, match="does not match bias shape"):
        ops.layer_norm(torch.ones(2, 4), torch.ones(4), torch.ones(3))
    with pytest.raises(ValueError, match="weight must be a 2D tensor"):
        ops.embedding_bag_mean(torch.ones(4), torch.ones(2, 2, dtype=torch.long))
    with pytest.raises(ValueError, match="values must be a 2D tensor"):
        ops.embedding_bag_mean(torch.ones(4, 4), torch.ones(2, dtype=torch.long))


def test_unknown_backend_is_value_error():
    with pytest.raises(ValueError, match="unsupported rms_norm backend: tilelang"):
        ops.rms_norm(torch.ones(2, 4), torch.ones(4), backend="tilelang")
    with pytest.raises(ValueError, match="unsupported layer_norm backend"):
        ops.layer_norm(torch.ones(2, 4), torch.ones(4), torch.ones(4), backend="triton")


def test_no_silent_cpu_fallback(monkeypatch):
    """An explicit accelerated backend on CPU tensors raises, even when the backend is available."""
    monkeypatch.setattr(ops, "cuda_available", lambda: True)
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        ops.rms_norm(torch.ones(2, 4), torch.ones(4))
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        ops.layer_norm(torch.ones(2, 4), torch.ones(4), torch.ones(4))
    with pytest.raises(RuntimeError, match="requires CUDA tensors"):
        ops.embedding_bag_mean(torch.ones(4, 4), torch.ones(2, 2, dtype=torch.long))


def test_unavailable_backend_is_runtime_error(monkeypatch):
    monkeypatch.setattr(ops, "cuda_available", lambda: False)
    with pytest.raises(RuntimeError, match="cuda backend requested but"):
        ops.rms_norm(torch.ones(2, 4), torch.ones(4))
    with pytest.raises(RuntimeError, match="cuda backend requested but"):
        ops.resolved_embedding_bag_mean_backend(torch.ones(4, 4), torch.ones(2, 2, dtype=torch.long))


def test_newer_entry_points_have_no_cpu_path_either(monkeypatch):
    """The fused tokenizer tail, the packed-layout index kernel, the grouped GEMM and the attention kernels refuse
    CPU tensors when the backend is available, and say that the backend is missing when it is not."""
    x = torch.ones(4, 64, dtype=torch.bfloat16)
    w = torch.ones(1, 256, 64, dtype=torch.bfloat16)
    ids = torch.zeros(4, dtype=torch.long)
    calls = [
        lambda: ops.grouped_linear(x[None], w),
        lambda: ops.token_tail(x, x[0], x[0], x, ids, None, None, x[0]),
        lambda: ops.packed_token_index(torch.zeros(1, 1, 4, dtype=torch.long), None, torch.zeros(1, dtype=torch.long),
                                       torch.zeros(1, 4, dtype=torch.int32), torch.tensor([0, 4]), torch.tensor([2]),
                                       torch.tensor([0]), torch.tensor([0]), 4),
        lambda: ops.varlen_attention(x.view(4, 1, 64), x.view(4, 1, 64), x.view(4, 1, 64), cu_rows=torch.tensor([0, 4], dtype=torch.int32),
                                     max_rows=4, kernel=4),
    ]
    monkeypatch.setattr(ops, "cuda_available", lambda: True)
    for call in calls:
        with pytest.raises(RuntimeError, match="requires CUDA tensors"):
            call()
    monkeypatch.setattr(ops, "cuda_available", lambda: False)
    for call in calls:
        with pytest.raises(RuntimeError, match="cuda backend requested but"):
            call()
