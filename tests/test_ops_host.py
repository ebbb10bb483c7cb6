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
