"""Shared pytest setup: marker registration and fixture loaders."""

from __future__ import annotations

import json
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden"


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100) and the built libtb200.so")


def bf16_from_bits(a: np.ndarray) -> torch.Tensor:
    """Fixtures store bf16 as raw int16 bit patterns."""
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def golden_tensor(a: np.ndarray, bf16: bool = False) -> torch.Tensor:
    return bf16_from_bits(a) if bf16 else torch.from_numpy(a.copy())


@pytest.fixture(scope="session")
def ops_golden() -> dict[str, np.ndarray]:
    with np.load(GOLDEN / "ops.npz") as data:
        return {k: data[k] for k in data.files}


def load_onetrans_fixture(name: str):
    """-> (state_dict, spec dict, inputs namespace, logits, embeddings) from tests/golden/<name>.npz."""
    with np.load(GOLDEN / f"{name}.npz") as data:
        arrays = {k: data[k] for k in data.files}
    sd = {k[3:]: torch.from_numpy(v.copy()) for k, v in arrays.items() if k.startswith("sd/")}
    spec = json.loads(bytes(arrays["spec_json"]).decode())
    spec["user_int_specs"] = [tuple(s) for s in spec["user_int_specs"]]
    spec["item_int_specs"] = [tuple(s) for s in spec["item_int_specs"]]
    t = lambda key: torch.from_numpy(arrays[key].copy())  # noqa: E731

    def entity(who: str):
        return SimpleNamespace(
            int_values=t(f"in/{who}/int_values"), int_missing_mask=t(f"in/{who}/int_missing_mask"),
            dense_values=t(f"in/{who}/dense_values"), dense_missing_mask=t(f"in/{who}/dense_missing_mask"),
        )

    domains = sorted({k.split("/")[2] for k in arrays if k.startswith("in/seq/")})
    sequences = {
        d: SimpleNamespace(values=t(f"in/seq/{d}/values"), lengths=t(f"in/seq/{d}/lengths"), timestamps=t(f"in/seq/{d}/timestamps"))
        for d in domains
    }
    inputs = SimpleNamespace(user=entity("user"), item=entity("item"), sequences=sequences,
                             request_timestamp=t("in/request_timestamp"))
    return sd, spec, inputs, t("out/logits"), t("out/embeddings")


def gpu_ready() -> bool:
    if not torch.cuda.is_available():
        return False
    from taac_2026_b200 import ops

    return ops.cuda_available()
