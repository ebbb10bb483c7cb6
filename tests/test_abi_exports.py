"""The shared library loads on a machine without a GPU and exports every symbol the public
header declares; the ctypes table in ``_lib.py`` and the header stay in step."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from taac_2026_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "tb200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    names = declared_symbols()
    assert "tb200_rmsnorm_fwd" in names and "tb200_strerror" in names


def test_ctypes_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_library_exports_every_symbol():
    if not _lib.library_available():
        pytest.fail("libtb200.so is not built; run `python -m taac_2026_b200.build`")
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in tb200.h but not exported"


def test_status_text_and_version():
    lib = _lib.load()
    assert lib.tb200_abi_version() >= 1
    assert _lib.strerror(0) == "ok"
    for code in range(-8, 0):
        assert _lib.strerror(code).startswith("tb200:")
    with pytest.raises(ValueError):
        _lib.check(-3, "x")
    with pytest.raises(RuntimeError):
        _lib.check(-6, "x")


def test_argument_errors_need_no_gpu():
    """Rejected arguments return before any CUDA call."""
    lib = _lib.load()
    assert lib.tb200_rmsnorm_fwd(None, None, None, -1, 8, 1e-6, _lib.F32, None) == -3
    assert lib.tb200_rmsnorm_fwd(None, None, None, 0, 8, 1e-6, _lib.F32, None) == 0  # empty input: nothing to do
    assert lib.tb200_rmsnorm_fwd(None, None, None, 4, 8, 1e-6, _lib.F32, None) == -1
    assert lib.tb200_layernorm_fwd(None, None, None, None, 4, 0, 1e-6, _lib.F32, None) == -3
    assert lib.tb200_bag_mean_fwd(None, 10, 8, None, _lib.I64, 4, 2, None, _lib.F32, None) == -1
    assert lib.tb200_gather_rows(None, 10, 8, None, 7, 4, 4, 0, None, 8, 0, _lib.F32, None) == -2
