"""ctypes binding of ``libtb200.so`` — the C-ABI library declared in ``include/tb200.h``.

There is no CPU fallback: if the library is missing or the current device is not an
sm_100 part, the operators raise ``RuntimeError`` exactly as the reference dispatchers do
for an accelerated backend that is unavailable
(src/taac2026/infrastructure/accelerators/normalization/rms_norm.py:89-104).
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libtb200.so"

F32, F16, BF16 = 0, 1, 2
I32, I64 = 0, 1

_c = ctypes
_P = _c.c_void_p
_I32 = _c.c_int32
_I64 = _c.c_int64
_INT = _c.c_int
_F = _c.c_float

# name -> (restype, argtypes); must list every symbol include/tb200.h declares.
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "tb200_strerror": (_c.c_char_p, [_INT]),
    "tb200_abi_version": (_INT, []),
    "tb200_device_ok": (_INT, []),
    "tb200_launch_count": (_I64, []),
    "tb200_rmsnorm_fwd": (_INT, [_P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_layernorm_fwd": (_INT, [_P, _P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_rmsnorm_bias_fwd": (_INT, [_P, _P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_layernorm_silu_fwd": (_INT, [_P, _P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_token_tail_fwd": (_INT, [_P, _P, _P, _P, _I64, _P, _P, _I64, _P, _P, _P, _P, _I64, _I32, _F, _F, _INT, _P]),
    "tb200_token_tail_select_fwd": (
        _INT, [_P, _P, _P, _P, _I64, _P, _P, _I64, _P, _P, _P, _I64, _P, _P, _I64, _I32, _F, _F, _INT, _P],
    ),
    "tb200_norm_bwd_workspace_bytes": (_I64, [_I32, _I32]),
    "tb200_rmsnorm_bwd": (_INT, [_P, _P, _P, _P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_layernorm_bwd": (_INT, [_P, _P, _P, _P, _P, _P, _P, _I64, _I32, _F, _INT, _P]),
    "tb200_token_project_fwd": (
        _INT, [_P, _P, _I32, _I32, _P, _P, _P, _P, _P, _P, _I64, _P, _P, _I64, _P, _P, _P, _I64, _P, _P, _I64, _I32, _F, _F, _P, _P],
    ),
    "tb200_add_gathered_rows": (_INT, [_P, _I64, _I32, _P, _I64, _P, _P, _I64, _P, _INT, _P]),
    "tb200_bias_act_rows": (_INT, [_P, _I64, _I32, _P, _I64, _I32, _INT, _P]),
    "tb200_bag_mean_fwd": (_INT, [_P, _I64, _I32, _P, _INT, _I64, _I32, _P, _INT, _P]),
    "tb200_bag_mean_bwd": (_INT, [_P, _INT, _P, _P, _P, _I64, _I32, _I32, _I64, _INT, _P]),
    "tb200_attn_bwd_workspace_bytes": (_I64, [_I32, _I32, _I32]),
    "tb200_attn_bwd": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _P, _P, _P, _I32, _I32, _I32,
                              _F, _INT, _P]),
    "tb200_mx_scale_bytes": (_I64, [_I64, _I32]),
    "tb200_quant_act_mx": (_INT, [_P, _P, _P, _I64, _I32, _P]),
    "tb200_mx_gemm": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _P, _P]),
    "tb200_pyramid_plan": (_INT, [_P, _I32, _I32, _P, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "tb200_pyramid_kept_rows": (_INT, [_P, _P, _P, _P, _I32, _I32, _P, _P, _P, _P]),
    "tb200_host_compact_offsets": (_INT, [_P, _I32, _I32, _P]),
    "tb200_host_compact_sequence": (_INT, [_P, _P, _P, _P, _I32, _I32, _I32, _P, _I64, _P, _I32]),
    "tb200_host_compact_from_lists": (_INT, [_P, _P, _I32, _P, _P, _I32, _P, _P, _P, _I32, _I32, _P, _P, _I64, _P, _I32]),
    "tb200_host_compact_from_lists_strict": (_INT, [_P, _P, _I32, _P, _P, _I32, _P, _P, _P, _I32, _I32, _P, _P, _I64, _P, _I32]),
    "tb200_expand_sequence": (_INT, [_P, _P, _P, _P, _P, _P, _P, _I32, _I32, _I32, _I64, _P]),
    "tb200_fields_bag_mean_fwd": (_INT, [_P, _P, _P, _P, _I32, _I32, _I32, _P, _INT, _I64, _I32, _P, _INT, _P]),
    "tb200_fields_bag_mean_missing_fwd": (_INT, [_P, _P, _P, _P, _I32, _I32, _I32, _P, _INT, _I64, _I32, _P, _I32, _P, _P, _INT, _P]),
    "tb200_attn_fwd": (
        _INT,
        [_P, _P, _P, _P, _I32, _I32, _I32, _I32, _I32, _P, _P, _P, _P, _P, _I32, _I32, _I32, _F, _INT, _I32, _I64, _P, _P],
    ),
    "tb200_quant_act_1x128": (_INT, [_P, _P, _P, _I64, _I32, _P]),
    "tb200_fp8_gemm": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _P, _P]),
    "tb200_packed_token_index": (_INT, [_P, _P, _P, _P, _P, _P, _P, _P, _I32, _P, _I64, _I32, _I32, _I64, _P, _P, _P, _P]),
    "tb200_gemm_bf16_grouped": (_INT, [_P, _P, _P, _P, _P, _I32, _I64, _I32, _I32, _I32, _P, _P]),
    "tb200_ffn_fp8_fwd_static": (
        _INT, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _I32, _P],
    ),
    "tb200_ffn_fp8_static_scratch_bytes": (_I64, []),
    "tb200_ffn_fp8_static_status": (_INT, [_P, _P]),
    "tb200_sequence_prepare": (_INT, [_P, _P, _P, _P, _I64, _I32, _I32, _P, _P, _P, _P]),
    "tb200_scatter_rows": (_INT, [_P, _I64, _I64, _I32, _P, _P, _I64, _I32, _P, _I64, _P, _I64, _INT, _P]),
    "tb200_gather_rows": (_INT, [_P, _I64, _I32, _P, _INT, _I64, _I64, _I64, _P, _I64, _I32, _INT, _P]),
}

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None


def library_available() -> bool:
    """True if the shared library file exists (says nothing about the device)."""
    return LIB_PATH.exists()


def load() -> ctypes.CDLL:
    """Load the library once (double-checked under a lock) and bind every signature."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"cuda backend requested but {LIB_PATH.name} is not built; run `python -m taac_2026_b200.build`"
            )
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
        return lib


def strerror(code: int) -> str:
    return load().tb200_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    """Raise for a non-zero status: ValueError for rejected arguments, RuntimeError otherwise."""
    if code == 0:
        return
    message = f"{what}: {strerror(code)} (status {code})"
    if code in (-3, -8):
        raise ValueError(message)
    if code == -9:
        raise OverflowError(message)
    raise RuntimeError(message)


def launch_count() -> int:
    return int(load().tb200_launch_count())
