"""Operator boundary of the ``cuda`` backend.

Each public function keeps the name, argument meaning, validation order, exception types
and messages of the reference operator it stands behind, so that a caller (or a test
written for the reference) can swap ``backend="tilelang"`` / ``"triton"`` for
``backend="cuda"``:

* ``rms_norm``            — src/taac2026/infrastructure/accelerators/normalization/rms_norm.py:377-401
* ``layer_norm``          — src/taac2026/infrastructure/accelerators/normalization/layer_norm.py:261-280
* ``embedding_bag_mean``  — src/taac2026/infrastructure/accelerators/embedding/embedding_bag.py:439-467
* ``flash_attention``     — src/taac2026/infrastructure/accelerators/attention/flash_attention.py:871-919

The functions marshal torch tensors into the C ABI of ``libtb200.so`` (device pointers,
sizes, the current CUDA stream) and return freshly allocated tensors.  Nothing here computes
on the CPU: CPU tensors, a missing library or a non-sm_100 device raise ``RuntimeError``.
"""

from __future__ import annotations

import ctypes
from typing import Literal

import torch

from taac_2026_b200 import _lib

CudaBackend = Literal["cuda"]

_DTYPE_CODES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_ID_CODES = {torch.int32: _lib.I32, torch.int64: _lib.I64}


# --------------------------------------------------------------------------------------------
# availability / validation (mirrors accelerators/tilelang_runtime.py, tensor_validation.py)
# --------------------------------------------------------------------------------------------
def cuda_available() -> bool:
    """True when the library is built, a CUDA device is visible and it is an sm_100 part."""
    if not _lib.library_available() or not torch.cuda.is_available():
        return False
    return bool(_lib.load().tb200_device_ok())


def cuda_supported_floating_dtype(dtype: torch.dtype) -> bool:
    return dtype in _DTYPE_CODES


def _require_cuda_tensors(operator_name: str, *tensors: torch.Tensor | None) -> torch.device | None:
    checked = [tensor for tensor in tensors if tensor is not None]
    if not checked:
        return None
    if len({tensor.device for tensor in checked}) != 1:
        raise RuntimeError(f"{operator_name} requires all tensors to live on the same device")
    if checked[0].device.type != "cuda":
        raise RuntimeError(f"{operator_name} requires CUDA tensors")
    return checked[0].device


def _require_backend(operator_name: str, backend: str) -> None:
    if backend != "cuda":
        raise ValueError(f"unsupported {operator_name} backend: {backend}")
    if not cuda_available():
        raise RuntimeError("cuda backend requested but libtb200 or an sm_100 CUDA device is not available")


def _stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


# --------------------------------------------------------------------------------------------
# RMSNorm / LayerNorm
# --------------------------------------------------------------------------------------------
def _normalize_rms_norm_inputs(x: torch.Tensor, weight: torch.Tensor):
    if x.ndim < 2:
        raise ValueError("rms_norm expects input with at least 2 dimensions")
    if weight.ndim != 1:
        raise ValueError("rms_norm weight must be a 1D tensor")
    if x.shape[-1] != weight.shape[0]:
        raise ValueError(f"last dimension {x.shape[-1]} does not match weight size {weight.shape[0]}")
    original_shape = x.shape
    matrix = x.reshape(-1, x.shape[-1]).contiguous()
    normalized_weight = weight.to(device=matrix.device, dtype=matrix.dtype).contiguous()
    return matrix, normalized_weight, original_shape


def resolved_rms_norm_backend(
    x: torch.Tensor, backend: str = "cuda", *, eps: float = 1e-6, block_rows: int | None = None
) -> str:
    del eps, block_rows
    _require_backend("rms_norm", backend)
    _require_cuda_tensors("cuda rms_norm", x)
    if not cuda_supported_floating_dtype(x.dtype):
        raise RuntimeError(f"cuda rms_norm does not support dtype {x.dtype}")
    return "cuda"


def rms_norm(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float = 1e-6,
    *,
    backend: str = "cuda",
    block_rows: int | None = None,
) -> torch.Tensor:
    """``x * rsqrt(mean(x^2, -1) + eps) * weight`` with fp32 accumulation, one fused kernel.

    ``block_rows`` is accepted for signature compatibility; the kernel sizes its own tiles.
    """
    matrix, normalized_weight, original_shape = _normalize_rms_norm_inputs(x, weight)
    resolved_rms_norm_backend(matrix, backend, eps=eps, block_rows=block_rows)
    out = torch.empty_like(matrix)
    with torch.cuda.device(matrix.device):
        code = _lib.load().tb200_rmsnorm_fwd(
            _ptr(matrix), _ptr(normalized_weight), _ptr(out), matrix.shape[0], matrix.shape[1], float(eps),
            _DTYPE_CODES[matrix.dtype], _stream_ptr(),
        )
    _lib.check(code, "cuda rms_norm")
    return out.reshape(original_shape)


def _normalize_layer_norm_inputs(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor):
    if x.ndim < 2:
        raise ValueError("layer_norm expects input with at least 2 dimensions")
    if weight.ndim != 1:
        raise ValueError("layer_norm weight must be a 1D tensor")
    if bias.ndim != 1:
        raise ValueError("layer_norm bias must be a 1D tensor")
    if x.shape[-1] != weight.shape[0]:
        raise ValueError(f"last dimension {x.shape[-1]} does not match weight size {weight.shape[0]}")
    if weight.shape != bias.shape:
        raise ValueError(
            f"layer_norm weight shape {tuple(weight.shape)} does not match bias shape {tuple(bias.shape)}"
        )
    original_shape = x.shape
    matrix = x.reshape(-1, x.shape[-1]).contiguous()
    normalized_weight = weight.to(device=matrix.device, dtype=matrix.dtype).contiguous()
    normalized_bias = bias.to(device=matrix.device, dtype=matrix.dtype).contiguous()
    return matrix, normalized_weight, normalized_bias, original_shape


def resolved_layer_norm_backend(
    x: torch.Tensor, backend: str = "cuda", *, eps: float = 1e-5, block_rows: int | None = None
) -> str:
    del eps, block_rows
    _require_backend("layer_norm", backend)
    _require_cuda_tensors("cuda layer_norm", x)
    if not cuda_supported_floating_dtype(x.dtype):
        raise RuntimeError(f"cuda layer_norm does not support dtype {x.dtype}")
    return "cuda"


def layer_norm(
    x: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    eps: float = 1e-5,
    *,
    backend: str = "cuda",
    block_rows: int | None = None,
) -> torch.Tensor:
    """``(x - mean) * rsqrt(var + eps) * weight + bias`` over the last dimension (fp32 statistics)."""
    matrix, normalized_weight, normalized_bias, original_shape = _normalize_layer_norm_inputs(x, weight, bias)
    resolved_layer_norm_backend(matrix, backend, eps=eps, block_rows=block_rows)
    out = torch.empty_like(matrix)
    with torch.cuda.device(matrix.device):
        code = _lib.load().tb200_layernorm_fwd(
            _ptr(matrix), _ptr(normalized_weight), _ptr(normalized_bias), _ptr(out), matrix.shape[0],
            matrix.shape[1], float(eps), _DTYPE_CODES[matrix.dtype], _stream_ptr(),
        )
    _lib.check(code, "cuda layer_norm")
    return out.reshape(original_shape)


# --------------------------------------------------------------------------------------------
# embedding gather / bag-mean
# --------------------------------------------------------------------------------------------
def _normalize_embedding_bag_mean_inputs(embedding_weight: torch.Tensor, values: torch.Tensor):
    if embedding_weight.ndim != 2:
        raise ValueError("embedding_bag_mean weight must be a 2D tensor")
    if values.ndim != 2:
        raise ValueError("embedding_bag_mean values must be a 2D tensor")
    if embedding_weight.device != values.device:
        raise RuntimeError("embedding_bag_mean requires all tensors to live on the same device")
    normalized_weight = embedding_weight.contiguous()
    normalized_values = values.to(device=normalized_weight.device).contiguous()
    return normalized_weight, normalized_values


def resolved_embedding_bag_mean_backend(
    embedding_weight: torch.Tensor,
    values: torch.Tensor,
    backend: str = "cuda",
    *,
    block_rows: int | None = None,
    block_cols: int | None = None,
) -> str:
    del block_rows, block_cols
    _require_backend("embedding_bag_mean", backend)
    _require_cuda_tensors("cuda embedding_bag_mean", embedding_weight)
    if not cuda_supported_floating_dtype(embedding_weight.dtype):
        raise RuntimeError(f"cuda embedding_bag_mean does not support dtype {embedding_weight.dtype}")
    if values.dtype not in _ID_CODES:
        raise RuntimeError(f"cuda embedding_bag_mean requires int32 or int64 values, got {values.dtype}")
    return "cuda"


def embedding_bag_mean(
    embedding_weight: torch.Tensor,
    values: torch.Tensor,
    *,
    backend: str = "cuda",
    block_rows: int | None = None,
    block_cols: int | None = None,
) -> torch.Tensor:
    """Fixed-hotness bag mean with padding id 0 (``F.embedding_bag(..., mode="mean", padding_idx=0)``)."""
    weight, ids = _normalize_embedding_bag_mean_inputs(embedding_weight, values)
    resolved_embedding_bag_mean_backend(weight, ids, backend, block_rows=block_rows, block_cols=block_cols)
    out = torch.empty((ids.shape[0], weight.shape[1]), dtype=weight.dtype, device=weight.device)
    with torch.cuda.device(weight.device):
        code = _lib.load().tb200_bag_mean_fwd(
            _ptr(weight), weight.shape[0], weight.shape[1], _ptr(ids), _ID_CODES[ids.dtype], ids.shape[0],
            ids.shape[1], _ptr(out), _DTYPE_CODES[weight.dtype], _stream_ptr(),
        )
    _lib.check(code, "cuda embedding_bag_mean")
    return out


class FieldTables:
    """Device-side description of the embedding tables of one entity's sparse fields.

    Built once per model from ``(vocab_size, offset, length)`` feature specs and the per-field
    tables (``FeatureEmbeddingBank.feature_specs`` / ``.embeddings`` in
    src/taac2026/infrastructure/modeling/embeddings.py:82-129); ``fields_bag_mean`` then pools
    every field of a batch in one launch.
    """

    def __init__(self, tables: list[torch.Tensor], offsets: list[int], lengths: list[int]) -> None:
        if not tables or not (len(tables) == len(offsets) == len(lengths)):
            raise ValueError("FieldTables needs one table, offset and length per field")
        first = tables[0]
        for table in tables:
            if table.ndim != 2 or table.shape[1] != first.shape[1]:
                raise ValueError("FieldTables tables must be 2D with one shared embedding dim")
            if table.dtype != first.dtype or table.device != first.device:
                raise ValueError("FieldTables tables must share dtype and device")
            if not table.is_contiguous():
                raise ValueError("FieldTables tables must be contiguous")
        _require_cuda_tensors("cuda fields_bag_mean", first)
        self.tables = list(tables)  # keeps the storage alive
        self.dim = int(first.shape[1])
        self.dtype = first.dtype
        self.device = first.device
        self.n_fields = len(tables)
        self.max_bag = max(int(length) for length in lengths)
        self.ptrs = torch.tensor([table.data_ptr() for table in tables], dtype=torch.int64, device=self.device)
        self.rows = torch.tensor([table.shape[0] for table in tables], dtype=torch.int64, device=self.device)
        self.offsets = torch.tensor(offsets, dtype=torch.int32, device=self.device)
        self.lengths = torch.tensor(lengths, dtype=torch.int32, device=self.device)


def fields_bag_mean(fields: FieldTables, int_feats: torch.Tensor) -> torch.Tensor:
    """``[B, ids_cols]`` raw ids -> ``[B, n_fields, dim]`` pooled embeddings, ids clamped per field."""
    if int_feats.ndim != 2:
        raise ValueError("fields_bag_mean ids must be a 2D tensor")
    _require_backend("fields_bag_mean", "cuda")
    _require_cuda_tensors("cuda fields_bag_mean", fields.tables[0], int_feats)
    if int_feats.dtype not in _ID_CODES:
        raise RuntimeError(f"cuda fields_bag_mean requires int32 or int64 values, got {int_feats.dtype}")
    ids = int_feats.contiguous()
    out = torch.empty((ids.shape[0], fields.n_fields, fields.dim), dtype=fields.dtype, device=fields.device)
    with torch.cuda.device(fields.device):
        code = _lib.load().tb200_fields_bag_mean_fwd(
            _ptr(fields.ptrs), _ptr(fields.rows), _ptr(fields.offsets), _ptr(fields.lengths), fields.n_fields,
            fields.max_bag, fields.dim, _ptr(ids), _ID_CODES[ids.dtype], ids.shape[0], ids.shape[1], _ptr(out),
            _DTYPE_CODES[fields.dtype], _stream_ptr(),
        )
    _lib.check(code, "cuda fields_bag_mean")
    return out


def sequence_gather(tables: list[torch.Tensor | None], sequence: torch.Tensor) -> torch.Tensor:
    """``[B, F, L]`` ids -> ``[B, L, F * dim]``: per-feature row gather written straight into the
    concatenated layout (the gather + ``torch.cat`` of ``SequenceTokenizer.forward``,
    src/taac2026/infrastructure/modeling/tokenizers.py:156-176).  ``tables[f] is None`` leaves
    that feature's slice zero, as the reference does for features without a table.
    """
    if sequence.ndim != 3:
        raise ValueError("sequence_gather ids must have shape (batch, features, length)")
    live = [table for table in tables if table is not None]
    if not live or len(tables) != sequence.shape[1]:
        raise ValueError("sequence_gather needs one table (or None) per feature and at least one table")
    _require_backend("sequence_gather", "cuda")
    _require_cuda_tensors("cuda sequence_gather", live[0], sequence)
    if sequence.dtype not in _ID_CODES:
        raise RuntimeError(f"cuda sequence_gather requires int32 or int64 values, got {sequence.dtype}")
    first = live[0]
    if not cuda_supported_floating_dtype(first.dtype):
        raise RuntimeError(f"cuda sequence_gather does not support dtype {first.dtype}")
    ids = sequence.contiguous()
    batch, n_feat, length = ids.shape
    dim = int(first.shape[1])
    if any(table is None for table in tables):
        out = torch.zeros((batch, length, n_feat * dim), dtype=first.dtype, device=first.device)
    else:
        out = torch.empty((batch, length, n_feat * dim), dtype=first.dtype, device=first.device)
    lib = _lib.load()
    item = ids.element_size()
    with torch.cuda.device(first.device):
        for f, table in enumerate(tables):
            if table is None:
                continue
            if table.shape[1] != dim or table.dtype != first.dtype or not table.is_contiguous():
                raise ValueError("sequence_gather tables must be contiguous and share dim and dtype")
            code = lib.tb200_gather_rows(
                _ptr(table), table.shape[0], dim, ctypes.c_void_p(ids.data_ptr() + f * length * item),
                _ID_CODES[ids.dtype], batch * length, length, n_feat * length, _ptr(out), n_feat * dim, f * dim,
                _DTYPE_CODES[first.dtype], _stream_ptr(),
            )
            _lib.check(code, "cuda sequence_gather")
    return out


def gather_rows(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """``table[clamp(ids)]`` for an id tensor of any shape (bit-exact ``nn.Embedding`` lookup)."""
    _require_backend("gather_rows", "cuda")
    _require_cuda_tensors("cuda gather_rows", table, ids)
    if ids.dtype not in _ID_CODES:
        raise RuntimeError(f"cuda gather_rows requires int32 or int64 values, got {ids.dtype}")
    if table.ndim != 2:
        raise ValueError("gather_rows table must be a 2D tensor")
    if not cuda_supported_floating_dtype(table.dtype):
        raise RuntimeError(f"cuda gather_rows does not support dtype {table.dtype}")
    weight = table.contiguous()
    flat = ids.contiguous().view(-1)
    out = torch.empty((flat.shape[0], weight.shape[1]), dtype=weight.dtype, device=weight.device)
    n = flat.shape[0]
    with torch.cuda.device(weight.device):
        code = _lib.load().tb200_gather_rows(
            _ptr(weight), weight.shape[0], weight.shape[1], _ptr(flat), _ID_CODES[flat.dtype], n, max(n, 1), 0,
            _ptr(out), weight.shape[1], 0, _DTYPE_CODES[weight.dtype], _stream_ptr(),
        )
    _lib.check(code, "cuda gather_rows")
    return out.view(*ids.shape, weight.shape[1])


__all__ = [
    "CudaBackend",
    "FieldTables",
    "cuda_available",
    "cuda_supported_floating_dtype",
    "embedding_bag_mean",
    "fields_bag_mean",
    "gather_rows",
    "layer_norm",
    "resolved_embedding_bag_mean_backend",
    "resolved_layer_norm_backend",
    "resolved_rms_norm_backend",
    "rms_norm",
    "sequence_gather",
]
