"""Arrow record batches -> model input in the compact host format.

``CompactRecordBatchConverter`` takes the reference's own schema layout and column plan objects
(``load_pcvr_schema_layout`` / ``build_pcvr_column_plan``, attribute access only) and does the job of
`PCVRRecordBatchConverter.convert` (src/taac2026/infrastructure/data/batch_converter.py:296-348) with one
difference: the behaviour sequences never exist as padded int64 buffers.  Their Arrow list columns (offsets +
values) go straight into the compact 32-bit record through the library's native packers
(``tb200_host_compact_from_lists`` / ``..._strict``), which apply the converter's prefix, ``<= 0 -> 0``,
clip-vocabulary and strict-time-filter rules; ``CompactModelInput.expand()`` rebuilds the padded tensors on the
device.  The entity features (a few dozen columns per sample) are filled with numpy under the same rules as the
reference (`_fill_int_features`, `_fill_dense_group`, :383-446).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np
import torch

from taac_2026_b200 import ops
from taac_2026_b200.inputs import CompactModelInput, CompactSequence, EntityInput


@dataclass(frozen=True, slots=True)
class CompactBatch:
    """What the loader hands to the prediction loop: the reference's ``PCVRBatch`` with compact inputs."""

    inputs: CompactModelInput
    label: torch.Tensor
    user_id: list


def _list_parts(column) -> tuple[np.ndarray, np.ndarray]:
    """Offsets and flat values of an Arrow list column (chunked arrays are combined first)."""
    if hasattr(column, "combine_chunks"):
        column = column.combine_chunks()
    return column.offsets.to_numpy(), column.values.to_numpy(zero_copy_only=False)


def _padded_prefix(offsets: np.ndarray, values: np.ndarray, rows: int, width: int, dtype) -> tuple[np.ndarray, np.ndarray]:
    """First ``width`` values of every row, zero filled (the rule of `pad_list_offsets_values`, :68-103), vectorised."""
    out = np.zeros((rows, width), dtype=dtype)
    if rows <= 0 or width <= 0:
        return out, np.zeros(max(rows, 0), dtype=np.int64)
    starts = offsets[:rows].astype(np.int64)
    lengths = np.clip(offsets[1:rows + 1].astype(np.int64) - starts, 0, width)
    if values.shape[0] == 0 or int(lengths.sum()) == 0:
        return out, lengths
    col = np.arange(width, dtype=np.int64)[None, :]
    inside = col < lengths[:, None]
    source = np.minimum(starts[:, None] + col, values.shape[0] - 1)
    out[inside] = values[source[inside]].astype(dtype, copy=False)
    return out, lengths


class CompactRecordBatchConverter:
    def __init__(self, *, layout: Any, column_plan: Any, clip_vocab: bool = True, is_training: bool = False,
                 strict_time_filter: bool = False, threads: int = 4, pin: bool = False) -> None:
        self.layout, self.column_plan = layout, column_plan
        self.clip_vocab, self.is_training = bool(clip_vocab), bool(is_training)
        self.strict_time_filter = bool(strict_time_filter)
        self.threads, self.pin = int(threads), bool(pin)
        self.oob_stats: dict[tuple[str, int], dict[str, int]] = {}

    # ------------------------------------------------------------------ out-of-vocabulary rule (:612-650)
    def _out_of_vocabulary(self, group: str, column_index: int, values: np.ndarray, vocab: int) -> None:
        beyond = values >= vocab
        if not beyond.any():
            return
        self._count_oob(group, column_index, int(beyond.sum()), vocab)
        if not self.clip_vocab:
            raise ValueError(f"{group} col_idx={column_index}: {int(beyond.sum())} values out of range [0, {vocab}). "
                             "Use clip_vocab=True to clip or fix schema.json")
        values[beyond] = 0

    def _count_oob(self, group: str, column_index: int, count: int, vocab: int) -> None:
        if count:
            entry = self.oob_stats.setdefault((group, column_index), {"count": 0, "vocab": vocab})
            entry["count"] += count

    # ------------------------------------------------------------------ entity features
    def _int_features(self, batch, rows: int, plan, width: int, group: str) -> tuple[torch.Tensor, torch.Tensor]:
        values = np.zeros((rows, width), dtype=np.int64)
        missing = np.ones((rows, width), dtype=np.bool_)
        for feature in plan:
            column = batch.column(feature.column_index)
            lo, hi = feature.output_offset, feature.output_offset + feature.dim
            if feature.dim == 1:
                scalar = column.fill_null(0).to_numpy(zero_copy_only=False).astype(np.int64)
                absent = column.is_null().to_numpy(zero_copy_only=False).astype(np.bool_)
                scalar[scalar <= 0] = 0
                block = scalar[:, None]
            else:
                block, _ = _padded_prefix(*_list_parts(column), rows, feature.dim, np.int64)
                block[block <= 0] = 0
                absent = None
            if feature.vocab_size > 0:
                self._out_of_vocabulary(group, feature.column_index, block, feature.vocab_size)
            else:
                block[:] = 0
            values[:, lo:hi] = block
            missing[:, lo:hi] = block <= 0 if absent is None else (absent[:, None] | (block <= 0))
        return torch.from_numpy(values), torch.from_numpy(missing)

    def _dense_features(self, batch, rows: int, plan, width: int) -> tuple[torch.Tensor, torch.Tensor]:
        values = np.zeros((rows, width), dtype=np.float32)
        missing = np.ones((rows, width), dtype=np.bool_)
        for feature in plan:
            block, lengths = _padded_prefix(*_list_parts(batch.column(feature.column_index)), rows, feature.dim, np.float32)
            present = np.arange(feature.dim)[None, :] < lengths[:, None]
            finite = np.isfinite(block)
            block[~finite] = 0.0
            lo, hi = feature.output_offset, feature.output_offset + feature.dim
            values[:, lo:hi] = block
            missing[:, lo:hi] = ~(present & finite)
        return torch.from_numpy(values), torch.from_numpy(missing)

    # ------------------------------------------------------------------ sequences
    def _sequence(self, batch, rows: int, domain: str, request_ts: np.ndarray) -> CompactSequence:
        plan = self.column_plan.sequences[domain]
        n_slots = len(self.layout.sideinfo_fids[domain])
        empty = (np.zeros(rows + 1, dtype=np.int32), np.zeros(0, dtype=np.int64))
        columns: list = [empty] * n_slots
        vocab = [0] * n_slots
        index_of = {}
        for side in plan.side_columns:
            columns[side.slot] = _list_parts(batch.column(side.column_index))
            vocab[side.slot] = int(side.vocab_size)
            index_of[side.slot] = side.column_index
        # every column of one call shares the offset width
        wide = any(np.asarray(c[0]).dtype == np.int64 for c in columns)
        columns = [(np.asarray(c[0]).astype(np.int64 if wide else np.int32, copy=False), c[1]) for c in columns]
        ts = None
        if plan.timestamp_column_index is not None:
            ts = _list_parts(batch.column(plan.timestamp_column_index))
            ts = (np.asarray(ts[0]).astype(np.int64 if wide else np.int32, copy=False), ts[1])
        if n_slots == 0:
            lengths = torch.zeros(rows + 1, dtype=torch.int32)
            return CompactSequence(lengths, torch.zeros(0, 0, dtype=torch.int32), None, int(plan.max_len))
        cu, ids, gaps, oob = ops.compact_sequence_from_lists(
            columns, ts, request_ts, int(plan.max_len), vocab_sizes=vocab,
            strict_time_filter=self.strict_time_filter, threads=self.threads, pin=self.pin)
        for slot, count in enumerate(oob.tolist()):
            if count:
                self._count_oob(f"seq_{domain}", index_of.get(slot, -1), int(count), vocab[slot])
                if not self.clip_vocab:
                    raise ValueError(f"seq_{domain} col_idx={index_of.get(slot, -1)}: {count} values out of range "
                                     f"[0, {vocab[slot]}). Use clip_vocab=True to clip or fix schema.json")
        return CompactSequence(cu, ids, gaps if ts is not None else None, int(plan.max_len))

    # ------------------------------------------------------------------ the batch
    def convert(self, batch) -> CompactBatch:
        rows = batch.num_rows
        indices = self.column_plan.column_indices
        request_ts = batch.column(indices["timestamp"]).to_numpy(zero_copy_only=False).astype(np.int64)
        layout = self.layout
        user = EntityInput(*self._int_features(batch, rows, self.column_plan.user_int, layout.user_int_schema.total_dim, "user_int"),
                           *self._dense_features(batch, rows, self.column_plan.user_dense, layout.user_dense_schema.total_dim))
        item = EntityInput(*self._int_features(batch, rows, self.column_plan.item_int, layout.item_int_schema.total_dim, "item_int"),
                           *self._dense_features(batch, rows, self.column_plan.item_dense, layout.item_dense_schema.total_dim))
        sequences = {domain: self._sequence(batch, rows, domain, request_ts) for domain in layout.seq_domains}
        if self.is_training:
            kinds = batch.column(indices["label_type"]).fill_null(0).to_numpy(zero_copy_only=False).astype(np.int64)
            label = torch.from_numpy((kinds == 2).astype(np.int64))
        else:
            label = torch.zeros(rows, dtype=torch.int64)
        inputs = CompactModelInput(user, item, sequences, torch.from_numpy(request_ts))
        return CompactBatch(inputs, label, batch.column(indices["user_id"]).to_pylist())


__all__ = ["CompactBatch", "CompactRecordBatchConverter"]
