"""The inference prediction loop of the reference on the B200 engine.

``run_inference_prediction_loop(model, loader)`` mirrors `_run_inference_prediction_loop`
(src/taac2026/application/evaluation/workflow.py:246-293): it walks a loader whose batches carry ``.inputs`` (the
padded int64 ``PCVRModelInput`` record, or ``taac_2026_b200.inputs.ModelInput``) and ``.user_id``, and returns the same
dictionary — ``predictions`` (``str(user_id) -> probability``), ``processed_rows``, ``batch_count``,
``loop_elapsed_sec``.  What differs is the order of the work, not the result:

* the record is packed into the compact 32-bit host format by the library's native packer (a batch whose values do
  not fit 32 bits is copied padded instead) and pinned;
* ``score_stream`` copies, expands and plans batch i + 1 on a side stream while batch i is scored;
* the scores of batch i come back into pinned host memory asynchronously, and the per-row dictionary fill of batch i
  (the reference's Python loop over ``zip(user_ids, probabilities)``) runs on the host while the device scores
  batch i + 1, instead of between two forwards with the device idle.
"""

from __future__ import annotations

import time
from collections import deque
from typing import Any, Iterable

import torch

from taac_2026_b200.inputs import EntityInput, ModelInput, SequenceInput, compact_model_input
from taac_2026_b200.onetrans import OneTransInference, score_stream


def as_model_input(record: Any) -> ModelInput:
    """Any record with the attributes of the reference's ``PCVRModelInput`` (infrastructure/data/batches.py:17-69)
    as this package's ``ModelInput`` (same tensors, no copy)."""
    if isinstance(record, ModelInput):
        return record

    def entity(e) -> EntityInput:
        return EntityInput(e.int_values, e.int_missing_mask, e.dense_values, e.dense_missing_mask)

    sequences = {name: SequenceInput(s.values, s.lengths, s.timestamps) for name, s in record.sequences.items()}
    return ModelInput(entity(record.user), entity(record.item), sequences, record.request_timestamp)


def run_inference_prediction_loop(model: OneTransInference, loader: Iterable[Any], *, compact: bool = True,
                                  pack_threads: int = 4, micro_batch: int | None = None) -> dict[str, Any]:
    """Scores every batch of ``loader`` and returns ``{"predictions", "processed_rows", "batch_count",
    "loop_elapsed_sec"}`` like the reference's loop; a batch without ``user_id`` is keyed by row number within the
    batch, as there (workflow.py:265)."""
    started = time.perf_counter()
    predictions: dict[str, float] = {}
    user_ids: deque = deque()
    counts = {"rows": 0, "batches": 0}

    def host_batches():
        for batch in loader:
            record = as_model_input(batch.inputs if hasattr(batch, "inputs") else batch)
            user_ids.append(getattr(batch, "user_id", None))
            staged = None
            if compact:
                try:
                    staged = compact_model_input(record, threads=pack_threads, pin=True)
                    staged = type(staged)(staged.user.pin_memory(), staged.item.pin_memory(), staged.sequences,
                                          staged.request_timestamp.pin_memory())
                except OverflowError:          # an id or a timestamp gap beyond 32 bits: the padded record travels
                    staged = None
            yield staged if staged is not None else record.pin_memory()

    def fill(ids, host_scores: torch.Tensor, ready: torch.cuda.Event) -> None:
        ready.synchronize()
        values = host_scores.tolist()
        keys = ids or list(range(len(values)))
        for user_id, probability in zip(keys, values, strict=False):
            predictions[str(user_id)] = float(probability)
        counts["rows"] += len(values)

    pending = None          # (user ids, pinned scores, event) of the previous batch
    with torch.inference_mode():
        for scores in score_stream(model, host_batches(), micro_batch=micro_batch):
            flat = scores.reshape(scores.shape[0], -1)[:, 0] if scores.ndim > 1 else scores
            host_scores = torch.empty(flat.shape, dtype=torch.float32, pin_memory=True)
            host_scores.copy_(flat, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record()
            if pending is not None:
                fill(*pending)      # the previous batch's dictionary fill runs under this batch's kernels
            pending = (user_ids.popleft(), host_scores, ready)
            counts["batches"] += 1
    if pending is not None:
        fill(*pending)
    return {"predictions": predictions, "processed_rows": counts["rows"], "batch_count": counts["batches"],
            "loop_elapsed_sec": time.perf_counter() - started}


__all__ = ["as_model_input", "run_inference_prediction_loop"]
