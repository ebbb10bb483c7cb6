"""Model-facing input records and seeded synthetic batches.

The three dataclasses carry the same fields, dtypes and shapes as the reference's
``PCVRSequenceInput`` / ``PCVREntityInput`` / ``PCVRModelInput``
(src/taac2026/infrastructure/data/batches.py:17-69), so either family can be handed to the
models here (attribute access only).  ``synthetic_batch`` draws the seeded Zipf / normal
inputs that stand in for the competition's parquet data.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True, slots=True)
class SequenceInput:
    values: torch.Tensor  # [B, F, L] int64
    lengths: torch.Tensor  # [B] int64
    timestamps: torch.Tensor  # [B, L] int64

    def to(self, device, *, non_blocking: bool = False) -> "SequenceInput":
        return SequenceInput(
            self.values.to(device, non_blocking=non_blocking),
            self.lengths.to(device, non_blocking=non_blocking),
            self.timestamps.to(device, non_blocking=non_blocking),
        )

    def pin_memory(self) -> "SequenceInput":
        return SequenceInput(self.values.pin_memory(), self.lengths.pin_memory(), self.timestamps.pin_memory())


@dataclass(frozen=True, slots=True)
class EntityInput:
    int_values: torch.Tensor  # [B, D] int64
    int_missing_mask: torch.Tensor  # [B, D] bool
    dense_values: torch.Tensor  # [B, Dd] float32
    dense_missing_mask: torch.Tensor  # [B, Dd] bool

    def to(self, device, *, non_blocking: bool = False) -> "EntityInput":
        return EntityInput(
            self.int_values.to(device, non_blocking=non_blocking),
            self.int_missing_mask.to(device, non_blocking=non_blocking),
            self.dense_values.to(device, non_blocking=non_blocking),
            self.dense_missing_mask.to(device, non_blocking=non_blocking),
        )

    def pin_memory(self) -> "EntityInput":
        return EntityInput(
            self.int_values.pin_memory(), self.int_missing_mask.pin_memory(), self.dense_values.pin_memory(),
            self.dense_missing_mask.pin_memory(),
        )


@dataclass(frozen=True, slots=True)
class ModelInput:
    user: EntityInput
    item: EntityInput
    sequences: dict[str, SequenceInput]
    request_timestamp: torch.Tensor  # [B] int64

    def to(self, device, *, non_blocking: bool = False) -> "ModelInput":
        return ModelInput(
            self.user.to(device, non_blocking=non_blocking),
            self.item.to(device, non_blocking=non_blocking),
            {name: seq.to(device, non_blocking=non_blocking) for name, seq in self.sequences.items()},
            self.request_timestamp.to(device, non_blocking=non_blocking),
        )

    def pin_memory(self) -> "ModelInput":
        return ModelInput(
            self.user.pin_memory(), self.item.pin_memory(),
            {name: seq.pin_memory() for name, seq in self.sequences.items()}, self.request_timestamp.pin_memory(),
        )

    @property
    def batch_size(self) -> int:
        return int(self.user.int_values.shape[0])

    def tensors(self) -> list[torch.Tensor]:
        """Every tensor of the record (for stream bookkeeping such as ``Tensor.record_stream``)."""
        out = []
        for entity in (self.user, self.item):
            out += [entity.int_values, entity.int_missing_mask, entity.dense_values, entity.dense_missing_mask]
        for seq in self.sequences.values():
            out += [seq.values, seq.lengths, seq.timestamps]
        out.append(self.request_timestamp)
        return out

    def nbytes(self) -> int:
        total = 0
        for entity in (self.user, self.item):
            for t in (entity.int_values, entity.int_missing_mask, entity.dense_values, entity.dense_missing_mask):
                total += t.numel() * t.element_size()
        for seq in self.sequences.values():
            for t in (seq.values, seq.lengths, seq.timestamps):
                total += t.numel() * t.element_size()
        return total + self.request_timestamp.numel() * self.request_timestamp.element_size()

    def slice(self, start: int, stop: int) -> "ModelInput":
        cut = lambda t: t[start:stop]  # noqa: E731
        ent = lambda e: EntityInput(cut(e.int_values), cut(e.int_missing_mask), cut(e.dense_values), cut(e.dense_missing_mask))  # noqa: E731
        return ModelInput(
            ent(self.user), ent(self.item),
            {n: SequenceInput(cut(s.values), cut(s.lengths), cut(s.timestamps)) for n, s in self.sequences.items()},
            cut(self.request_timestamp),
        )


@dataclass(frozen=True, slots=True)
class CompactSequence:
    """One domain in the compact 32-bit host format (``ops.compact_sequence_host``): the valid prefix of every
    sample back to back instead of the reference's padded int64 buffers (batch_converter.py:446-488)."""

    cu: torch.Tensor  # [B + 1] int32
    ids: torch.Tensor  # [F, total] int32
    gaps: torch.Tensor | None  # [total] int32: request timestamp - event timestamp, INT32_MIN = no timestamp
    max_len: int  # L of the padded layout

    def to(self, device, *, non_blocking: bool = False) -> "CompactSequence":
        if self.ids.is_contiguous():
            ids = self.ids.to(device, non_blocking=non_blocking)
        else:           # rows of a larger host buffer: one copy per feature row, no staging copy on the host
            ids = torch.empty(self.ids.shape, dtype=self.ids.dtype, device=device)
            for f in range(self.ids.shape[0]):
                ids[f].copy_(self.ids[f], non_blocking=non_blocking)
        return CompactSequence(self.cu.to(device, non_blocking=non_blocking), ids,
                               None if self.gaps is None else self.gaps.to(device, non_blocking=non_blocking), self.max_len)

    def pin_memory(self) -> "CompactSequence":
        return CompactSequence(self.cu.pin_memory(), self.ids.contiguous().pin_memory(),
                               None if self.gaps is None else self.gaps.pin_memory(), self.max_len)

    def tensors(self) -> list[torch.Tensor]:
        return [t for t in (self.cu, self.ids, self.gaps) if t is not None]


@dataclass(frozen=True, slots=True)
class CompactModelInput:
    """A ``ModelInput`` whose sequences travel in the compact format.  ``to(device)`` copies it (about a third of
    the bytes of the padded record at the benchmark's lengths) and ``expand()`` rebuilds the padded ``ModelInput`` on
    the device, bit for bit, so everything behind it is unchanged."""

    user: EntityInput
    item: EntityInput
    sequences: dict[str, CompactSequence]
    request_timestamp: torch.Tensor  # [B] int64

    def to(self, device, *, non_blocking: bool = False) -> "CompactModelInput":
        return CompactModelInput(
            self.user.to(device, non_blocking=non_blocking), self.item.to(device, non_blocking=non_blocking),
            {name: seq.to(device, non_blocking=non_blocking) for name, seq in self.sequences.items()},
            self.request_timestamp.to(device, non_blocking=non_blocking),
        )

    def pin_memory(self) -> "CompactModelInput":
        return CompactModelInput(self.user.pin_memory(), self.item.pin_memory(),
                                 {name: seq.pin_memory() for name, seq in self.sequences.items()},
                                 self.request_timestamp.pin_memory())

    @property
    def batch_size(self) -> int:
        return int(self.user.int_values.shape[0])

    def tensors(self) -> list[torch.Tensor]:
        out = []
        for entity in (self.user, self.item):
            out += [entity.int_values, entity.int_missing_mask, entity.dense_values, entity.dense_missing_mask]
        for seq in self.sequences.values():
            out += seq.tensors()
        out.append(self.request_timestamp)
        return out

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors())

    def expand(self) -> ModelInput:
        """The padded record, rebuilt by ``ops.expand_sequence`` on the device the tensors live on."""
        from taac_2026_b200 import ops

        sequences = {}
        for name, seq in self.sequences.items():
            values, lengths, timestamps = ops.expand_sequence(seq.cu, seq.ids, seq.gaps, self.request_timestamp, seq.max_len)
            sequences[name] = SequenceInput(values, lengths, timestamps)
        return ModelInput(self.user, self.item, sequences, self.request_timestamp)


def compact_model_input(batch: ModelInput, *, threads: int = 4, pin: bool = False) -> CompactModelInput:
    """Host ``ModelInput`` -> ``CompactModelInput`` (native host code, ``threads`` workers).  Raises ``OverflowError``
    when an id or a timestamp gap needs more than 32 bits; such a batch is copied in its padded form instead.  An
    all-zero timestamp buffer (a domain without timestamps) is not carried at all."""
    from taac_2026_b200 import ops

    sequences = {}
    for name, seq in batch.sequences.items():
        timed = bool(seq.timestamps.any())
        cu, ids, gaps = ops.compact_sequence_host(seq.values, seq.lengths, seq.timestamps if timed else None,
                                                  batch.request_timestamp if timed else None, threads=threads, pin=pin)
        sequences[name] = CompactSequence(cu, ids, gaps, int(seq.values.shape[2]))
    return CompactModelInput(batch.user, batch.item, sequences, batch.request_timestamp)


@dataclass(frozen=True)
class OneTransSpec:
    """Everything ``PCVROneTrans._init_specs`` receives that shapes the forward
    (experiments/onetrans/model.py:148-238), as plain data."""

    user_int_specs: list[tuple[int, int, int]]  # (vocab, offset, length) per user field
    item_int_specs: list[tuple[int, int, int]]
    user_dense_dim: int
    item_dense_dim: int
    seq_vocab_sizes: dict[str, list[int]]
    d_model: int = 64
    emb_dim: int = 64
    num_blocks: int = 2
    num_heads: int = 4
    hidden_mult: int = 4
    seq_top_k: int = 50
    emb_skip_threshold: int = 0
    num_time_buckets: int = 0
    user_ns_tokens: int = 5
    item_ns_tokens: int = 2
    force_auto_split: bool = True
    action_num: int = 1
    user_ns_groups: list[list[int]] = field(default_factory=list)
    item_ns_groups: list[list[int]] = field(default_factory=list)

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name in self.__dataclass_fields__}


def zipf_ids(n: int, vocab: int, exponent: float, generator: torch.Generator) -> torch.Tensor:
    """n ids in [1, vocab] with P(id = r) proportional to r^-exponent (id 0 stays the padding id).
    Inverse-CDF sampling in float64 from seeded uniforms."""
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64)
    cdf = torch.cumsum(ranks.pow(-exponent), dim=0)
    cdf /= cdf[-1].clone()
    u = torch.rand(n, dtype=torch.float64, generator=generator)
    return (torch.searchsorted(cdf, u).clamp_(max=vocab - 1) + 1).to(torch.int64)


def synthetic_batch(
    spec: OneTransSpec,
    batch: int,
    *,
    seq_len: int,
    min_len: int,
    max_len: int | None = None,
    seed: int = 0,
    field_exponent: float = 1.2,
    seq_exponent: float = 1.1,
) -> ModelInput:
    """Seeded CPU batch: Zipf ids per sparse field (one id per unit of field length), N(0,1) dense
    features, one behaviour sequence per domain with lengths uniform in [min_len, max_len],
    right-padded with id 0 to ``seq_len``; timestamps are all zero and the request time constant."""
    g = torch.Generator().manual_seed(seed)
    max_len = seq_len if max_len is None else max_len

    def entity(specs: list[tuple[int, int, int]], dense_dim: int) -> EntityInput:
        cols = max((off + ln for _v, off, ln in specs), default=0)
        ints = torch.zeros(batch, cols, dtype=torch.int64)
        for vocab, off, ln in specs:
            if vocab > 0:
                ints[:, off : off + ln] = zipf_ids(batch * ln, vocab, field_exponent, g).view(batch, ln)
        dense = torch.randn(batch, dense_dim, generator=g)
        return EntityInput(ints, torch.zeros(batch, cols, dtype=torch.bool), dense, torch.zeros(batch, dense_dim, dtype=torch.bool))

    user = entity(spec.user_int_specs, spec.user_dense_dim)
    item = entity(spec.item_int_specs, spec.item_dense_dim)
    sequences: dict[str, SequenceInput] = {}
    for domain in sorted(spec.seq_vocab_sizes):
        vocabs = spec.seq_vocab_sizes[domain]
        lengths = torch.randint(min_len, max_len + 1, (batch,), generator=g, dtype=torch.int64)
        values = torch.zeros(batch, len(vocabs), seq_len, dtype=torch.int64)
        valid = torch.arange(seq_len).unsqueeze(0) < lengths.unsqueeze(1)
        for f, vocab in enumerate(vocabs):
            if vocab > 0:
                ids = zipf_ids(batch * seq_len, vocab, seq_exponent, g).view(batch, seq_len)
                values[:, f, :] = torch.where(valid, ids, torch.zeros_like(ids))
        sequences[domain] = SequenceInput(values, lengths, torch.zeros(batch, seq_len, dtype=torch.int64))
    return ModelInput(user, item, sequences, torch.full((batch,), 1_700_000_000, dtype=torch.int64))


__all__ = ["EntityInput", "ModelInput", "OneTransSpec", "SequenceInput", "synthetic_batch", "zipf_ids"]
