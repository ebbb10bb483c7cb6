"""Operator-level restatements of the reference's torch backend (CPU, fp32 / int64).

Floating-point operators take and return torch CPU tensors and compute in fp32 (fp64 where
noted); integer operators are numpy with explicit per-row loops, written from the operators'
definitions rather than from the reference's sort-based tensor code, so that agreement with
the golden vectors is a real check.
"""

from __future__ import annotations

import math

import numpy as np
import torch

# ---------------------------------------------------------------------------------------------
# normalisation
# ---------------------------------------------------------------------------------------------


def rms_norm_input_dtype(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """`_torch_rms_norm` exactly as written — every step in the INPUT dtype
    (src/taac2026/infrastructure/accelerators/normalization/rms_norm.py:71-73)."""
    scale = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * scale * weight


def rms_norm_fp32(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Same formula with fp32 arithmetic and one final rounding to the input dtype: what the
    reference's accelerated kernels compute
    (normalization/kernels/triton.py:31-50) and the value parity is measured against."""
    xf = x.float()
    scale = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * scale * weight.float()).to(x.dtype)


def layer_norm_fp32(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    """Closed form of `F.layer_norm` over the last dim with two-pass centred variance in fp32
    (`_torch_layer_norm`, normalization/layer_norm.py:65-66; kernel form
    normalization/kernels/triton.py:225-247)."""
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    centred = xf - mean
    var = centred.pow(2).mean(dim=-1, keepdim=True)
    return (centred * torch.rsqrt(var + eps) * weight.float() + bias.float()).to(x.dtype)


# ---------------------------------------------------------------------------------------------
# embedding gather / bag mean / id hashing
# ---------------------------------------------------------------------------------------------


def embedding_bag_mean(weight: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    """`F.embedding_bag(values, weight, mode="mean", padding_idx=0)`
    (accelerators/embedding/embedding_bag.py:82-83): fp32 sum over the non-padding ids of a
    bag in hot order, one division by their count, zeros for an empty bag.  Ids outside
    (0, rows) are skipped like the accelerated kernels do
    (embedding/kernels/cuembed_embedding_bag_mean.cu:30-44)."""
    w = weight.float().numpy()
    ids = values.numpy().astype(np.int64)
    batch, bag = ids.shape
    out = np.zeros((batch, w.shape[1]), dtype=np.float32)
    for b in range(batch):
        acc = np.zeros(w.shape[1], dtype=np.float32)
        count = 0
        for h in range(bag):
            i = int(ids[b, h])
            if 0 < i < w.shape[0]:
                acc = (acc + w[i]).astype(np.float32)
                count += 1
        if count:
            out[b] = (acc / np.float32(count)).astype(np.float32)
    return torch.from_numpy(out).to(weight.dtype)


def feature_bank(tables: list[torch.Tensor | None], specs: list[tuple[int, int, int]], int_feats: torch.Tensor,
                 compressed: list[bool] | None = None) -> torch.Tensor:
    """`FeatureEmbeddingBank.forward` (src/taac2026/infrastructure/modeling/embeddings.py:137-173):
    per field clamp the raw ids to [0, vocab], bag-mean them, stack to [B, F, emb].  Fields
    without a table give zeros; `compressed[f]` fields hash their ids first (:162-169)."""
    batch = int_feats.shape[0]
    emb = next(t.shape[1] for t in tables if t is not None)
    dtype = next(t.dtype for t in tables if t is not None)
    tokens = []
    for f, (vocab, offset, length) in enumerate(specs):
        table = tables[f]
        if table is None:
            tokens.append(torch.zeros(batch, emb, dtype=dtype))
            continue
        values = int_feats[:, offset : offset + length].to(torch.int64)
        if compressed is not None and compressed[f]:
            values = torch.from_numpy(hash_compress_ids(values.clamp(min=0).numpy(), table.shape[0] - 1))
        else:
            values = values.clamp(min=0, max=int(vocab))
        tokens.append(embedding_bag_mean(table, values))
    return torch.stack(tokens, dim=1)


def gather_rows(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """`nn.Embedding` lookup after the tokenizer's clamp
    (src/taac2026/infrastructure/modeling/tokenizers.py:168-170): a row copy."""
    idx = ids.to(torch.int64).clamp(min=0, max=weight.shape[0] - 1)
    return weight[idx]


def hash_compress_ids(values: np.ndarray, num_buckets: int) -> np.ndarray:
    """`hash_compress_ids` (src/taac2026/infrastructure/modeling/embeddings.py:74-79):
    positive ids map to ((v - 1) mod buckets) + 1, everything else to 0."""
    values = np.asarray(values, dtype=np.int64)
    if num_buckets <= 0:
        return np.zeros_like(values)
    out = np.zeros_like(values)
    flat_in = values.reshape(-1)
    flat_out = out.reshape(-1)
    for i, v in enumerate(flat_in):
        if v > 0:
            flat_out[i] = (int(v) - 1) % int(num_buckets) + 1
    return out


# ---------------------------------------------------------------------------------------------
# integer sequence preprocessing
# ---------------------------------------------------------------------------------------------

BUCKET_BOUNDARIES = np.array(
    [5, 10, 15, 20, 25, 30, 35, 40, 45, 50, 55, 60]
    + [120 + 60 * i for i in range(9)]  # 120 .. 600
    + [900 + 300 * i for i in range(10)]  # 900 .. 3600
    + [5400 + 1800 * i for i in range(10)]  # 5400 .. 21600
    + [32400 + 10800 * i for i in range(6)]  # 32400 .. 86400
    + [172800 + 86400 * i for i in range(6)]  # 2 .. 7 days
    + [1123200, 1641600, 2160000, 2592000, 4320000, 6048000, 7776000, 11664000, 15552000, 31536000],
    dtype=np.int64,
)
"""Gap-time bucket edges in seconds (src/taac2026/infrastructure/modeling/time_features.py:16-28)."""


def sequence_time_buckets(seq_timestamps: np.ndarray, request_timestamps: np.ndarray) -> np.ndarray:
    """`compute_sequence_time_buckets` (modeling/time_features.py:31-46): bucket =
    min(#edges < gap, 62) + 1 with gap = max(request - event, 0); events with timestamp 0 -> 0."""
    ts = np.asarray(seq_timestamps, dtype=np.int64)
    req = np.asarray(request_timestamps, dtype=np.int64)
    out = np.zeros(ts.shape, dtype=np.int64)
    for b in range(ts.shape[0]):
        for l in range(ts.shape[1]):
            if ts[b, l] == 0:
                continue
            gap = max(int(req[b]) - int(ts[b, l]), 0)
            below = int(np.sum(BUCKET_BOUNDARIES < gap))  # searchsorted(side="left")
            out[b, l] = min(below, len(BUCKET_BOUNDARIES) - 1) + 1
    return out


def _active_events(values: np.ndarray, lengths: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    max_len = values.shape[2]
    raw = np.clip(np.asarray(lengths, dtype=np.int64), 0, max_len)
    active = (values > 0).any(axis=1) & (np.arange(max_len)[None, :] < raw[:, None])
    return raw, active


def deduplicate_sequence_events(values: np.ndarray, lengths: np.ndarray, timestamps: np.ndarray):
    """`deduplicate_sequence_events` (src/taac2026/infrastructure/modeling/sequence.py:141-198).

    An event is the tuple of all feature values at one position; it is active if it lies inside
    the row's length and any feature is positive.  Of several active events with the same tuple
    only the LAST survives; survivors keep their original order.  Rows whose survivor count
    equals the raw length, or whose raw length is <= 1, are returned untouched; changed rows
    are compacted to the front and zero-filled behind the new length."""
    values = np.asarray(values, dtype=np.int64)
    timestamps = np.asarray(timestamps, dtype=np.int64)
    lengths = np.asarray(lengths)
    batch, _n_feat, max_len = values.shape
    raw, active = _active_events(values, lengths)
    new_values = values.copy()
    new_ts = timestamps.copy()
    new_len = lengths.copy()
    for b in range(batch):
        last_pos: dict[tuple[int, ...], int] = {}
        for l in range(max_len):
            if active[b, l]:
                last_pos[tuple(int(v) for v in values[b, :, l])] = l
        keep = sorted(last_pos.values())
        if len(keep) == raw[b] or raw[b] <= 1:
            continue
        new_values[b] = 0
        new_ts[b] = 0
        for rank, l in enumerate(keep):
            new_values[b, :, rank] = values[b, :, l]
            new_ts[b, rank] = timestamps[b, l]
        new_len[b] = len(keep)
    return new_values, new_len, new_ts


def sequence_stats(values: np.ndarray, lengths: np.ndarray, timestamps: np.ndarray,
                   request_timestamps: np.ndarray) -> np.ndarray:
    """`compute_sequence_stats` (src/taac2026/infrastructure/modeling/time_features.py:49-105):
    [length, active events, distinct active events, 1 - distinct/active, share of positive
    values inside the length, gap bucket of the last position]; all-zero for rows without an
    active event.  Every column is produced in fp32 like the reference (int64 -> fp32 casts,
    fp32 division)."""
    values = np.asarray(values, dtype=np.int64)
    batch, n_feat, max_len = values.shape
    stats = np.zeros((batch, 6), dtype=np.float32)
    if n_feat <= 0:
        return stats
    raw, active = _active_events(values, lengths)
    buckets = sequence_time_buckets(timestamps, request_timestamps)
    for b in range(batch):
        n_active = int(active[b].sum())
        if n_active == 0:
            continue
        distinct = {tuple(int(v) for v in values[b, :, l]) for l in range(max_len) if active[b, l]}
        positive = int((values[b] > 0).sum())
        denom = max(int(raw[b]) * n_feat, 1)
        stats[b, 0] = np.float32(raw[b])
        stats[b, 1] = np.float32(n_active)
        stats[b, 2] = np.float32(len(distinct))
        stats[b, 3] = np.float32(1.0) - np.float32(len(distinct)) / max(np.float32(n_active), np.float32(1.0))
        # torch divides int64 by int64 -> fp32 true division
        stats[b, 4] = (torch.tensor(positive) / torch.tensor(denom)).to(torch.float32).item()
        if raw[b] > 0:
            stats[b, 5] = np.float32(buckets[b, max(int(raw[b]) - 1, 0)])
    return stats


# ---------------------------------------------------------------------------------------------
# masks, pooling, positions
# ---------------------------------------------------------------------------------------------


def make_padding_mask(lengths: torch.Tensor, max_len: int) -> torch.Tensor:
    """True = padding (src/taac2026/infrastructure/modeling/sequence.py:32-34)."""
    return torch.arange(max_len).unsqueeze(0) >= lengths.unsqueeze(1)


def causal_valid_attention_mask(padding_mask: torch.Tensor) -> torch.Tensor:
    """[B, T, T] bool, True = attend (modeling/sequence.py:119-127): key valid and key <= query;
    a padded query attends to itself only."""
    batch, tokens = padding_mask.shape
    mask = torch.zeros(batch, tokens, tokens, dtype=torch.bool)
    for b in range(batch):
        for q in range(tokens):
            if padding_mask[b, q]:
                mask[b, q, q] = True
            else:
                mask[b, q, : q + 1] = ~padding_mask[b, : q + 1]
    return mask


def masked_mean(tokens: torch.Tensor, padding_mask: torch.Tensor) -> torch.Tensor:
    """Mean over non-padding positions, count clamped to >= 1 (modeling/sequence.py:54-60)."""
    if tokens.shape[1] == 0:
        return tokens.new_zeros(tokens.shape[0], tokens.shape[-1])
    valid = (~padding_mask).to(tokens.dtype).unsqueeze(-1)
    return (tokens * valid).sum(dim=1) / valid.sum(dim=1).clamp_min(1.0)


def sinusoidal_positions(length: int, dim: int) -> torch.Tensor:
    """sin on even, cos on odd channels, frequency exp(-ln(1e4) * 2i / dim), fp32
    (modeling/sequence.py:130-138)."""
    if length == 0:
        return torch.empty(0, dim)
    positions = torch.arange(length, dtype=torch.float32).unsqueeze(1)
    frequencies = torch.exp(torch.arange(0, dim, 2, dtype=torch.float32) * (-math.log(10000.0) / dim))
    values = torch.zeros(length, dim)
    values[:, 0::2] = torch.sin(positions * frequencies)
    values[:, 1::2] = torch.cos(positions * frequencies[: values[:, 1::2].shape[1]])
    return values


# ---------------------------------------------------------------------------------------------
# attention / FFN
# ---------------------------------------------------------------------------------------------


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None,
              scale: float | None = None) -> torch.Tensor:
    """softmax(q k^T * scale + mask) v in fp32 with an explicit max-subtracted softmax — the
    manual reference of the GPU tests (tests/gpu/infrastructure/accelerators/
    test_tilelang_ops_cuda.py:37-57) and the math of `F.scaled_dot_product_attention` as
    called at accelerators/attention/flash_attention.py:563-570.
    q, k, v: [B, H, L, D]; mask: bool broadcastable to [B, H, Lq, Lk], True = attend.
    Rows with no attended key return zeros (the accelerated kernel's rule,
    attention/kernels/tilelang.py:127-133)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    row_max = scores.max(dim=-1, keepdim=True).values
    row_max = torch.where(torch.isinf(row_max), torch.zeros_like(row_max), row_max)
    weights = torch.exp(scores - row_max)
    denom = weights.sum(dim=-1, keepdim=True)
    weights = torch.where(denom > 0, weights / denom.clamp_min(1e-30), torch.zeros_like(weights))
    return torch.matmul(weights, vf)


def structured_attention_mask(seq_lens: torch.Tensor, total: int, ns_start: int, causal: bool,
                              padded_query_self: bool) -> torch.Tensor:
    """[B, T, T] bool mask described by (seq_len[b], ns_start): key k is valid iff
    k < seq_len[b] or k >= ns_start; with `causal` also k <= q; with `padded_query_self`
    a query at an invalid position attends to itself only.  ns_start == total gives the
    plain prefix key-padding mask; this family contains both masks the reference's planner
    accepts (accelerators/attention/flash_attention.py:149-198) and OneTrans's
    [sequence | always-valid NS tokens] layout (experiments/onetrans/model.py:325-330)."""
    batch = seq_lens.shape[0]
    pos = torch.arange(total)
    key_valid = (pos[None, :] < seq_lens[:, None]) | (pos[None, :] >= ns_start)
    mask = key_valid[:, None, :].expand(batch, total, total).clone()
    if causal:
        mask &= (pos[None, :] <= pos[:, None])[None]
    if padded_query_self:
        invalid_q = ~key_valid
        eye = torch.eye(total, dtype=torch.bool)
        mask = torch.where(invalid_q[:, :, None], eye[None], mask)
    return mask


def swiglu_ffn(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, *, gate_first: bool = True,
               b_up: torch.Tensor | None = None, b_down: torch.Tensor | None = None) -> torch.Tensor:
    """down(silu(gate) * value) with [gate | value] = up(x) split in halves; gate is the first
    half (experiments/tokenformer/model.py:118-128, experiments/symbiosis/backbone.py:11-21) or
    the second (experiments/baseline/model.py:99-113).  fp32 math."""
    h = torch.nn.functional.linear(x.float(), w_up.float(), None if b_up is None else b_up.float())
    first, second = h.chunk(2, dim=-1)
    gate, value = (first, second) if gate_first else (second, first)
    hidden = torch.nn.functional.silu(gate) * value
    return torch.nn.functional.linear(hidden, w_down.float(), None if b_down is None else b_down.float())


def silu_ffn(x: torch.Tensor, w1: torch.Tensor, b1: torch.Tensor | None, w2: torch.Tensor,
             b2: torch.Tensor | None) -> torch.Tensor:
    """OneTrans's ungated FFN: Linear -> SiLU -> Linear (experiments/onetrans/model.py:33-44)."""
    h = torch.nn.functional.silu(torch.nn.functional.linear(x.float(), w1.float(), None if b1 is None else b1.float()))
    return torch.nn.functional.linear(h, w2.float(), None if b2 is None else b2.float())


def binary_auc(labels: np.ndarray, scores: np.ndarray) -> float:
    """Rank-sum AUC with tie-averaged ranks in float64 (src/taac2026/domain/metrics.py:30-59)."""
    labels = np.asarray(labels).astype(np.int64).reshape(-1)
    scores = np.asarray(scores, dtype=np.float64).reshape(-1)
    n_pos = int((labels == 1).sum())
    n_neg = int(labels.shape[0] - n_pos)
    if n_pos == 0 or n_neg == 0:
        return 0.5
    order = np.argsort(scores, kind="stable")
    sorted_scores = scores[order]
    ranks = np.empty(scores.shape[0], dtype=np.float64)
    i = 0
    while i < scores.shape[0]:
        j = i
        while j + 1 < scores.shape[0] and sorted_scores[j + 1] == sorted_scores[i]:
            j += 1
        ranks[order[i : j + 1]] = (i + j) / 2.0 + 1.0
        i = j + 1
    pos_rank_sum = ranks[labels == 1].sum()
    return float((pos_rank_sum - n_pos * (n_pos + 1) / 2.0) / (n_pos * n_neg))


# ---------------------------------------------------------------------------------------------
# FP8 (e4m3) block-scaled FFN emulation — PARITY UNPINNED BY THE REFERENCE
# ---------------------------------------------------------------------------------------------
# The reference has no FP8 code and no FP8 test.  The contract is the task's own: quantise bf16
# activations per 1 x 128 block and weights per 128 x 128 block (scale = amax / 448), compute the
# SiLU-gated FFN, and stay within 5e-2 relative of the bf16 torch FFN (`swiglu_ffn` above).  The
# functions below additionally emulate the quantised arithmetic itself on the CPU (e4m3 values are
# exact in fp32, so the only differences left are fp32 summation order and exp rounding), which lets
# the tests hold the kernel to a much tighter bound than the contract.

E4M3_MAX = 448.0


def quantize_blocks(x: torch.Tensor, block_rows: int, block_cols: int) -> tuple[torch.Tensor, torch.Tensor]:
    """-> (dequantised-grid values q as fp32 with x ~= q * scale, scales [R / br, C / bc])."""
    rows, cols = x.shape
    blocks = x.float().view(rows // block_rows, block_rows, cols // block_cols, block_cols)
    amax = blocks.abs().amax(dim=(1, 3))
    scales = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blocks / scales[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()
    return q.view(rows, cols), scales


def quantize_blocks_reciprocal(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """1 x 128 activation quantisation exactly as the kernels do it: q = rn_e4m3(x * (1 / scale))."""
    rows, cols = x.shape
    blocks = x.float().view(rows, cols // 128, 128)
    amax = blocks.abs().amax(dim=2)
    scales = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    inv = 1.0 / scales
    q = (blocks * inv[:, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()
    return q.view(rows, cols), scales


def block_scaled_matmul(qa: torch.Tensor, sa: torch.Tensor, qb: torch.Tensor, sb: torch.Tensor) -> torch.Tensor:
    """sum over K blocks of (qa_blk @ qb_blk^T) * sa[m, kb] * sb[n / 128, kb], fp32."""
    m, k = qa.shape
    n = qb.shape[0]
    out = torch.zeros(m, n)
    for kb in range(k // 128):
        part = qa[:, kb * 128 : (kb + 1) * 128] @ qb[:, kb * 128 : (kb + 1) * 128].t()
        out += part * sa[:, kb : kb + 1] * sb[:, kb].repeat_interleave(128)[None, :]
    return out


def fp8_ffn_emulated(x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, *, gated: bool, gate_first: bool = True,
                     b_up: torch.Tensor | None = None, b_down: torch.Tensor | None = None,
                     residual: torch.Tensor | None = None, quantized_weights=None) -> torch.Tensor:
    """The quantised FFN step by step: x (bf16) -> e4m3, GEMM 1, (gated) SiLU, e4m3 again, GEMM 2, bf16.
    `quantized_weights = ((q_up, s_up), (q_down, s_down))` (fp32 grid values, in w_up / w_down row order)
    replaces the weight quantisation done here, so that a caller can feed the very same weight codes to
    the emulation and to the kernel."""
    qx, sx = quantize_blocks_reciprocal(x.float())
    if quantized_weights is None:
        qw1, sw1 = quantize_blocks(w_up, 128, 128)
        qw2, sw2 = quantize_blocks(w_down, 128, 128)
    else:
        (qw1, sw1), (qw2, sw2) = quantized_weights
    h = block_scaled_matmul(qx, sx, qw1, sw1)
    if b_up is not None:
        h = h + b_up.float()
    if gated:
        first, second = h.chunk(2, dim=-1)
        gate, value = (first, second) if gate_first else (second, first)
        h = torch.nn.functional.silu(gate) * value
    else:
        h = torch.nn.functional.silu(h)
    qh, sh = quantize_blocks_reciprocal(h)
    y = block_scaled_matmul(qh, sh, qw2, sw2)
    if b_down is not None:
        y = y + b_down.float()
    if residual is not None:
        y = y + residual.float()
    return y.to(torch.bfloat16)
