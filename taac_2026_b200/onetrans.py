"""Inference engine for the OneTrans-style PCVR model on the ``cuda`` backend.

``OneTransInference`` runs the forward of the reference's ``PCVROneTrans``
(experiments/onetrans/model.py:110-359) from a plain ``state_dict`` (same parameter names),
re-organised for a B200:

* all sparse fields of an entity are pooled by ONE gather kernel (``ops.fields_bag_mean``)
  instead of one ``F.embedding_bag`` launch per field (modeling/embeddings.py:137-173);
* sequence ids are gathered straight into the concatenated ``[B, L, F * emb]`` layout
  (``ops.sequence_gather``; modeling/tokenizers.py:156-176);
* RMSNorm / LayerNorm are the fused TMA-staged kernels (``ops.rms_norm`` / ``ops.layer_norm``);
* attention runs on strided views of the fused QKV projection with the mask described by
  per-sample lengths — the ``[B, H, T, T]`` bool mask of ``causal_valid_attention_mask``
  (modeling/sequence.py:119-127) is never built;
* the per-NS-token projections and FFNs (model.py:60-67, :89-93) are batched matmuls;
* duplicate-event removal and the sequence statistics share one stable sort
  (modeling/sequence.py:141-198, modeling/time_features.py:49-105).

Dense layers whose widths are whole tiles run on this library's tcgen05 GEMM with bias, SiLU and
residual in its epilogue (``ops.grouped_linear``); the fp32 score-parity mode and odd widths use
``torch.nn.functional.linear``.  Everything runs on the GPU; there is no CPU path.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from taac_2026_b200 import ops
from taac_2026_b200.inputs import OneTransSpec

# Gap-time bucket edges in seconds (the constant table of modeling/time_features.py:16-28).
_BUCKET_EDGES = (
    [5 * i for i in range(1, 13)]
    + [60 * i for i in range(2, 11)]
    + [300 * i for i in range(3, 13)]
    + [1800 * i for i in range(3, 13)]
    + [10800 * i for i in range(3, 9)]
    + [86400 * i for i in range(2, 8)]
    + [1123200, 1641600, 2160000, 2592000, 4320000, 6048000, 7776000, 11664000, 15552000, 31536000]
)


def _table_kind(vocab: int, threshold: int, compress: bool) -> str:
    """Which embedding table a feature owns (modeling/embeddings.py:99-127)."""
    if int(vocab) <= 0:
        return "none"
    if threshold > 0 and int(vocab) > threshold:
        return "compressed" if compress else "none"
    return "table"


def hash_compress_ids(values: torch.Tensor, num_buckets: int) -> torch.Tensor:
    """Positive ids -> ((v - 1) mod buckets) + 1, everything else -> 0 (modeling/embeddings.py:74-79)."""
    if num_buckets <= 0:
        return torch.zeros_like(values)
    hashed = torch.remainder(values.clamp_min(1) - 1, int(num_buckets)) + 1
    return torch.where(values > 0, hashed, torch.zeros_like(values))


def pyramid_keep_count(seq_tokens: int, layer: int, n_layers: int, num_ns: int) -> int:
    """Sequence positions kept after block ``layer`` (experiments/onetrans/model.py:317-323)."""
    if seq_tokens <= max(1, num_ns):
        return seq_tokens
    remaining = max(1, n_layers - layer)
    target = max(1, num_ns)
    decay = (target / seq_tokens) ** (1.0 / remaining)
    return max(target, min(seq_tokens, math.ceil(seq_tokens * decay)))


@dataclass
class _Bank:
    """Sparse fields of one entity, ready for the fused pooling kernel."""

    fields: ops.FieldTables | None
    n_fields: int
    hashed: list[tuple[int, int, int]]  # (offset, length, buckets) of hashed high-cardinality fields


class _SequenceSort:
    """One lexicographic stable sort of a domain's events, shared by duplicate removal and the
    statistics token.  An event is the tuple of all feature values at a position; it is active when
    it lies inside the row's length and any feature is positive."""

    def __init__(self, values: torch.Tensor, lengths: torch.Tensor) -> None:
        batch, n_feat, max_len = values.shape
        dev = values.device
        self.raw_len = lengths.clamp(min=0, max=max_len).to(torch.long)
        self.positions = torch.arange(max_len, device=dev)
        self.active = (values > 0).any(dim=1) & (self.positions[None, :] < self.raw_len[:, None])
        keys = torch.where(self.active[:, None, :], values, torch.full_like(values, -1))  # [B, F, L]
        order = self.positions.expand(batch, -1).contiguous()
        for f in range(n_feat - 1, -1, -1):  # least-significant feature first; every pass is stable
            order = order.gather(1, torch.sort(keys[:, f].gather(1, order), dim=1, stable=True).indices)
        sorted_keys = keys.gather(2, order[:, None, :].expand(-1, n_feat, -1))
        differs = (sorted_keys[:, :, 1:] != sorted_keys[:, :, :-1]).any(dim=1)  # [B, L-1]
        true_col = torch.ones(batch, 1, dtype=torch.bool, device=dev)
        sorted_active = self.active.gather(1, order)
        self.order = order
        self.group_last = torch.cat([differs, true_col], dim=1) & sorted_active
        self.group_first = torch.cat([true_col, differs], dim=1) & sorted_active


def deduplicate_sequence_events(values: torch.Tensor, lengths: torch.Tensor, timestamps: torch.Tensor,
                                sort: _SequenceSort | None = None):
    """Keep the LAST occurrence of every distinct active event, in original order; rows that lose
    nothing (or have raw length <= 1) are returned untouched, changed rows are compacted to the front
    and zero-filled (modeling/sequence.py:141-198).  Integer work: bit-exact."""
    batch, n_feat, max_len = values.shape
    sort = sort or _SequenceSort(values, lengths)
    keep = torch.zeros_like(sort.group_last).scatter_(1, sort.order, sort.group_last)
    keep_count = keep.sum(dim=1)
    changed = (keep_count != sort.raw_len) & (sort.raw_len > 1)
    # stable compaction: the j-th kept position of a row moves to slot j
    slot = torch.cumsum(keep.to(torch.long), dim=1) - 1
    src = torch.zeros(batch, max_len, dtype=torch.long, device=values.device)
    rows = torch.arange(batch, device=values.device)[:, None].expand(-1, max_len)
    src.index_put_((rows[keep], slot[keep]), sort.positions.expand(batch, -1)[keep])
    tail = (sort.positions[None, :] >= keep_count[:, None]) & changed[:, None]
    new_values = values.gather(2, src[:, None, :].expand(-1, n_feat, -1)).masked_fill(tail[:, None, :], 0)
    new_ts = timestamps.gather(1, src).masked_fill(tail, 0)
    return (
        torch.where(changed[:, None, None], new_values, values),
        torch.where(changed, keep_count.to(lengths.dtype), lengths),
        torch.where(changed[:, None], new_ts, timestamps),
    )


def sequence_time_buckets(timestamps: torch.Tensor, request_ts: torch.Tensor, edges: torch.Tensor) -> torch.Tensor:
    """Gap bucket of every event: min(#edges < gap, 62) + 1, 0 for zero timestamps
    (modeling/time_features.py:31-46)."""
    if timestamps.shape[1] == 0:
        return timestamps.new_zeros(timestamps.shape, dtype=torch.long)
    gap = (request_ts[:, None] - timestamps).clamp_min(0)
    bucket = torch.searchsorted(edges, gap).clamp_max(edges.numel() - 1) + 1
    return torch.where(timestamps == 0, torch.zeros_like(bucket), bucket)


def sequence_stats(values: torch.Tensor, lengths: torch.Tensor, timestamps: torch.Tensor, request_ts: torch.Tensor,
                   edges: torch.Tensor, sort: _SequenceSort | None = None) -> torch.Tensor:
    """[length, active, distinct, 1 - distinct / active, positive share, last gap bucket] in fp32,
    zero rows without active events (modeling/time_features.py:49-105)."""
    batch, n_feat, max_len = values.shape
    stats = torch.zeros(batch, 6, dtype=torch.float32, device=values.device)
    if n_feat <= 0:
        return stats
    sort = sort or _SequenceSort(values, lengths)
    active = sort.active.sum(dim=1)
    distinct = sort.group_first.sum(dim=1)
    has = active > 0
    positive = (values > 0).sum(dim=(1, 2))
    share = positive / torch.maximum(sort.raw_len * n_feat, torch.ones_like(sort.raw_len))
    buckets = sequence_time_buckets(timestamps, request_ts, edges)
    last_bucket = buckets[torch.arange(batch, device=values.device), (sort.raw_len - 1).clamp_min(0)]
    zero = torch.zeros(batch, dtype=torch.float32, device=values.device)
    active_f = active.to(torch.float32)
    stats[:, 0] = torch.where(has, sort.raw_len.to(torch.float32), zero)
    stats[:, 1] = torch.where(has, active_f, zero)
    stats[:, 2] = torch.where(has, distinct.to(torch.float32), zero)
    stats[:, 3] = torch.where(has, 1.0 - distinct.to(torch.float32) / torch.maximum(active_f, torch.ones_like(active_f)), zero)
    stats[:, 4] = torch.where(has, share.to(torch.float32), zero)
    stats[:, 5] = torch.where(has & (sort.raw_len > 0), last_bucket.to(torch.float32), zero)
    return stats


class OneTransInference:
    """Forward-only OneTrans on one GPU.

    ``dtype`` is the activation / weight type of the dense path: ``torch.bfloat16`` (serving) or
    ``torch.float32`` (score-parity runs against the reference's fp32 torch path: dense layers in fp32 through
    the library, attention through this library's plain fp32 kernel, so nothing between the inputs and the
    scores is rounded to 16 bits).

    ``ffn="fp8"`` runs the shared FFN of every block through the e4m3 block-scaled tcgen05 GEMMs
    (bf16 activations only; needs d_model % 256 == 0 and hidden % 256 == 0); ``"bf16"`` uses cuBLAS.

    ``packed=True`` (single sequence domain) stores only VALID tokens: padded positions never influence
    a score (they are masked as keys, excluded from the pooled means, and as queries only produce rows
    that nothing reads), so the engine drops them after the tokenizer and runs every layer on a packed
    ``[sum_b (len_b + ns), d]`` matrix with per-sample row offsets.  ``packed=False`` keeps the
    reference's padded ``[B, T, d]`` layout (used for several sequence domains and as a cross-check).
    """

    def __init__(self, state_dict: dict[str, torch.Tensor], spec: OneTransSpec, *, device: torch.device | str = "cuda",
                 dtype: torch.dtype = torch.bfloat16, attention_kernel: int = 0, ffn: str = "bf16",
                 packed: bool = True, select_early: bool = True, fused_tokenizer: bool = False) -> None:
        if not ops.cuda_available():
            raise RuntimeError("OneTransInference needs the cuda backend (libtb200 + an sm_100 device)")
        self.spec = spec
        self.device = torch.device(device)
        self.dtype = dtype
        self.attention_kernel = attention_kernel
        # packed layout: apply the pyramid's row selection right after attention, before the row-wise half of the
        # block (same rows, same values; False keeps the reference's order: whole block, then selection)
        self.select_early = select_early
        # packed layout, bf16: gather -> projection -> SiLU / LayerNorm / time and position rows / first RMSNorm of the
        # sequence tokenizer as ONE kernel (`ops.token_project`) instead of the row gather, the projection GEMM and the
        # fused tail.  Off by default: measured on 1 M rows the one-kernel form takes 1.27 ms against 0.79 ms.
        self.fused_tokenizer = bool(fused_tokenizer)
        self._meta_ring: list[torch.Tensor] = []
        self._copy_stream: torch.cuda.Stream | None = None
        self._meta_next = 0
        if ffn not in ("bf16", "fp8", "fp8_precise", "fp8_mx"):
            raise ValueError(f"unknown ffn mode {ffn}")
        # "fp8_mx": power-of-two block scales applied inside the block-scaled tensor-core instruction (ops.ffn_mx)
        self.ffn_mx = ffn == "fp8_mx"
        ffn = "fp8" if self.ffn_mx else ffn
        # "fp8_precise": GEMM 1 of the shared FFN on the bf16 tensor cores, only its hidden activation and the down
        # projection in e4m3 (ops.ffn_fp8(precise=True))
        self.ffn_precise = ffn == "fp8_precise"
        ffn = "fp8" if self.ffn_precise else ffn
        if ffn == "fp8" and (dtype != torch.bfloat16 or spec.d_model % 256 or (spec.d_model * spec.hidden_mult) % 256):
            raise RuntimeError("ffn='fp8' needs bf16 activations, d_model % 256 == 0 and hidden % 256 == 0")
        self.ffn_mode = ffn
        self.packed = bool(packed)
        self.d = spec.d_model
        heads = max(1, spec.num_heads)
        if self.d % heads:  # choose_num_heads (modeling/sequence.py:70-78)
            heads = next(h for h in range(min(heads, self.d), 0, -1) if self.d % h == 0)
        self.heads = heads
        self.head_dim = self.d // heads
        if self.head_dim not in (32, 64, 128):
            raise RuntimeError(f"cuda attention supports head_dim 32, 64 or 128, got {self.head_dim}")
        self.domains = sorted(spec.seq_vocab_sizes)
        self.n_blocks = max(1, spec.num_blocks)
        self.seq_keep = max(1, int(spec.seq_top_k))
        self.w = {k: v.to(self.device) for k, v in state_dict.items()}
        self._edges = torch.tensor(_BUCKET_EDGES, dtype=torch.long, device=self.device)
        self._cast_cache: dict[str, torch.Tensor] = {}

        self.user_bank = self._make_bank("user_tokenizer.bank", spec.user_int_specs, compress=False)
        self.item_bank = self._make_bank("item_tokenizer.bank", spec.item_int_specs, compress=True)
        self.user_tokens = self._ns_token_count(spec.user_ns_tokens, spec.user_ns_groups, spec.user_int_specs)
        self.item_tokens = self._ns_token_count(spec.item_ns_tokens, spec.item_ns_groups, spec.item_int_specs)
        self.num_ns = (self.user_tokens + self.item_tokens + int(spec.user_dense_dim > 0) + int(spec.item_dense_dim > 0)
                       + int(bool(self.domains)))
        self.seq_tables: dict[str, list[tuple[str, torch.Tensor | None]]] = {}
        for domain in self.domains:
            entries: list[tuple[str, torch.Tensor | None]] = []
            n_plain = n_comp = 0
            for vocab in spec.seq_vocab_sizes[domain]:
                kind = _table_kind(vocab, spec.emb_skip_threshold, True)
                if kind == "table":
                    entries.append((kind, self._table(f"sequence_tokenizers.{domain}.embeddings.{n_plain}.weight")))
                    n_plain += 1
                elif kind == "compressed":
                    entries.append((kind, self._table(f"sequence_tokenizers.{domain}.compressed_embeddings.{n_comp}.weight")))
                    n_comp += 1
                else:
                    entries.append((kind, None))
            self.seq_tables[domain] = entries
        self._prepare_blocks()
        self._pos_cache: dict[int, torch.Tensor] = {}
        # One persistent device word for every tcgen05 launch of this engine (attention, FP8 and grouped GEMMs):
        # a kernel whose bounded wait gives up raises it.  Passing it costs nothing per call; it is read back by
        # `raise_if_incomplete` (one small device-to-host copy), which `score_stream` calls for the caller.
        self.status_word = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._hash_buckets: dict[str, torch.Tensor] = {}   # per sequence domain: how each feature's ids are hashed

    # ------------------------------------------------------------------ weights
    def _p(self, name: str) -> torch.Tensor:
        """Parameter in the compute dtype (cast once)."""
        t = self._cast_cache.get(name)
        if t is None:
            t = self.w[name].to(self.dtype).contiguous()
            self._cast_cache[name] = t
        return t

    def _table(self, name: str) -> torch.Tensor:
        return self._p(name)

    @staticmethod
    def _ns_token_count(n_tokens: int, groups: list[list[int]], specs) -> int:
        groups = list(groups) or [[i] for i in range(len(specs))]
        return int(n_tokens) if n_tokens > 0 else len(groups)

    def _make_bank(self, prefix: str, specs, *, compress: bool) -> _Bank:
        if not specs:
            return _Bank(None, 0, [])
        zero_table = torch.zeros(1, self.spec.emb_dim, dtype=self.dtype, device=self.device)
        tables, hashed = [], []
        n_plain = n_comp = 0
        for vocab, offset, length in specs:
            kind = _table_kind(vocab, self.spec.emb_skip_threshold, compress)
            if kind == "table":
                tables.append(self._table(f"{prefix}.embeddings.{n_plain}.weight"))
                n_plain += 1
            elif kind == "compressed":
                table = self._table(f"{prefix}.compressed_embeddings.{n_comp}.weight")
                tables.append(table)
                hashed.append((offset, length, table.shape[0] - 1))
                n_comp += 1
            else:
                tables.append(zero_table)  # every id clamps to the padding row -> zeros
        fields = ops.FieldTables(tables, [s[1] for s in specs], [s[2] for s in specs])
        return _Bank(fields, len(specs), hashed)

    def _prepare_blocks(self) -> None:
        """Stack the per-NS-token projections so that each block needs three batched matmuls."""
        ns = self.num_ns
        self.blocks = []
        for layer in range(self.n_blocks):
            p = f"blocks.{layer}"
            blk = {"p": p}
            if self.ffn_mode == "fp8":
                if self.ffn_mx:
                    blk["ffn_fp8"] = ops.MxFfnWeights(
                        self.w[p + ".ffn.shared.net.0.weight"], self.w[p + ".ffn.shared.net.3.weight"], gated=False,
                        b_up=self.w[p + ".ffn.shared.net.0.bias"], b_down=self.w[p + ".ffn.shared.net.3.bias"])
                else:
                    blk["ffn_fp8"] = ops.Fp8FfnWeights(
                        self.w[p + ".ffn.shared.net.0.weight"], self.w[p + ".ffn.shared.net.3.weight"], gated=False,
                        b_up=self.w[p + ".ffn.shared.net.0.bias"], b_down=self.w[p + ".ffn.shared.net.3.bias"],
                        precise=self.ffn_precise)
                # The packed path leaves the attention output bias out of the residual stream it hands to the
                # FFN (the norm in between adds it on the fly), so the FFN's own output bias carries it.
                folded = copy.copy(blk["ffn_fp8"])
                folded.b_down = (folded.b_down + self.w[p + ".attention.out.bias"].float()).contiguous()
                blk["ffn_fp8_folded"] = folded
            blk["out_w_t"] = self._p(p + ".attention.out.weight").t()
            blk["out_b"] = self._p(p + ".attention.out.bias")
            # shared projections as `nn.Linear` weights ([out, in], contiguous row blocks) with fp32 biases: what the
            # tcgen05 GEMM takes.  Rows [0, d) of shared_qkv are the queries, [d, 3d) keys and values.
            d_model = self.d
            w_qkv, b_qkv = self._p(p + ".attention.shared_qkv.weight"), self.w[p + ".attention.shared_qkv.bias"].float()
            blk["qkv_w"], blk["qkv_b"] = w_qkv, b_qkv.contiguous()
            blk["q_w"], blk["q_b"] = w_qkv[:d_model], b_qkv[:d_model].contiguous()
            blk["kv_w"], blk["kv_b"] = w_qkv[d_model:], b_qkv[d_model:].contiguous()
            blk["out_w"] = self._p(p + ".attention.out.weight")
            blk["out_b32"] = self.w[p + ".attention.out.bias"].float().contiguous()
            if ns > 0:
                def stack(fmt: str, kind: str) -> torch.Tensor:
                    return torch.stack([self._p(fmt.format(i=i) + "." + kind) for i in range(ns)])

                wq, wk, wv = (stack(p + f".attention.ns_{n}." + "{i}", "weight") for n in "qkv")
                bq, bk, bv = (stack(p + f".attention.ns_{n}." + "{i}", "bias") for n in "qkv")
                blk["ns_qkv_w"] = torch.cat([wq, wk, wv], dim=1).transpose(1, 2).contiguous()  # [ns, d, 3d]
                blk["ns_qkv_b"] = torch.cat([bq, bk, bv], dim=1).unsqueeze(1)  # [ns, 1, 3d]
                blk["ns_q_w"] = blk["ns_qkv_w"][:, :, :d_model].contiguous()     # query / key-value halves for blocks
                blk["ns_kv_w"] = blk["ns_qkv_w"][:, :, d_model:].contiguous()    # that project fewer queries than keys
                blk["ns_q_b"] = blk["ns_qkv_b"][:, :, :d_model].contiguous()
                blk["ns_kv_b"] = blk["ns_qkv_b"][:, :, d_model:].contiguous()
                blk["ns_w1"] = stack(p + ".ffn.ns_specific.{i}.net.0", "weight").transpose(1, 2).contiguous()
                blk["ns_b1"] = stack(p + ".ffn.ns_specific.{i}.net.0", "bias").unsqueeze(1)
                blk["ns_w2"] = stack(p + ".ffn.ns_specific.{i}.net.3", "weight").transpose(1, 2).contiguous()
                blk["ns_b2"] = stack(p + ".ffn.ns_specific.{i}.net.3", "bias").unsqueeze(1)
                blk["ns_b2_folded"] = (blk["ns_b2"].float() + blk["out_b"].float()).to(blk["ns_b2"].dtype)
                # The same layers for the grouped tcgen05 GEMM, which takes stacked `nn.Linear` weights as they are
                # ([token, out, in]) and adds bias, SiLU and residual in its epilogue (bf16, widths in whole tiles).
                hidden = blk["ns_w1"].shape[2]
                if self.dtype == torch.bfloat16 and self.device.type == "cuda" and d_model % 256 == 0 and hidden % 256 == 0:
                    blk["g_qkv_w"] = torch.cat([wq, wk, wv], dim=1).contiguous()                       # [ns, 3d, d]
                    blk["g_qkv_b"] = blk["ns_qkv_b"].reshape(ns, 3 * d_model).float().contiguous()
                    blk["g_q_w"], blk["g_kv_w"] = wq.contiguous(), torch.cat([wk, wv], dim=1).contiguous()
                    blk["g_q_b"] = blk["g_qkv_b"][:, :d_model].contiguous()
                    blk["g_kv_b"] = blk["g_qkv_b"][:, d_model:].contiguous()
                    blk["g_b2"] = blk["ns_b2"].reshape(ns, d_model).float().contiguous()
                    blk["g_w1"] = stack(p + ".ffn.ns_specific.{i}.net.0", "weight").contiguous()       # [ns, hidden, d]
                    blk["g_b1"] = blk["ns_b1"].reshape(ns, hidden).float().contiguous()
                    blk["g_w2"] = stack(p + ".ffn.ns_specific.{i}.net.3", "weight").contiguous()       # [ns, d, hidden]
                    blk["g_b2_folded"] = (blk["ns_b2"].float() + blk["out_b"].float()).reshape(ns, d_model).contiguous()
                    blk["g_out_w"] = self._p(p + ".attention.out.weight").contiguous()                 # [d, d]
            self.blocks.append(blk)

    # ------------------------------------------------------------------ pieces
    def _linear(self, x: torch.Tensor, prefix: str, *, silu: bool = False, residual: torch.Tensor | None = None) -> torch.Tensor:
        key = prefix + "#b32"
        if key not in self._cast_cache:
            self._cast_cache[key] = self.w[prefix + ".bias"].float().contiguous()
        return self._proj(x, self._p(prefix + ".weight"), self._cast_cache[key], silu=silu, residual=residual)

    def _ffn_fp8(self, x: torch.Tensor, weights, residual: torch.Tensor) -> torch.Tensor:
        if self.ffn_mx:
            return ops.ffn_mx(x, weights, residual=residual, status=self.status_word)
        return ops.ffn_fp8(x, weights, residual=residual, status=self.status_word, precise=self.ffn_precise)

    def _own_gemm(self, n: int, k: int) -> bool:
        """The tcgen05 GEMM serves bf16 layers whose widths are whole tiles; the fp32 score-parity mode and odd
        shapes (the 32-wide dense token, d_model below 256) go to the library."""
        return self.dtype == torch.bfloat16 and self.device.type == "cuda" and n % 256 == 0 and k % 64 == 0

    def _proj(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, *, silu: bool = False,
              residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """``act(x @ weight.T + bias) (+ residual)`` for a shared `nn.Linear` ([N, K] weight, fp32 bias): this
        library's tcgen05 GEMM with the epilogue inside where it applies, the library GEMM otherwise."""
        n, k = weight.shape
        lead = x.shape[:-1]
        if self._own_gemm(n, k):
            x2 = x.reshape(-1, k)
            y = ops.grouped_linear(x2 if x2.is_contiguous() else x2.contiguous(), weight, bias, silu=silu,
                                   residual=None if residual is None else residual.reshape(-1, n),
                                   out=None if out is None else out.view(-1, n), status=self.status_word)
            return y.view(*lead, n)
        with ops.timed("cublas_linear", m=x.numel() // k, n=n, k=k):
            y = F.linear(x, weight, None if bias is None else bias.to(x.dtype))
        if silu:
            y = F.silu(y)
        if residual is not None:
            y = y + residual
        if out is not None:
            out.copy_(y)
            return out
        return y

    def _grouped(self, x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, **kw) -> torch.Tensor:
        return ops.grouped_linear(x, weight, bias, status=self.status_word, **kw)

    def raise_if_incomplete(self) -> None:
        """Read the engine's status word (a 4-byte device-to-host copy, which waits for the work enqueued so far)
        and raise if a bounded wait inside one of the tcgen05 kernels gave up since the last call: the scores
        computed in between are then incomplete."""
        if int(self.status_word.item()) != 0:
            self.status_word.zero_()
            raise RuntimeError("cuda backend: a bounded wait inside a tcgen05 kernel gave up; scores are incomplete")

    def _layer_norm(self, x: torch.Tensor, prefix: str, pre_silu: bool = False) -> torch.Tensor:
        return ops.layer_norm(x, self._p(prefix + ".weight"), self._p(prefix + ".bias"), 1e-5, pre_silu=pre_silu)

    def _bank_tokens(self, bank: _Bank, int_feats: torch.Tensor, missing: torch.Tensor | None = None,
                     missing_rows: torch.Tensor | None = None) -> torch.Tensor:
        if bank.fields is None:
            return torch.zeros(int_feats.shape[0], 0, self.spec.emb_dim, dtype=self.dtype, device=self.device)
        if bank.hashed:
            int_feats = int_feats.clone()
            for offset, length, buckets in bank.hashed:
                cols = int_feats[:, offset : offset + length]
                int_feats[:, offset : offset + length] = hash_compress_ids(cols.clamp_min(0), buckets)
        return ops.fields_bag_mean(bank.fields, int_feats, missing, missing_rows)

    def _ns_tokenizer(self, prefix: str, bank: _Bank, n_tokens: int, groups, int_feats, missing) -> torch.Tensor:
        """`NonSequentialTokenizer.forward` (modeling/tokenizers.py:63-87)."""
        batch = int_feats.shape[0]
        key = prefix + ".missing_embeddings"
        if key in self.w and missing is not None and bank.fields is not None and missing.dtype == torch.bool \
                and missing.shape[1] >= bank.fields.n_fields:
            feats = self._bank_tokens(bank, int_feats, missing, self._p(key))     # the missing rows ride in the gather kernel
        else:
            feats = self._bank_tokens(bank, int_feats)
            if key in self.w and missing is not None and feats.shape[1] > 0:
                m = missing[:, : feats.shape[1]].to(self.dtype)
                feats = feats + m.unsqueeze(-1) * self._p(key)[: feats.shape[1]].unsqueeze(0)
        if n_tokens <= 0:
            return torch.zeros(batch, 0, self.d, dtype=self.dtype, device=self.device)
        groups = [list(g) for g in groups] or [[i] for i in range(bank.n_fields)]
        if self.spec.force_auto_split or n_tokens != len(groups):
            flat = feats.reshape(batch, -1) if feats.shape[1] > 0 else torch.zeros(batch, 1, dtype=self.dtype, device=self.device)
            h = self._linear(flat, prefix + ".project.0")
            return self._layer_norm(h, prefix + ".project.2", pre_silu=True).view(batch, n_tokens, self.d)
        grouped = []
        for g in groups:
            idx = [i for i in g if 0 <= i < feats.shape[1]]
            grouped.append(feats[:, idx, :].mean(dim=1) if idx else torch.zeros(batch, self.spec.emb_dim, dtype=self.dtype, device=self.device))
        return self._layer_norm(self._linear(torch.stack(grouped, dim=1), prefix + ".project.0"), prefix + ".project.1")

    def _dense_token(self, prefix: str, dim: int, values: torch.Tensor, missing: torch.Tensor | None):
        """`DenseTokenProjector.forward` (modeling/tokenizers.py:101-111)."""
        if dim <= 0:
            return None
        values = values.to(self.dtype)
        miss = torch.zeros_like(values) if missing is None else missing[:, : values.shape[1]].to(self.dtype)
        h = self._linear(torch.cat([values, miss], dim=-1), prefix + ".project.0")
        return self._layer_norm(h, prefix + ".project.2", pre_silu=True).unsqueeze(1)

    def _sequence_tokens(self, domain: str, values: torch.Tensor, timestamps: torch.Tensor, request_ts: torch.Tensor):
        """`SequenceTokenizer.forward` (modeling/tokenizers.py:156-190)."""
        prefix = f"sequence_tokenizers.{domain}"
        entries = self.seq_tables[domain]
        batch, n_feat, length = values.shape
        if any(kind == "compressed" for kind, _ in entries):
            values = values.clone()
            for f, (kind, table) in enumerate(entries):
                if kind == "compressed":
                    values[:, f] = hash_compress_ids(values[:, f].clamp_min(0), table.shape[0] - 1)
        tables = [entries[f][1] if f < len(entries) else None for f in range(n_feat)]
        if all(t is None for t in tables):
            width = max(1, n_feat * self.spec.emb_dim) if n_feat else 1
            token_input = torch.zeros(batch, length, width, dtype=self.dtype, device=self.device)
        else:
            token_input = ops.sequence_gather(tables, values)
        h = F.silu(self._linear(token_input, prefix + ".project.0"))
        tokens = self._layer_norm(h, prefix + ".project.2")
        key = prefix + ".time_embedding.weight"
        if key in self.w:
            buckets = sequence_time_buckets(timestamps, request_ts, self._edges)
            tokens = tokens + ops.gather_rows(self._p(key), buckets)
        return tokens

    def _positions(self, length: int) -> torch.Tensor:
        """Sinusoidal table, computed in fp32 like the reference (modeling/sequence.py:130-138)."""
        table = self._pos_cache.get(length)
        if table is None:
            pos = torch.arange(length, dtype=torch.float32, device=self.device).unsqueeze(1)
            freq = torch.exp(torch.arange(0, self.d, 2, dtype=torch.float32, device=self.device) * (-math.log(10000.0) / self.d))
            table = torch.zeros(length, self.d, device=self.device)
            table[:, 0::2] = torch.sin(pos * freq)
            table[:, 1::2] = torch.cos(pos * freq[: table[:, 1::2].shape[1]])
            table = table.to(self.dtype)
            self._pos_cache[length] = table
        return table

    def _tail_crop(self, tokens: torch.Tensor, lengths: torch.Tensor) -> torch.Tensor:
        """Last ``seq_top_k`` valid positions of every row (experiments/onetrans/model.py:278-285)."""
        keep = self.seq_keep
        if tokens.shape[1] <= keep:
            return tokens
        start = (lengths - keep).clamp_min(0)
        idx = (start[:, None] + torch.arange(keep, device=self.device)[None, :]).clamp_max(tokens.shape[1] - 1)
        return tokens.gather(1, idx[:, :, None].expand(-1, -1, tokens.shape[-1]))

    # ------------------------------------------------------------------ blocks
    def _shared_ffn_residual(self, blk: dict, x: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
        """tokens + FFN(x) for every row (`FeedForward`, experiments/onetrans/model.py:33-44)."""
        if self.ffn_mode == "fp8":
            return self._ffn_fp8(x, blk["ffn_fp8"], tokens)
        p = blk["p"]
        return self._linear(self._linear(x, p + ".ffn.shared.net.0", silu=True), p + ".ffn.shared.net.3", residual=tokens)

    def _block(self, blk: dict, tokens: torch.Tensor, mask: dict, seq_count: int) -> torch.Tensor:
        """`OneTransBlock.forward` (experiments/onetrans/model.py:97-107)."""
        p = blk["p"]
        batch, total, d = tokens.shape
        ns_here = max(0, min(self.num_ns, total - seq_count))
        x = ops.rms_norm(tokens, self._p(p + ".attn_norm.weight"), 1e-6)
        qkv = self._linear(x, p + ".attention.shared_qkv")  # [B, T, 3d]
        if ns_here > 0:
            x_ns = x[:, seq_count : seq_count + ns_here].transpose(0, 1)  # [ns, B, d]
            qkv[:, seq_count : seq_count + ns_here] = torch.baddbmm(
                blk["ns_qkv_b"][:ns_here], x_ns, blk["ns_qkv_w"][:ns_here]
            ).transpose(0, 1)
        q, k, v = (qkv[:, :, i * d : (i + 1) * d].unflatten(-1, (self.heads, self.head_dim)) for i in range(3))
        attn = ops.varlen_attention(q, k, v, causal=True, padded_query_self=True, layout="blhd",
                                    kernel=self.attention_kernel, **mask, status=self.status_word)
        attn = attn.view(batch, total, d).to(self.dtype)
        tokens = tokens + self._linear(attn, p + ".attention.out")

        x = ops.rms_norm(tokens, self._p(p + ".ffn_norm.weight"), 1e-6)
        out = self._shared_ffn_residual(blk, x, tokens.contiguous())
        if ns_here > 0:  # the NS tokens own their FFNs (model.py:89-93): overwrite their rows
            x_ns = x[:, seq_count : seq_count + ns_here].transpose(0, 1)
            h = F.silu(torch.baddbmm(blk["ns_b1"][:ns_here], x_ns, blk["ns_w1"][:ns_here]))
            y_ns = torch.baddbmm(blk["ns_b2"][:ns_here], h, blk["ns_w2"][:ns_here]).transpose(0, 1)
            out[:, seq_count : seq_count + ns_here] = tokens[:, seq_count : seq_count + ns_here] + y_ns
        return out

    # ------------------------------------------------------------------ forward
    def _ns_tokens(self, inputs, stat_vectors: list[torch.Tensor]) -> torch.Tensor:
        """All non-sequence tokens [B, ns, d] (experiments/onetrans/model.py:240-252)."""
        spec = self.spec
        parts = [self._ns_tokenizer("user_tokenizer", self.user_bank, self.user_tokens, spec.user_ns_groups,
                                    inputs.user.int_values, inputs.user.int_missing_mask)]
        tok = self._dense_token("user_dense", spec.user_dense_dim, inputs.user.dense_values, inputs.user.dense_missing_mask)
        if tok is not None:
            parts.append(tok)
        parts.append(self._ns_tokenizer("item_tokenizer", self.item_bank, self.item_tokens, spec.item_ns_groups,
                                        inputs.item.int_values, inputs.item.int_missing_mask))
        tok = self._dense_token("item_dense", spec.item_dense_dim, inputs.item.dense_values, inputs.item.dense_missing_mask)
        if tok is not None:
            parts.append(tok)
        if stat_vectors:
            parts.append(torch.stack(stat_vectors, dim=1).mean(dim=1, keepdim=True).to(self.dtype))
        return torch.cat(parts, dim=1)

    def _stats_vector(self, stats: torch.Tensor) -> torch.Tensor:
        # raw counts (up to the sequence length) do not survive bf16: this small projector stays fp32
        h = F.silu(F.linear(stats, self.w["sequence_stats_projector.0.weight"].float(),
                            self.w["sequence_stats_projector.0.bias"].float()))
        return ops.layer_norm(h, self.w["sequence_stats_projector.2.weight"].float(),
                              self.w["sequence_stats_projector.2.bias"].float(), 1e-5)

    def _classify(self, seq_summary: torch.Tensor, ns_summary: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        embeddings = torch.cat([seq_summary, ns_summary], dim=-1)
        if self._own_gemm(self.d, 2 * self.d):
            # serving mode: the wide layer on the tcgen05 GEMM (bias + SiLU in its epilogue); its inputs come out of a
            # bf16 network, so bf16 operands with fp32 accumulation lose nothing that was still there
            h = self._linear(embeddings.to(self.dtype), "classifier.0", silu=True).float()
        else:
            h = F.silu(F.linear(embeddings, self.w["classifier.0.weight"].float(), self.w["classifier.0.bias"].float()))
        logits = F.linear(h, self.w["classifier.3.weight"].float(), self.w["classifier.3.bias"].float())
        return logits, embeddings

    @torch.inference_mode()
    def predict(self, inputs, prepared: dict | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """(logits [B, action_num], pooled embeddings [B, 2 d]) in fp32 — `PCVROneTrans.predict`.  ``prepared`` is
        what ``prepare(inputs)`` returned for these inputs (the serving loop computes it ahead of time)."""
        if self.packed and len(self.domains) == 1:
            return self._predict_packed(inputs, prepared)
        return self._predict_padded(inputs)

    @torch.inference_mode()
    def prepare(self, inputs) -> dict | None:
        """Everything of a forward that the host has to wait for, enqueued on the current stream: duplicate removal
        and statistics of the behaviour sequence, the row plan of the packed layout, and the asynchronous copy of the
        plan's per-layer totals into pinned host memory (with an event).  A serving loop calls this for batch i + 1 on
        a side stream while batch i is being scored; the forward of batch i + 1 then finds its buffer sizes on the
        host already and never drains the device.  None when the engine does not run the packed layout.  At most
        three results may be outstanding at a time: the pinned landing buffers are a ring of four."""
        if not (self.packed and len(self.domains) == 1):
            return None
        seq = inputs.sequences[self.domains[0]]
        ns = self.num_ns
        lengths, src_map, stats = ops.sequence_prepare(seq.values, seq.lengths, seq.timestamps, inputs.request_timestamp)
        max_len = seq.values.shape[2]
        width = min(max_len, self.seq_keep)            # padded sequence width S[0] after the tail crop
        widths = [width]                               # static schedule of padded widths
        for layer in range(self.n_blocks):
            widths.append(pyramid_keep_count(widths[-1], layer, self.n_blocks, ns))
        plan = ops.pyramid_plan(lengths.to(torch.long), max_len, widths, ns)
        # pinned landing buffers are kept in a small ring: allocating pinned memory per batch can stall on the device
        # when the host runs a batch ahead (a buffer comes round again four batches later, long after its forward
        # has read it)
        ring = self._meta_ring
        if not ring or ring[0].shape != plan["meta"].shape:
            ring[:] = [torch.empty(plan["meta"].shape, dtype=torch.int64, pin_memory=True) for _ in range(4)]
        meta_host = ring[self._meta_next % len(ring)]
        self._meta_next += 1
        meta_host.copy_(plan["meta"], non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        return {"src_map": src_map, "stats": stats, "plan": plan, "widths": widths, "meta_host": meta_host, "ready": ready,
                "batch": int(lengths.shape[0])}

    @staticmethod
    def prepared_tensors(prepared: dict) -> list[torch.Tensor]:
        """Device tensors of a ``prepare`` result (for ``Tensor.record_stream`` when it was made on another stream)."""
        plan = prepared["plan"]
        return [prepared["src_map"], prepared["stats"], plan["start"], plan["cu32"]]   # plan's int64 outputs share one allocation

    def _predict_padded(self, inputs) -> tuple[torch.Tensor, torch.Tensor]:
        dev = self.device
        batch = inputs.user.int_values.shape[0]
        request_ts = inputs.request_timestamp

        # ---- sequence stream (experiments/onetrans/model.py:287-315)
        pieces, valid_parts, stat_vectors = [], [], []
        single_len = None
        for di, domain in enumerate(self.domains):
            seq = inputs.sequences[domain]
            lengths, src_map, stats = ops.sequence_prepare(seq.values, seq.lengths, seq.timestamps, request_ts)
            stat_vectors.append(self._stats_vector(stats))
            keep_pos = src_map.clamp_min(0).long()
            gone = src_map < 0
            values = seq.values.gather(2, keep_pos[:, None, :].expand(-1, seq.values.shape[1], -1)).masked_fill(gone[:, None, :], 0)
            ts = seq.timestamps.gather(1, keep_pos).masked_fill(gone, 0)
            seq_len = lengths.clamp(min=0, max=values.shape[2])
            tokens = self._sequence_tokens(domain, values, ts, request_ts)
            tokens = self._tail_crop(tokens, seq_len)
            seq_len = seq_len.clamp_max(tokens.shape[1])
            tokens = tokens + self._positions(tokens.shape[1]).unsqueeze(0)
            pieces.append(tokens)
            valid_parts.append(torch.arange(tokens.shape[1], device=dev)[None, :] < seq_len[:, None])
            single_len = seq_len
            if di < len(self.domains) - 1:
                pieces.append(self._p("separator_tokens")[di].view(1, 1, -1).expand(batch, -1, -1))
                valid_parts.append(torch.ones(batch, 1, dtype=torch.bool, device=dev))
        seq_tokens = torch.cat(pieces, dim=1) if pieces else torch.zeros(batch, 0, self.d, dtype=self.dtype, device=dev)
        seq_count = seq_tokens.shape[1]
        ns_tokens = self._ns_tokens(inputs, stat_vectors)
        tokens = torch.cat([seq_tokens, ns_tokens], dim=1)

        # ---- mask description: one valid prefix (single domain) or a per-key validity map
        structured = len(self.domains) <= 1
        if structured:
            base_len = single_len if single_len is not None else torch.zeros(batch, dtype=torch.long, device=dev)
            valid_map = None
        else:
            base_len = None
            valid_map = torch.cat(valid_parts + [torch.ones(batch, ns_tokens.shape[1], dtype=torch.bool, device=dev)], dim=1)
        dropped = 0  # sequence positions removed from the front so far

        for layer, blk in enumerate(self.blocks):
            if structured:
                mask = {"seq_len": (base_len - dropped).clamp(min=0, max=seq_count).to(torch.int32), "ns_start": seq_count}
            else:
                mask = {"key_valid": valid_map}
            tokens = self._block(blk, tokens, mask, seq_count)
            keep = pyramid_keep_count(seq_count, layer, self.n_blocks, self.num_ns)
            if keep < seq_count:  # keep the LAST `keep` sequence positions (:340-348)
                cut = seq_count - keep
                tokens = tokens[:, cut:]
                if valid_map is not None:
                    valid_map = valid_map[:, cut:]
                dropped += cut
                seq_count = keep

        tokens = ops.rms_norm(tokens.contiguous(), self._p("final_norm.weight"), 1e-6).float()
        if structured:
            seq_valid = torch.arange(seq_count, device=dev)[None, :] < (base_len - dropped).clamp(min=0)[:, None]
        else:
            seq_valid = valid_map[:, :seq_count]
        if seq_count > 0:
            wgt = seq_valid.to(torch.float32).unsqueeze(-1)
            seq_summary = (tokens[:, :seq_count] * wgt).sum(dim=1) / wgt.sum(dim=1).clamp_min(1.0)
        else:
            seq_summary = torch.zeros(batch, self.d, device=dev)
        ns_part = tokens[:, seq_count:]
        ns_summary = ns_part.mean(dim=1) if ns_part.shape[1] > 0 else torch.zeros(batch, self.d, device=dev)
        return self._classify(seq_summary, ns_summary)

    def _predict_packed(self, inputs, prepared: dict | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Same forward on valid tokens only (one sequence domain).

        Sample b owns ``n[b] + ns`` consecutive rows: its valid sequence tokens in order, then its NS
        tokens.  After block i the reference keeps the last ``S[i+1]`` padded positions; in packed form
        that drops the first ``min(n[b], S[i] - S[i+1])`` sequence rows of every sample.  All row counts
        follow from the per-sample lengths and the static pyramid schedule, so one device-to-host read
        of a few integers sizes every buffer of the forward."""
        dev = self.device
        domain = self.domains[0]
        batch = inputs.user.int_values.shape[0]
        ns = self.num_ns
        seq = inputs.sequences[domain]
        request_ts = inputs.request_timestamp
        # duplicate removal + statistics: one kernel; `src` maps output slots to input positions, so the
        # compacted [B, F, L] / [B, L] tensors of the reference are never materialised.  The valid counts, row
        # offsets and totals that the static pyramid schedule implies come from a second kernel; the totals are the
        # one host read of the forward (already on the host when the serving loop prepared this batch ahead of time)
        if prepared is None or prepared["batch"] != batch:
            prepared = self.prepare(inputs)
        src_map, stats, plan, widths = prepared["src_map"], prepared["stats"], prepared["plan"], prepared["widths"]
        stat_vectors = [self._stats_vector(stats)]
        values, ts = seq.values, seq.timestamps
        max_len = values.shape[2]
        width = widths[0]
        start, n0 = plan["start"], plan["n0"]          # first kept position / valid sequence tokens at layer 0
        counts = list(plan["counts"].unbind(0))        # [layers + 1] x [B] valid sequence tokens per sample
        cu = list(plan["cu"].unbind(0))                # [layers + 1] x [B + 1] row offsets
        cu_i32 = list(plan["cu32"].unbind(0))
        prepared["ready"].synchronize()
        meta = prepared["meta_host"].tolist()
        totals = [int(m[0]) for m in meta]
        max_rows = [int(m[1]) for m in meta]

        # ---- sequence tokenizer on the valid events only (modeling/tokenizers.py:156-190).  It works
        # directly in the packed layout of layer 0: the rows reserved for the NS tokens carry id 0 (the
        # zero padding row) through the projection and are overwritten afterwards, which costs ns / (n + ns)
        # extra rows but saves a full scatter of the token matrix.
        total0 = totals[0]
        prefix = f"sequence_tokenizers.{domain}"
        entries = self.seq_tables[domain]
        n_feat = values.shape[1]
        emb = self.spec.emb_dim
        live = [f for f in range(n_feat) if f < len(entries) and entries[f][1] is not None]
        has_time = prefix + ".time_embedding.weight" in self.w
        # ids of every feature, position and time-gap bucket of every packed row: one kernel instead of a dozen
        # index operations over the token rows
        if domain not in self._hash_buckets:
            self._hash_buckets[domain] = torch.tensor(
                [(-1 if f not in live else (entries[f][1].shape[0] - 1 if entries[f][0] == "compressed" else 0))
                 for f in range(n_feat)], dtype=torch.long, device=dev)
        ids_all, pos_full, buckets_full = ops.packed_token_index(
            values, ts if has_time else None, request_ts, src_map, cu[0], n0, start, self._hash_buckets[domain], total0,
            edges=self._edges if has_time else None)
        seq_tables = [entries[f][1] if f in live else None for f in range(n_feat)]
        proj_w = self._p(prefix + ".project.0.weight")
        # gather -> projection -> SiLU -> LayerNorm -> time / position rows -> first RMSNorm as ONE kernel where the
        # shapes allow it (bf16, whole-tile widths); else the row gather, the projection GEMM and the fused tail
        one_kernel = (self.fused_tokenizer and self.dtype == torch.bfloat16 and bool(self.blocks) and bool(live)
                      and ops.token_project_supported(seq_tables, proj_w))
        projected = None
        if not one_kernel:
            if live:
                token_input = (torch.empty if len(live) == n_feat else torch.zeros)(
                    (total0, n_feat * emb), dtype=self.dtype, device=dev)
                for f in live:
                    ops.gather_rows(entries[f][1], ids_all[f], out=token_input, col0=f * emb)
            else:
                token_input = torch.zeros(total0, max(1, n_feat * emb), dtype=self.dtype, device=dev)
            # Linear -> SiLU -> LayerNorm, the time-bucket and position rows and the first block's RMSNorm in one pass
            # over the token matrix (`token_tail`); the NS rows are filled in afterwards
            projected = self._linear(token_input, prefix + ".project.0")
        ln_w, ln_b = self._p(prefix + ".project.2.weight"), self._p(prefix + ".project.2.bias")
        pos_table = self._positions(width).to(self.dtype).contiguous()
        rows_a, rows_b = (pos_table, pos_full), (None, None)
        if has_time:
            rows_a, rows_b = (self._p(prefix + ".time_embedding.weight"), buckets_full), (pos_table, pos_full)
        first_norm_w = self._p(self.blocks[0]["p"] + ".attn_norm.weight") if self.blocks else None

        def kept_rows(layer: int, want_row_dst: bool = False):
            """Rows of layer ``layer`` that the pyramid keeps for the next one (in the next layer's order), the NS
            rows [B, ns] of the next layer and, on request, the destination of every row of this layer (-1 = dropped)."""
            src, next_ns, dst = ops.pyramid_kept_rows(cu[layer], cu[layer + 1], counts[layer], counts[layer + 1], ns,
                                                      totals[layer], totals[layer + 1], want_row_dst=want_row_dst)
            return (src, next_ns, dst) if want_row_dst else (src, next_ns)

        # When the first block is evaluated for the kept rows only, its residual stream is needed for those rows
        # alone: the fused pass then writes `tokens` already compacted and only `x_first` at full height.
        first_kept = None
        fused_tail = one_kernel or (first_norm_w is not None and projected.shape[1] % (16 // projected.element_size()) == 0)
        if fused_tail and self.select_early and widths[1] < widths[0] and not (ns > 0 and max_rows[0] == ns) \
                and totals[1] < 2**31:
            *first_kept, row_dst = kept_rows(0, want_row_dst=True)
        if one_kernel:
            key = prefix + ".project.0#b32"
            if key not in self._cast_cache:
                self._cast_cache[key] = self.w[prefix + ".project.0.bias"].float().contiguous()
            tokens, x_first = ops.token_project(seq_tables, ids_all, proj_w, self._cast_cache[key], ln_w, ln_b, rows_a[0],
                                                rows_a[1], rows_b[0], rows_b[1], first_norm_w,
                                                row_dst=None if first_kept is None else row_dst,
                                                rows_out=None if first_kept is None else totals[1],
                                                status=self.status_word)
        elif fused_tail:
            tokens, x_first = ops.token_tail(projected, ln_w, ln_b, rows_a[0], rows_a[1], rows_b[0], rows_b[1], first_norm_w,
                                             row_dst=None if first_kept is None else row_dst,
                                             rows_out=None if first_kept is None else totals[1])
        else:
            tokens = ops.layer_norm(projected, ln_w, ln_b, 1e-5, pre_silu=True)
            ops.add_gathered_rows(tokens, rows_a[0], rows_a[1], rows_b[0], rows_b[1])
            x_first = None

        # ---- the NS tokens take the rows left for them: [seq rows of b | ns rows of b]
        ns_tokens = self._ns_tokens(inputs, stat_vectors)                          # [B, ns, d]
        ns_rows = plan["ns_rows0"]                                                 # [B, ns]
        ns_flat = ns_tokens.reshape(batch * ns, self.d).contiguous()
        ops.scatter_rows(tokens, (ns_rows if first_kept is None else first_kept[1]).reshape(-1), ns_flat)
        if x_first is not None:   # the fused pass normalised placeholder rows there
            ops.scatter_rows(x_first, ns_rows.reshape(-1), ops.rms_norm(ns_flat, first_norm_w, 1e-6))

        d, heads, hd = self.d, self.heads, self.head_dim
        for layer, blk in enumerate(self.blocks):
            if ns > 0 and max_rows[layer] == ns:
                # no sample has a sequence token left from here on: the remaining blocks only see the NS tokens
                seq_summary = torch.zeros(batch, d, device=dev)
                ns_summary = self._ns_only_blocks(tokens, layer, batch)
                return self._classify(seq_summary, ns_summary)
            p = blk["p"]
            cu32 = cu_i32[layer]
            x = x_first if (layer == 0 and x_first is not None) else ops.rms_norm(tokens, self._p(p + ".attn_norm.weight"), 1e-6)
            flat_ns = ns_rows.t().reshape(-1)                                      # token-major: [ns, B] row ids
            x_ns = ops.gather_rows(x, flat_ns).view(ns, batch, d)                  # [ns, B, d], contiguous
            selected = self.select_early and widths[layer + 1] < widths[layer]
            if selected:
                # The pyramid keeps only the last rows of every sample after this block, and a row of the block's
                # output depends on the other rows through its keys and values alone.  So keys and values are
                # projected for every row, but queries, the attention rows, the output projection, the residual,
                # the norm and the FFN only for the rows that survive: the same rows, bit for bit in exact
                # arithmetic, as "whole block, then selection", without the work whose result would be dropped.
                src, next_ns_rows = first_kept if (layer == 0 and first_kept is not None) else kept_rows(layer)
                next_flat_ns = next_ns_rows.t().reshape(-1)
                # every row the pyramid keeps is an NS row: the shared query projection and the shared FeedForward
                # would be overwritten row for row by the per-token layers, so they are not run at all
                only_ns_kept = ns > 0 and max_rows[layer + 1] == ns and "g_w1" in blk
                kv = self._proj(x, blk["kv_w"], blk["kv_b"])                                        # [N, 2d]
                if only_ns_kept:
                    qm = torch.empty(totals[layer + 1], d, dtype=self.dtype, device=dev)
                else:
                    qm = self._proj(ops.gather_rows(x, src), blk["q_w"], blk["q_b"])                # [N', d]
                if "g_kv_w" in blk:   # the per-token overrides of the NS rows: grouped GEMM, bias in its epilogue
                    ops.scatter_rows(kv, flat_ns, self._grouped(x_ns, blk["g_kv_w"], blk["g_kv_b"]).view(ns * batch, 2 * d))
                    ops.scatter_rows(qm, next_flat_ns, self._grouped(x_ns, blk["g_q_w"], blk["g_q_b"]).view(ns * batch, d))
                else:
                    ops.scatter_rows(kv, flat_ns, torch.bmm(x_ns, blk["ns_kv_w"]).view(ns * batch, 2 * d), bias=blk["ns_kv_b"])
                    ops.scatter_rows(qm, next_flat_ns, torch.bmm(x_ns, blk["ns_q_w"]).view(ns * batch, d), bias=blk["ns_q_b"])
                q = qm.unflatten(-1, (heads, hd))
                k, v = (kv[:, i * d : (i + 1) * d].unflatten(-1, (heads, hd)) for i in range(2))
                attn = ops.varlen_attention(q, k, v, causal=True, cu_rows=cu32, max_rows=max_rows[layer],
                                            cu_rows_q=cu_i32[layer + 1], max_rows_q=max_rows[layer + 1],
                                            kernel=self.attention_kernel if self.attention_kernel in (0, 1, 4) else 0, status=self.status_word)
                if not (layer == 0 and first_kept is not None):   # else the tokenizer already wrote the kept rows only
                    tokens = ops.gather_rows(tokens, src)
                ns_rows, flat_ns = next_ns_rows, next_flat_ns
            else:
                qkv = self._proj(x, blk["qkv_w"], blk["qkv_b"])                       # [N, 3d]
                if "g_qkv_w" in blk:
                    ops.scatter_rows(qkv, flat_ns, self._grouped(x_ns, blk["g_qkv_w"], blk["g_qkv_b"]).view(ns * batch, 3 * d))
                else:
                    ops.scatter_rows(qkv, flat_ns, torch.bmm(x_ns, blk["ns_qkv_w"]).view(ns * batch, 3 * d), bias=blk["ns_qkv_b"])
                q, k, v = (qkv[:, i * d : (i + 1) * d].unflatten(-1, (heads, hd)) for i in range(3))
                attn = ops.varlen_attention(q, k, v, causal=True, cu_rows=cu32, max_rows=max_rows[layer],
                                            kernel=self.attention_kernel, status=self.status_word)
            attn2d = attn.view(-1, d).to(self.dtype)
            folded = self.ffn_mode == "fp8"
            if selected and only_ns_kept:
                # the rest of this block for NS rows only, finishing token-major ([ns, B, d]) as the NS-only blocks
                # want it: out projection with the residual in its epilogue, norm with the projection's bias added
                # on the fly, per-token FeedForward with bias (+ that bias) and residual in the epilogues
                tokens = self._proj(attn2d, blk["out_w"], None, residual=tokens, out=tokens)
                x = ops.rms_norm(tokens, self._p(p + ".ffn_norm.weight"), 1e-6, in_bias=blk["out_b"])
                x_ns = ops.gather_rows(x, flat_ns).view(ns, batch, d)
                tok = ops.gather_rows(tokens, flat_ns).view(ns, batch, d)
                h = self._grouped(x_ns, blk["g_w1"], blk["g_b1"], silu=True)
                tok = self._grouped(h, blk["g_w2"], blk["g_b2_folded"], residual=tok, out=tok)
                seq_summary = torch.zeros(batch, d, device=dev)
                if layer + 1 == len(self.blocks):
                    final = ops.rms_norm(tok.view(ns * batch, d), self._p("final_norm.weight"), 1e-6)
                    return self._classify(seq_summary, final.view(ns, batch, d).mean(dim=0, dtype=torch.float32))
                return self._classify(seq_summary, self._ns_only_blocks(tok, layer + 1, batch, token_major=True))
            if folded:
                # tokens + attention out-projection with the residual inside the GEMM's epilogue, in place; its bias
                # is added by the norm on the fly and rides on the FFN output biases into the next residual
                tokens = self._proj(attn2d, blk["out_w"], None, residual=tokens, out=tokens)
                x = ops.rms_norm(tokens, self._p(p + ".ffn_norm.weight"), 1e-6, in_bias=blk["out_b"])
                out = self._ffn_fp8(x, blk["ffn_fp8_folded"], tokens)
            else:
                tokens = self._proj(attn2d, blk["out_w"], blk["out_b32"], residual=tokens)
                x = ops.rms_norm(tokens, self._p(p + ".ffn_norm.weight"), 1e-6)
                out = self._shared_ffn_residual(blk, x, tokens)
            x_ns = ops.gather_rows(x, flat_ns).view(ns, batch, d)
            if "g_w1" in blk:   # per-token FeedForward on the grouped GEMM: bias + SiLU, then bias, in the epilogues
                h = self._grouped(x_ns, blk["g_w1"], blk["g_b1"], silu=True)
                y_ns = self._grouped(h, blk["g_w2"], blk["g_b2_folded" if folded else "g_b2"]).view(ns * batch, d)
                ops.scatter_rows(out, flat_ns, y_ns, residual=tokens)              # tokens + b2 + FFN_ns(x)
            else:
                h = ops.bias_silu_rows(torch.bmm(x_ns, blk["ns_w1"]), blk["ns_b1"])
                y_ns = torch.bmm(h, blk["ns_w2"]).view(ns * batch, d)
                ops.scatter_rows(out, flat_ns, y_ns, bias=blk["ns_b2_folded" if folded else "ns_b2"], residual=tokens)
            tokens = out
            if not selected and widths[layer + 1] < widths[layer]:  # pyramid: drop the earliest sequence rows of every sample
                src, ns_rows = kept_rows(layer)
                tokens = ops.gather_rows(tokens, src)

        last = len(widths) - 1
        tokens = ops.rms_norm(tokens, self._p("final_norm.weight"), 1e-6).float()
        n_last = counts[last]
        total_seq = totals[last] - batch * ns
        owner = torch.repeat_interleave(torch.arange(batch, device=dev), n_last, output_size=total_seq)
        first_seq = torch.zeros(batch + 1, dtype=torch.long, device=dev)
        first_seq[1:] = torch.cumsum(n_last, dim=0)
        seq_rows = cu[last][owner] + (torch.arange(total_seq, device=dev) - first_seq[owner])
        # rows of a sample are consecutive: a segmented sum in row order (no floating-point atomics, so the scores
        # of a batch do not depend on which GPU or which run computed them)
        seq_sum = torch.segment_reduce(tokens[seq_rows], "sum", lengths=n_last, axis=0, unsafe=True)
        seq_summary = seq_sum / n_last.clamp_min(1).to(torch.float32)[:, None]
        ns_summary = tokens[ns_rows.reshape(-1)].view(batch, ns, d).mean(dim=1)
        return self._classify(seq_summary, ns_summary)

    def _ns_only_blocks(self, tokens: torch.Tensor, first_layer: int, batch: int, token_major: bool = False) -> torch.Tensor:
        """Blocks ``first_layer`` .. end for a batch whose samples hold nothing but their NS tokens, then the final
        norm and the NS mean -> [B, d] fp32.

        With no sequence token left, every row of `OneTransBlock.forward` (experiments/onetrans/model.py:97-107)
        takes the per-token projections and the per-token FeedForward, and every sample attends causally over
        its ``ns`` tokens.  The block then is six batched or shared matrix products on a token-major
        ``[ns, B, d]`` tensor with no gathers, scatters or shared-weight work that would be overwritten."""
        ns, d, heads, hd = self.num_ns, self.d, self.heads, self.head_dim
        tok = tokens if token_major else tokens.view(batch, ns, d).transpose(0, 1).contiguous()            # [ns, B, d]
        flat = tok.view(ns * batch, d)
        for blk in self.blocks[first_layer:]:
            p = blk["p"]
            x = ops.rms_norm(flat, self._p(p + ".attn_norm.weight"), 1e-6)
            fused = "g_qkv_w" in blk   # every layer of the block in one tcgen05 GEMM each, epilogues inside
            if fused:
                qkv = self._grouped(x.view(ns, batch, d), blk["g_qkv_w"], blk["g_qkv_b"])
            else:
                qkv = ops.bias_act_rows(torch.bmm(x.view(ns, batch, d), blk["ns_qkv_w"]), blk["ns_qkv_b"], silu=False)
            # sample-major views of the token-major tensors: (B, L = ns, H, hd) with strides (3d, B * 3d, hd, 1)
            q, k, v = (qkv[:, :, i * d : (i + 1) * d].unflatten(-1, (heads, hd)).permute(1, 0, 2, 3) for i in range(3))
            attn = torch.empty(ns, batch, heads, hd, dtype=q.dtype, device=q.device)
            ops.varlen_attention(q, k, v, causal=True, layout="blhd", kernel=self.attention_kernel,
                                 out=attn.permute(1, 0, 2, 3), status=self.status_word)
            # attention output projection onto the residual stream; its bias is added by the norm on the fly and
            # rides on the FFN's output bias into the next residual
            if fused:
                self._grouped(attn.view(ns * batch, d), blk["g_out_w"], None, residual=flat, out=flat)
            else:
                flat.addmm_(attn.view(ns * batch, d).to(self.dtype), blk["out_w_t"])
            x = ops.rms_norm(flat, self._p(p + ".ffn_norm.weight"), 1e-6, in_bias=blk["out_b"])
            if fused:
                h = self._grouped(x.view(ns, batch, d), blk["g_w1"], blk["g_b1"], silu=True)
                tok = self._grouped(h, blk["g_w2"], blk["g_b2_folded"], residual=tok, out=tok)
            else:
                h = ops.bias_act_rows(torch.bmm(x.view(ns, batch, d), blk["ns_w1"]), blk["ns_b1"], silu=True)
                tok = ops.bias_act_rows(torch.baddbmm(tok, h, blk["ns_w2"]), blk["ns_b2_folded"], silu=False)
            flat = tok.view(ns * batch, d)
        final = ops.rms_norm(flat, self._p("final_norm.weight"), 1e-6)
        return final.view(ns, batch, d).mean(dim=0, dtype=torch.float32)     # widened inside the reduction, no fp32 copy

    @torch.inference_mode()
    def scores(self, inputs, micro_batch: int | None = None, prepared: dict | None = None) -> torch.Tensor:
        """Sigmoid conversion probabilities (fp32, on the device): [B] for one action, else [B, actions].
        ``micro_batch`` bounds the rows that go through the network at once (samples are independent,
        so the result does not depend on it); it caps activation memory at large batches.  ``prepared``: the
        result of ``prepare(inputs)`` for a batch that goes through in one piece."""
        batch = inputs.user.int_values.shape[0]
        if micro_batch is None or micro_batch >= batch:
            logits, _ = self.predict(inputs, prepared)
        else:
            logits = torch.cat([self.predict(inputs.slice(lo, min(lo + micro_batch, batch)))[0]
                                for lo in range(0, batch, micro_batch)])
        probs = torch.sigmoid(logits.float())
        return probs.reshape(-1) if probs.shape[1] == 1 else probs


def score_stream(model: "OneTransInference", host_batches, *, micro_batch: int | None = None, check_every: int = 0,
                 prepare_ahead: bool = True):
    """Scores for a stream of host-resident batches, one ``scores`` tensor (on the device) per batch.

    The serving loop of `evaluation/workflow.py:246-293` with the host-to-device copy taken off the critical
    path: the copy of batch i + 1 runs on a side stream while batch i is scored, so that in steady state a
    step costs max(copy, compute) instead of their sum.  ``host_batches`` should be pinned
    (``ModelInput.pin_memory()``) for the copies to be asynchronous.  A batch may also be a ``CompactModelInput``
    (``inputs.compact_model_input``): its sequences cross the link as 32-bit valid prefixes and are expanded to the
    padded int64 record by one kernel on the device.  Duplicate removal, sequence statistics and the row plan of
    batch i + 1 (``model.prepare``) also run on the side stream, and the few integers the host needs from them are
    in pinned memory before the forward of batch i + 1 starts: the host never drains the device between batches
    and can enqueue a whole batch ahead.

    The engine's status word (raised by a tcgen05 kernel whose bounded wait gave up) is read when the stream
    ends and, with ``check_every=n``, after every n-th batch; a raised word turns into a ``RuntimeError``
    instead of silently wrong scores."""
    dev = model.device
    compute = torch.cuda.current_stream(dev)
    # one copy stream per engine, kept across calls: device memory is pooled per stream, so a fresh stream per call
    # would have every call allocate its staging buffers anew
    if model._copy_stream is None:
        model._copy_stream = torch.cuda.Stream(dev)
    copier = model._copy_stream

    def stage(batch):
        copier.wait_stream(compute)          # pinned source and allocator state are in a known order
        with torch.cuda.stream(copier):
            staged = batch.to(dev, non_blocking=True)
            held = staged.tensors()
            if hasattr(staged, "expand"):    # compact host format: rebuild the padded record on the device
                staged = staged.expand()
                held = held + staged.tensors()
            # what the host must read before it can size the forward's buffers (row totals per layer) is computed
            # here, under the previous batch's kernels, so that the forward itself never waits for the device
            prepared = None
            if prepare_ahead and (micro_batch is None or micro_batch >= staged.batch_size):
                prepared = model.prepare(staged)
                if prepared is not None:
                    held = held + model.prepared_tensors(prepared)
            done = torch.cuda.Event()
            done.record(copier)
        return staged, prepared, held, done

    it = iter(host_batches)
    first = next(it, None)
    if first is None:
        return
    pending = stage(first)
    served = 0
    while pending is not None:
        staged, prepared, held, done = pending
        nxt = next(it, None)
        compute.wait_event(done)
        for t in held:                       # allocated on the copy stream, consumed on the compute stream
            t.record_stream(compute)
        pending = stage(nxt) if nxt is not None else None
        yield model.scores(staged, micro_batch=micro_batch, prepared=prepared)
        served += 1
        if check_every > 0 and served % check_every == 0:
            model.raise_if_incomplete()
    model.raise_if_incomplete()


def random_state_dict(spec: OneTransSpec, *, seed: int = 0, device: torch.device | str = "cpu",
                      dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """Seeded random weights with the parameter names, shapes and init scales of the reference module
    tree (xavier-normal tables with a zero padding row, modeling/embeddings.py:131-134; default
    `nn.Linear` / `nn.LayerNorm` init).  Generated directly on ``device`` so that multi-GB tables never
    touch the host.  The values are NOT the reference's seed-0 stream; golden-score checks use
    state_dicts exported from the reference itself."""
    g = torch.Generator(device=device).manual_seed(seed)
    sd: dict[str, torch.Tensor] = {}
    d, emb = spec.d_model, spec.emb_dim

    def table(name: str, rows: int, cols: int) -> None:
        std = math.sqrt(2.0 / (rows + cols))
        t = torch.empty(rows, cols, device=device, dtype=dtype).normal_(0.0, std, generator=g)
        t[0].zero_()
        sd[name] = t

    def linear(name: str, fan_in: int, fan_out: int) -> None:
        bound = 1.0 / math.sqrt(fan_in)
        sd[name + ".weight"] = (torch.rand(fan_out, fan_in, device=device, generator=g, dtype=dtype) * 2 - 1) * bound
        sd[name + ".bias"] = (torch.rand(fan_out, device=device, generator=g, dtype=dtype) * 2 - 1) * bound

    def norm(name: str, dim: int, bias: bool = True) -> None:
        sd[name + ".weight"] = torch.ones(dim, device=device, dtype=dtype)
        if bias:
            sd[name + ".bias"] = torch.zeros(dim, device=device, dtype=dtype)

    def bank(prefix: str, specs, compress: bool) -> None:
        n_plain = n_comp = 0
        for vocab, _o, _l in specs:
            kind = _table_kind(vocab, spec.emb_skip_threshold, compress)
            if kind == "table":
                table(f"{prefix}.embeddings.{n_plain}.weight", vocab + 1, emb)
                n_plain += 1
            elif kind == "compressed":
                table(f"{prefix}.compressed_embeddings.{n_comp}.weight", spec.emb_skip_threshold + 1, emb)
                n_comp += 1

    def ns_tokenizer(prefix: str, specs, n_tokens: int, groups, compress: bool) -> int:
        sd[prefix + ".missing_embeddings"] = torch.empty(len(specs), emb, device=device, dtype=dtype).normal_(0.0, 0.02, generator=g)
        bank(prefix + ".bank", specs, compress)
        groups = list(groups) or [[i] for i in range(len(specs))]
        n_tok = int(n_tokens) if n_tokens > 0 else len(groups)
        if spec.force_auto_split or n_tok != len(groups):
            linear(prefix + ".project.0", max(1, len(specs) * emb), n_tok * d)
            norm(prefix + ".project.2", n_tok * d)
        else:
            linear(prefix + ".project.0", emb, d)
            norm(prefix + ".project.1", d)
        return n_tok

    n_domains = len(spec.seq_vocab_sizes)
    sd["separator_tokens"] = torch.empty(max(1, n_domains - 1), d, device=device, dtype=dtype).normal_(0.0, 0.02, generator=g)
    num_ns = ns_tokenizer("user_tokenizer", spec.user_int_specs, spec.user_ns_tokens, spec.user_ns_groups, False)
    num_ns += ns_tokenizer("item_tokenizer", spec.item_int_specs, spec.item_ns_tokens, spec.item_ns_groups, True)
    for name, dim in (("user_dense", spec.user_dense_dim), ("item_dense", spec.item_dense_dim)):
        if dim > 0:
            linear(name + ".project.0", dim * 2, d)
            norm(name + ".project.2", d)
            num_ns += 1
    for domain in sorted(spec.seq_vocab_sizes):
        prefix = f"sequence_tokenizers.{domain}"
        n_plain = n_comp = 0
        vocabs = spec.seq_vocab_sizes[domain]
        for vocab in vocabs:
            kind = _table_kind(vocab, spec.emb_skip_threshold, True)
            if kind == "table":
                table(f"{prefix}.embeddings.{n_plain}.weight", vocab + 1, emb)
                n_plain += 1
            elif kind == "compressed":
                table(f"{prefix}.compressed_embeddings.{n_comp}.weight", spec.emb_skip_threshold + 1, emb)
                n_comp += 1
        linear(prefix + ".project.0", max(1, len(vocabs) * emb), d)
        norm(prefix + ".project.2", d)
        if spec.num_time_buckets > 0:
            table(prefix + ".time_embedding.weight", spec.num_time_buckets, d)
    num_ns += int(n_domains > 0)
    linear("sequence_stats_projector.0", 6, d)
    norm("sequence_stats_projector.2", d)
    hidden = d * spec.hidden_mult
    for layer in range(max(1, spec.num_blocks)):
        p = f"blocks.{layer}"
        norm(p + ".attn_norm", d, bias=False)
        linear(p + ".attention.shared_qkv", d, 3 * d)
        for n in "qkv":
            for i in range(num_ns):
                linear(f"{p}.attention.ns_{n}.{i}", d, d)
        linear(p + ".attention.out", d, d)
        norm(p + ".ffn_norm", d, bias=False)
        linear(p + ".ffn.shared.net.0", d, hidden)
        linear(p + ".ffn.shared.net.3", hidden, d)
        for i in range(num_ns):
            linear(f"{p}.ffn.ns_specific.{i}.net.0", d, hidden)
            linear(f"{p}.ffn.ns_specific.{i}.net.3", hidden, d)
    norm("final_norm", d, bias=False)
    linear("classifier.0", 2 * d, d)
    linear("classifier.3", d, spec.action_num)
    return sd


__all__ = [
    "OneTransInference",
    "deduplicate_sequence_events",
    "hash_compress_ids",
    "pyramid_keep_count",
    "random_state_dict",
    "score_stream",
    "sequence_stats",
    "sequence_time_buckets",
]
