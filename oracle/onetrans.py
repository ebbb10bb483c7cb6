"""fp32 CPU restatement of `PCVROneTrans.predict` (experiments/onetrans/model.py:110-359).

TEST INFRASTRUCTURE: a functional forward over a plain ``state_dict`` (parameter names as the
reference module tree produces them) with dense [B, T, T] masks and padded [B, T, d] tensors —
no kernels, no packing, no fusion.  It is pinned against logits and pooled embeddings computed
by the reference model itself (``tests/golden/onetrans_*.npz``).

``spec`` is a plain dict:
    user_int_specs / item_int_specs : [(vocab, offset, length), ...]   (model_contract.py:26-31)
    user_dense_dim / item_dense_dim : int
    seq_vocab_sizes                 : {domain: [vocab per feature]}
    d_model, emb_dim, num_blocks, num_heads, hidden_mult, seq_top_k, emb_skip_threshold,
    num_time_buckets, user_ns_tokens, item_ns_tokens, force_auto_split (bool),
    user_ns_groups / item_ns_groups : [[field index, ...], ...]
``inputs`` is any object shaped like the reference's `PCVRModelInput`
(src/taac2026/infrastructure/data/batches.py:17-69).
"""

from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from oracle import reference_ops as R


def _linear(x: torch.Tensor, sd: dict, prefix: str) -> torch.Tensor:
    return F.linear(x, sd[prefix + ".weight"].float(), sd[prefix + ".bias"].float())


def _layer_norm(x: torch.Tensor, sd: dict, prefix: str) -> torch.Tensor:
    return R.layer_norm_fp32(x, sd[prefix + ".weight"], sd[prefix + ".bias"], 1e-5)


def _table_kind(vocab: int, threshold: int, compress: bool) -> str:
    """Which table a feature owns (modeling/embeddings.py:99-127, tokenizers.py:125-139)."""
    if int(vocab) <= 0:
        return "none"
    if threshold > 0 and int(vocab) > threshold:
        return "compressed" if compress else "none"
    return "table"


def _bank(sd: dict, prefix: str, specs, threshold: int, compress: bool, int_feats: torch.Tensor, emb: int):
    tables, compressed = [], []
    n_plain = n_comp = 0
    for vocab, _off, _len in specs:
        kind = _table_kind(vocab, threshold, compress)
        if kind == "table":
            tables.append(sd[f"{prefix}.embeddings.{n_plain}.weight"].float())
            compressed.append(False)
            n_plain += 1
        elif kind == "compressed":
            tables.append(sd[f"{prefix}.compressed_embeddings.{n_comp}.weight"].float())
            compressed.append(True)
            n_comp += 1
        else:
            tables.append(None)
            compressed.append(False)
    if not specs:
        return torch.zeros(int_feats.shape[0], 0, emb)
    if all(t is None for t in tables):
        return torch.zeros(int_feats.shape[0], len(specs), emb)
    return R.feature_bank(tables, list(specs), int_feats, compressed)


def _ns_tokenizer(sd: dict, prefix: str, specs, groups, spec: dict, num_tokens: int, compress: bool,
                  int_feats: torch.Tensor, missing: torch.Tensor | None) -> torch.Tensor:
    """`NonSequentialTokenizer.forward` (modeling/tokenizers.py:63-87)."""
    d, emb = spec["d_model"], spec["emb_dim"]
    batch = int_feats.shape[0]
    feats = _bank(sd, prefix + ".bank", specs, spec["emb_skip_threshold"], compress, int_feats, emb)
    key = prefix + ".missing_embeddings"
    if key in sd and missing is not None and feats.shape[1] > 0:
        m = missing[:, : feats.shape[1]].float()
        feats = feats + m.unsqueeze(-1) * sd[key].float()[: feats.shape[1]].unsqueeze(0)
    groups = [list(g) for g in groups] or [[i] for i in range(len(specs))]
    n_tok = int(num_tokens) if num_tokens > 0 else len(groups)
    if n_tok <= 0:
        return torch.zeros(batch, 0, d)
    auto_split = bool(spec.get("force_auto_split", True)) or n_tok != len(groups)
    if auto_split:
        flat = feats.reshape(batch, -1) if feats.shape[1] > 0 else torch.zeros(batch, 1)
        h = F.silu(_linear(flat, sd, prefix + ".project.0"))
        return _layer_norm(h, sd, prefix + ".project.2").view(batch, n_tok, d)
    grouped = []
    for g in groups:
        idx = [i for i in g if 0 <= i < feats.shape[1]]
        grouped.append(feats[:, idx, :].mean(dim=1) if idx else torch.zeros(batch, emb))
    h = _linear(torch.stack(grouped, dim=1), sd, prefix + ".project.0")
    return _layer_norm(h, sd, prefix + ".project.1")


def _dense_token(sd: dict, prefix: str, dim: int, values: torch.Tensor, missing: torch.Tensor | None):
    """`DenseTokenProjector.forward` (modeling/tokenizers.py:101-111)."""
    if dim <= 0:
        return None
    miss = torch.zeros_like(values) if missing is None else missing[:, : values.shape[1]].to(values.dtype)
    h = F.silu(_linear(torch.cat([values.float(), miss.float()], dim=-1), sd, prefix + ".project.0"))
    return _layer_norm(h, sd, prefix + ".project.2").unsqueeze(1)


def _sequence_tokens(sd: dict, prefix: str, vocabs, spec: dict, values: torch.Tensor, timestamps: torch.Tensor,
                     request_ts: torch.Tensor) -> torch.Tensor:
    """`SequenceTokenizer.forward` (modeling/tokenizers.py:156-190)."""
    batch, n_feat, length = values.shape
    emb = spec["emb_dim"]
    pieces = []
    n_plain = n_comp = 0
    for f in range(n_feat):
        kind = _table_kind(vocabs[f], spec["emb_skip_threshold"], True) if f < len(vocabs) else "none"
        if kind == "table":
            table = sd[f"{prefix}.embeddings.{n_plain}.weight"].float()
            n_plain += 1
            pieces.append(R.gather_rows(table, values[:, f, :].clamp(min=0, max=int(vocabs[f]))))
        elif kind == "compressed":
            table = sd[f"{prefix}.compressed_embeddings.{n_comp}.weight"].float()
            n_comp += 1
            ids = R.hash_compress_ids(values[:, f, :].clamp(min=0).numpy(), table.shape[0] - 1)
            pieces.append(R.gather_rows(table, torch.from_numpy(ids)))
        else:
            pieces.append(torch.zeros(batch, length, emb))
    token_input = torch.cat(pieces, dim=-1) if pieces else torch.zeros(batch, length, 1)
    h = F.silu(_linear(token_input, sd, prefix + ".project.0"))
    tokens = _layer_norm(h, sd, prefix + ".project.2")
    key = prefix + ".time_embedding.weight"
    if key in sd:
        buckets = R.sequence_time_buckets(timestamps.numpy(), request_ts.numpy())
        table = sd[key].float()
        tokens = tokens + table[torch.from_numpy(buckets).clamp(min=0, max=table.shape[0] - 1)]
    return tokens


def _tail_crop(tokens: torch.Tensor, lengths: torch.Tensor, keep: int) -> torch.Tensor:
    """Keep the last `keep` valid positions of each row (experiments/onetrans/model.py:278-285)."""
    if tokens.shape[1] <= keep:
        return tokens
    out = torch.empty(tokens.shape[0], keep, tokens.shape[2])
    for b in range(tokens.shape[0]):
        start = max(int(lengths[b]) - keep, 0)
        for j in range(keep):
            out[b, j] = tokens[b, min(start + j, tokens.shape[1] - 1)]
    return out


def pyramid_keep_count(seq_tokens: int, layer: int, n_layers: int, num_ns: int) -> int:
    """Sequence positions kept after block `layer` (experiments/onetrans/model.py:317-323)."""
    if seq_tokens <= max(1, num_ns):
        return seq_tokens
    remaining = max(1, n_layers - layer)
    target = max(1, num_ns)
    decay = (target / seq_tokens) ** (1.0 / remaining)
    return max(target, min(seq_tokens, math.ceil(seq_tokens * decay)))


def _block(sd: dict, p: str, tokens: torch.Tensor, padding_mask: torch.Tensor, seq_count: int, heads: int,
           num_ns: int) -> torch.Tensor:
    """`OneTransBlock.forward` (experiments/onetrans/model.py:97-107) with its mixed attention
    (:47-78) and mixed FFN (:81-94)."""
    batch, total, d = tokens.shape
    x = R.rms_norm_fp32(tokens, sd[p + ".attn_norm.weight"], 1e-6)
    q, k, v = (part.clone() for part in _linear(x, sd, p + ".attention.shared_qkv").chunk(3, dim=-1))
    for i in range(num_ns):
        pos = seq_count + i
        if pos >= total:
            continue
        q[:, pos] = _linear(x[:, pos], sd, f"{p}.attention.ns_q.{i}")
        k[:, pos] = _linear(x[:, pos], sd, f"{p}.attention.ns_k.{i}")
        v[:, pos] = _linear(x[:, pos], sd, f"{p}.attention.ns_v.{i}")
    hd = d // heads
    split = lambda t: t.view(batch, total, heads, hd).transpose(1, 2)  # noqa: E731
    mask = R.causal_valid_attention_mask(padding_mask).unsqueeze(1)
    attn = R.attention(split(q), split(k), split(v), mask).transpose(1, 2).reshape(batch, total, d)
    tokens = tokens + _linear(attn, sd, p + ".attention.out")

    x = R.rms_norm_fp32(tokens, sd[p + ".ffn_norm.weight"], 1e-6)
    ffn = lambda t, q_: R.silu_ffn(  # noqa: E731
        t, sd[q_ + ".net.0.weight"], sd[q_ + ".net.0.bias"], sd[q_ + ".net.3.weight"], sd[q_ + ".net.3.bias"]
    )
    out = ffn(x, p + ".ffn.shared")
    for i in range(num_ns):
        pos = seq_count + i
        if pos >= total:
            continue
        out[:, pos] = ffn(x[:, pos], f"{p}.ffn.ns_specific.{i}")
    return tokens + out


def num_ns_tokens(spec: dict) -> int:
    """NS token count (experiments/onetrans/model.py:221-224)."""

    def tok(n_tokens: int, groups, specs) -> int:
        groups = list(groups) or [[i] for i in range(len(specs))]
        return int(n_tokens) if n_tokens > 0 else len(groups)

    n = tok(spec["user_ns_tokens"], spec.get("user_ns_groups", []), spec["user_int_specs"])
    n += tok(spec["item_ns_tokens"], spec.get("item_ns_groups", []), spec["item_int_specs"])
    n += int(spec["user_dense_dim"] > 0) + int(spec["item_dense_dim"] > 0)
    n += int(bool(spec["seq_vocab_sizes"]))
    return n


@torch.no_grad()
def predict(sd: dict, spec: dict, inputs) -> tuple[torch.Tensor, torch.Tensor]:
    """(logits [B, action_num], pooled embeddings [B, 2 d]) — `PCVROneTrans.predict` (:357-359)."""
    d = spec["d_model"]
    heads = spec["num_heads"]
    if d % heads != 0:  # choose_num_heads (modeling/sequence.py:70-78)
        heads = next(h for h in range(min(heads, d), 0, -1) if d % h == 0)
    domains = sorted(spec["seq_vocab_sizes"])
    num_ns = num_ns_tokens(spec)
    n_blocks = max(1, spec["num_blocks"])
    keep = max(1, int(spec["seq_top_k"]))
    batch = inputs.user.int_values.shape[0]

    # ---- sequence stream (:287-315)
    pieces, masks = [], []
    for di, domain in enumerate(domains):
        seq = inputs.sequences[domain]
        values, lengths, ts = R.deduplicate_sequence_events(seq.values.numpy(), seq.lengths.numpy(), seq.timestamps.numpy())
        values, lengths, ts = torch.from_numpy(values), torch.from_numpy(lengths), torch.from_numpy(ts)
        seq_len = lengths.clamp_min(0).clamp_max(values.shape[2])
        tokens = _sequence_tokens(sd, f"sequence_tokenizers.{domain}", spec["seq_vocab_sizes"][domain], spec, values, ts,
                                  inputs.request_timestamp)
        tokens = _tail_crop(tokens, seq_len, keep)
        seq_len = seq_len.clamp_max(tokens.shape[1])
        tokens = tokens + R.sinusoidal_positions(tokens.shape[1], d).unsqueeze(0)
        pieces.append(tokens)
        masks.append(R.make_padding_mask(seq_len, tokens.shape[1]))
        if di < len(domains) - 1:
            pieces.append(sd["separator_tokens"].float()[di].view(1, 1, -1).expand(batch, -1, -1))
            masks.append(torch.zeros(batch, 1, dtype=torch.bool))
    if pieces:
        seq_tokens, seq_mask = torch.cat(pieces, dim=1), torch.cat(masks, dim=1)
    else:
        seq_tokens, seq_mask = torch.zeros(batch, 0, d), torch.zeros(batch, 0, dtype=torch.bool)

    # ---- non-sequence tokens (:240-252)
    parts = [_ns_tokenizer(sd, "user_tokenizer", spec["user_int_specs"], spec.get("user_ns_groups", []), spec,
                           spec["user_ns_tokens"], False, inputs.user.int_values, inputs.user.int_missing_mask)]
    tok = _dense_token(sd, "user_dense", spec["user_dense_dim"], inputs.user.dense_values, inputs.user.dense_missing_mask)
    if tok is not None:
        parts.append(tok)
    parts.append(_ns_tokenizer(sd, "item_tokenizer", spec["item_int_specs"], spec.get("item_ns_groups", []), spec,
                               spec["item_ns_tokens"], True, inputs.item.int_values, inputs.item.int_missing_mask))
    tok = _dense_token(sd, "item_dense", spec["item_dense_dim"], inputs.item.dense_values, inputs.item.dense_missing_mask)
    if tok is not None:
        parts.append(tok)
    if domains:  # sequence statistics token (:254-276): RAW (not deduplicated) sequences
        vecs = []
        for domain in domains:
            seq = inputs.sequences[domain]
            stats = torch.from_numpy(R.sequence_stats(seq.values.numpy(), seq.lengths.numpy(), seq.timestamps.numpy(),
                                                      inputs.request_timestamp.numpy()))
            h = F.silu(_linear(stats, sd, "sequence_stats_projector.0"))
            vecs.append(_layer_norm(h, sd, "sequence_stats_projector.2"))
        parts.append(torch.stack(vecs, dim=1).mean(dim=1, keepdim=True))
    ns_tokens = torch.cat(parts, dim=1)

    # ---- blocks with pyramid shrink (:325-352)
    tokens = torch.cat([seq_tokens, ns_tokens], dim=1)
    padding_mask = torch.cat([seq_mask, torch.zeros(batch, ns_tokens.shape[1], dtype=torch.bool)], dim=1)
    seq_count = seq_tokens.shape[1]
    for layer in range(n_blocks):
        tokens = _block(sd, f"blocks.{layer}", tokens, padding_mask, seq_count, heads, num_ns)
        kc = pyramid_keep_count(seq_count, layer, n_blocks, num_ns)
        if kc < seq_count:
            tokens = torch.cat([tokens[:, seq_count - kc : seq_count], tokens[:, seq_count:]], dim=1)
            padding_mask = torch.cat([padding_mask[:, seq_count - kc : seq_count], padding_mask[:, seq_count:]], dim=1)
            seq_count = kc
    tokens = R.rms_norm_fp32(tokens, sd["final_norm.weight"], 1e-6)
    seq_summary = R.masked_mean(tokens[:, :seq_count], padding_mask[:, :seq_count])
    ns_summary = R.masked_mean(tokens[:, seq_count:], padding_mask[:, seq_count:])
    embeddings = torch.cat([seq_summary, ns_summary], dim=-1)
    h = F.silu(_linear(embeddings, sd, "classifier.0"))
    return _linear(h, sd, "classifier.3"), embeddings


def sigmoid_scores(logits: torch.Tensor) -> np.ndarray:
    """`sigmoid_probabilities_numpy` (src/taac2026/infrastructure/modeling/tensors.py:9-10)."""
    return torch.sigmoid(logits.float()).cpu().numpy()
