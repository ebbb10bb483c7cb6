"""Vectorised CPU port of the reference's torch path for the OneTrans forward — the TIMED CPU
baseline (TEST / BENCHMARK INFRASTRUCTURE, never imported by the product).

Where ``oracle/onetrans.py`` spells every step out with explicit loops so that it can serve as
the checker, this module computes the same forward the way the reference itself does on a CPU:
library calls (`F.embedding_bag`, `F.embedding`, `F.layer_norm`, `F.scaled_dot_product_attention`
with the dense bool mask of `causal_valid_attention_mask`, `F.linear`) over all host threads, one
Python-level loop per field and per NS token exactly as the reference modules have them
(modeling/embeddings.py:137-173, experiments/onetrans/model.py:58-107).  It is pinned to the same
golden fixtures as the loop oracle.  Tables may be stored in bf16 (rows are widened after the
gather), everything else runs in fp32.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle.onetrans import _table_kind, num_ns_tokens, pyramid_keep_count
from taac_2026_b200.onetrans import (  # device-agnostic integer preprocessing (plain tensor code)
    _BUCKET_EDGES,
    _SequenceSort,
    deduplicate_sequence_events,
    hash_compress_ids,
    sequence_stats,
    sequence_time_buckets,
)


def _lin(x, sd, prefix):
    return F.linear(x, sd[prefix + ".weight"].float(), sd[prefix + ".bias"].float())


def _ln(x, sd, prefix):
    return F.layer_norm(x, (x.shape[-1],), sd[prefix + ".weight"].float(), sd[prefix + ".bias"].float(), 1e-5)


def _rms(x, w, eps=1e-6):  # `_torch_rms_norm`, accelerators/normalization/rms_norm.py:71-73
    return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * w.float()


def _bank(sd, prefix, specs, threshold, compress, int_feats, emb):
    batch = int_feats.shape[0]
    if not specs:
        return torch.zeros(batch, 0, emb)
    tokens = []
    n_plain = n_comp = 0
    for vocab, offset, length in specs:  # the reference's per-field loop
        kind = _table_kind(vocab, threshold, compress)
        values = int_feats[:, offset : offset + length].to(torch.long)
        if kind == "table":
            table = sd[f"{prefix}.embeddings.{n_plain}.weight"]
            n_plain += 1
            values = values.clamp(min=0, max=int(vocab))
        elif kind == "compressed":
            table = sd[f"{prefix}.compressed_embeddings.{n_comp}.weight"]
            n_comp += 1
            values = hash_compress_ids(values.clamp(min=0), table.shape[0] - 1)
        else:
            tokens.append(torch.zeros(batch, emb))
            continue
        if table.dtype == torch.float32:
            tokens.append(F.embedding_bag(values, table, mode="mean", padding_idx=0))
        else:  # narrow tables: gather, widen, pool
            rows = F.embedding(values, table).float()
            valid = (values != 0).unsqueeze(-1)
            tokens.append((rows * valid).sum(dim=1) / valid.sum(dim=1).clamp_min(1))
    return torch.stack(tokens, dim=1)


def _ns_tokenizer(sd, prefix, specs, groups, spec, n_tokens, compress, int_feats, missing):
    d, emb = spec["d_model"], spec["emb_dim"]
    batch = int_feats.shape[0]
    feats = _bank(sd, prefix + ".bank", specs, spec["emb_skip_threshold"], compress, int_feats, emb)
    key = prefix + ".missing_embeddings"
    if key in sd and missing is not None and feats.shape[1] > 0:
        feats = feats + missing[:, : feats.shape[1]].float().unsqueeze(-1) * sd[key].float()[: feats.shape[1]].unsqueeze(0)
    groups = [list(g) for g in groups] or [[i] for i in range(len(specs))]
    n_tok = int(n_tokens) if n_tokens > 0 else len(groups)
    if n_tok <= 0:
        return torch.zeros(batch, 0, d)
    if bool(spec.get("force_auto_split", True)) or n_tok != len(groups):
        flat = feats.reshape(batch, -1) if feats.shape[1] > 0 else torch.zeros(batch, 1)
        return _ln(F.silu(_lin(flat, sd, prefix + ".project.0")), sd, prefix + ".project.2").view(batch, n_tok, d)
    grouped = [feats[:, [i for i in g if 0 <= i < feats.shape[1]], :].mean(dim=1) for g in groups]
    return _ln(_lin(torch.stack(grouped, dim=1), sd, prefix + ".project.0"), sd, prefix + ".project.1")


def _dense(sd, prefix, dim, values, missing):
    if dim <= 0:
        return None
    miss = torch.zeros_like(values) if missing is None else missing[:, : values.shape[1]].to(values.dtype)
    h = F.silu(_lin(torch.cat([values.float(), miss.float()], dim=-1), sd, prefix + ".project.0"))
    return _ln(h, sd, prefix + ".project.2").unsqueeze(1)


def _causal_valid_mask(padding_mask: torch.Tensor) -> torch.Tensor:  # modeling/sequence.py:119-127
    total = padding_mask.shape[1]
    causal = torch.ones(total, total, dtype=torch.bool).tril()
    mask = causal.unsqueeze(0) & (~padding_mask).unsqueeze(1)
    eye = torch.eye(total, dtype=torch.bool).unsqueeze(0)
    return torch.where(padding_mask.unsqueeze(-1), eye, mask).unsqueeze(1)


@torch.no_grad()
def predict(sd: dict, spec: dict, inputs) -> tuple[torch.Tensor, torch.Tensor]:
    d, heads = spec["d_model"], spec["num_heads"]
    if d % heads:
        heads = next(h for h in range(min(heads, d), 0, -1) if d % h == 0)
    domains = sorted(spec["seq_vocab_sizes"])
    num_ns = num_ns_tokens(spec)
    n_blocks = max(1, spec["num_blocks"])
    keep = max(1, int(spec["seq_top_k"]))
    batch = inputs.user.int_values.shape[0]
    edges = torch.tensor(_BUCKET_EDGES, dtype=torch.long)
    req = inputs.request_timestamp

    pieces, masks, stat_vecs = [], [], []
    for di, domain in enumerate(domains):
        seq = inputs.sequences[domain]
        sort = _SequenceSort(seq.values, seq.lengths)
        stats = sequence_stats(seq.values, seq.lengths, seq.timestamps, req, edges, sort)
        stat_vecs.append(_ln(F.silu(_lin(stats, sd, "sequence_stats_projector.0")), sd, "sequence_stats_projector.2"))
        values, lengths, ts = deduplicate_sequence_events(seq.values, seq.lengths, seq.timestamps, sort)
        seq_len = lengths.clamp(min=0, max=values.shape[2])
        prefix = f"sequence_tokenizers.{domain}"
        vocabs = spec["seq_vocab_sizes"][domain]
        cols = []
        n_plain = n_comp = 0
        for f in range(values.shape[1]):
            kind = _table_kind(vocabs[f], spec["emb_skip_threshold"], True) if f < len(vocabs) else "none"
            if kind == "table":
                table = sd[f"{prefix}.embeddings.{n_plain}.weight"]
                n_plain += 1
                cols.append(F.embedding(values[:, f].clamp(min=0, max=int(vocabs[f])), table).float())
            elif kind == "compressed":
                table = sd[f"{prefix}.compressed_embeddings.{n_comp}.weight"]
                n_comp += 1
                cols.append(F.embedding(hash_compress_ids(values[:, f].clamp(min=0), table.shape[0] - 1), table).float())
            else:
                cols.append(torch.zeros(batch, values.shape[2], spec["emb_dim"]))
        tokens = _ln(F.silu(_lin(torch.cat(cols, dim=-1), sd, prefix + ".project.0")), sd, prefix + ".project.2")
        if prefix + ".time_embedding.weight" in sd:
            table = sd[prefix + ".time_embedding.weight"].float()
            buckets = sequence_time_buckets(ts, req, edges).clamp(min=0, max=table.shape[0] - 1)
            tokens = tokens + F.embedding(buckets, table)
        if tokens.shape[1] > keep:  # tail crop, model.py:278-285
            start = (seq_len - keep).clamp_min(0)
            idx = (start[:, None] + torch.arange(keep)[None, :]).clamp_max(tokens.shape[1] - 1)
            tokens = tokens.gather(1, idx[:, :, None].expand(-1, -1, d))
        seq_len = seq_len.clamp_max(tokens.shape[1])
        length = tokens.shape[1]
        pos = torch.arange(length, dtype=torch.float32).unsqueeze(1)
        freq = torch.exp(torch.arange(0, d, 2, dtype=torch.float32) * (-torch.log(torch.tensor(10000.0)) / d))
        table = torch.zeros(length, d)
        table[:, 0::2] = torch.sin(pos * freq)
        table[:, 1::2] = torch.cos(pos * freq[: table[:, 1::2].shape[1]])
        pieces.append(tokens + table.unsqueeze(0))
        masks.append(torch.arange(length)[None, :] >= seq_len[:, None])
        if di < len(domains) - 1:
            pieces.append(sd["separator_tokens"].float()[di].view(1, 1, -1).expand(batch, -1, -1))
            masks.append(torch.zeros(batch, 1, dtype=torch.bool))
    seq_tokens = torch.cat(pieces, dim=1) if pieces else torch.zeros(batch, 0, d)
    seq_mask = torch.cat(masks, dim=1) if masks else torch.zeros(batch, 0, dtype=torch.bool)

    parts = [_ns_tokenizer(sd, "user_tokenizer", spec["user_int_specs"], spec.get("user_ns_groups", []), spec,
                           spec["user_ns_tokens"], False, inputs.user.int_values, inputs.user.int_missing_mask)]
    tok = _dense(sd, "user_dense", spec["user_dense_dim"], inputs.user.dense_values, inputs.user.dense_missing_mask)
    if tok is not None:
        parts.append(tok)
    parts.append(_ns_tokenizer(sd, "item_tokenizer", spec["item_int_specs"], spec.get("item_ns_groups", []), spec,
                               spec["item_ns_tokens"], True, inputs.item.int_values, inputs.item.int_missing_mask))
    tok = _dense(sd, "item_dense", spec["item_dense_dim"], inputs.item.dense_values, inputs.item.dense_missing_mask)
    if tok is not None:
        parts.append(tok)
    if stat_vecs:
        parts.append(torch.stack(stat_vecs, dim=1).mean(dim=1, keepdim=True))
    ns_tokens = torch.cat(parts, dim=1)

    tokens = torch.cat([seq_tokens, ns_tokens], dim=1)
    padding_mask = torch.cat([seq_mask, torch.zeros(batch, ns_tokens.shape[1], dtype=torch.bool)], dim=1)
    seq_count = seq_tokens.shape[1]
    hd = d // heads
    for layer in range(n_blocks):
        p = f"blocks.{layer}"
        total = tokens.shape[1]
        x = _rms(tokens, sd[p + ".attn_norm.weight"])
        q, k, v = (t.clone() for t in _lin(x, sd, p + ".attention.shared_qkv").chunk(3, dim=-1))
        for i in range(num_ns):  # the reference's per-NS-token loop, model.py:60-67
            pos_i = seq_count + i
            if pos_i >= total:
                continue
            q[:, pos_i] = _lin(x[:, pos_i], sd, f"{p}.attention.ns_q.{i}")
            k[:, pos_i] = _lin(x[:, pos_i], sd, f"{p}.attention.ns_k.{i}")
            v[:, pos_i] = _lin(x[:, pos_i], sd, f"{p}.attention.ns_v.{i}")
        split = lambda t: t.view(batch, total, heads, hd).transpose(1, 2)  # noqa: E731
        attn = F.scaled_dot_product_attention(split(q), split(k), split(v), attn_mask=_causal_valid_mask(padding_mask))
        tokens = tokens + _lin(attn.transpose(1, 2).reshape(batch, total, d), sd, p + ".attention.out")
        x = _rms(tokens, sd[p + ".ffn_norm.weight"])
        out = _lin(F.silu(_lin(x, sd, p + ".ffn.shared.net.0")), sd, p + ".ffn.shared.net.3")
        for i in range(num_ns):
            pos_i = seq_count + i
            if pos_i >= total:
                continue
            q_ = f"{p}.ffn.ns_specific.{i}"
            out[:, pos_i] = _lin(F.silu(_lin(x[:, pos_i], sd, q_ + ".net.0")), sd, q_ + ".net.3")
        tokens = tokens + out
        kc = pyramid_keep_count(seq_count, layer, n_blocks, num_ns)
        if kc < seq_count:
            tokens = torch.cat([tokens[:, seq_count - kc : seq_count], tokens[:, seq_count:]], dim=1)
            padding_mask = torch.cat([padding_mask[:, seq_count - kc : seq_count], padding_mask[:, seq_count:]], dim=1)
            seq_count = kc
    tokens = _rms(tokens, sd["final_norm.weight"])

    def masked_mean(t, m):
        if t.shape[1] == 0:
            return t.new_zeros(t.shape[0], t.shape[-1])
        valid = (~m).to(t.dtype).unsqueeze(-1)
        return (t * valid).sum(dim=1) / valid.sum(dim=1).clamp_min(1.0)

    emb = torch.cat([masked_mean(tokens[:, :seq_count], padding_mask[:, :seq_count]),
                     masked_mean(tokens[:, seq_count:], padding_mask[:, seq_count:])], dim=-1)
    return _lin(F.silu(_lin(emb, sd, "classifier.0")), sd, "classifier.3"), emb
