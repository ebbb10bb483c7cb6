"""Writes the golden fixtures in this directory by running the REFERENCE project's own code.

Run it only where the reference checkout is available (``--reference /path/to/TAAC_2026``);
the fixtures it writes (``*.npz``) are committed so that the tests need nothing but numpy.
Every array in a fixture is either a seeded input or the output of an unmodified reference
function on that input:

* ``ops.npz``       — `rms_norm`, `layer_norm`, `embedding_bag_mean`, `flash_attention` through
                      their ``backend="torch"`` dispatchers, the attention mask planner, and the
                      integer helpers (`hash_compress_ids`, `deduplicate_sequence_events`,
                      `compute_sequence_stats`, `compute_sequence_time_buckets`, `masked_mean`,
                      `sinusoidal_positions`, `causal_valid_attention_mask`, `binary_auc`).
* ``onetrans_a.npz`` / ``onetrans_b.npz`` — two small `PCVROneTrans` models (seed-0 weights):
                      state_dict, inputs, logits and pooled embeddings from `predict`.

The reference imports `orjson` for JSON file I/O only; where it is not installed an in-process
stand-in backed by the standard `json` module is registered first (no arithmetic involved).
"""

from __future__ import annotations

import argparse
import json
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def _import_reference(root: Path) -> None:
    try:
        import orjson  # noqa: F401
    except ImportError:
        shim = types.ModuleType("orjson")
        shim.OPT_INDENT_2, shim.OPT_SORT_KEYS, shim.OPT_SERIALIZE_NUMPY, shim.OPT_NON_STR_KEYS = 1, 2, 4, 8
        shim.dumps = lambda obj, default=None, option=0: json.dumps(obj, default=default, indent=2 if option & 1 else None).encode()
        shim.loads = json.loads
        shim.JSONDecodeError = json.JSONDecodeError
        sys.modules["orjson"] = shim
    for path in (root / "src", root):
        if str(path) not in sys.path:
            sys.path.insert(0, str(path))


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:  # numpy has no bf16: keep the raw 16-bit pattern
        return t.view(torch.int16).numpy()
    return t.numpy()


def make_ops(out: Path) -> None:
    from taac2026.domain.metrics import binary_auc
    from taac2026.infrastructure.accelerators import embedding_bag_mean, flash_attention, layer_norm, rms_norm
    from taac2026.infrastructure.accelerators.attention.flash_attention import _plan_tilelang_flash_attention_mask
    from taac2026.infrastructure.modeling.embeddings import hash_compress_ids
    from taac2026.infrastructure.modeling.sequence import (
        causal_valid_attention_mask,
        deduplicate_sequence_events,
        make_padding_mask,
        masked_mean,
        sinusoidal_positions,
    )
    from taac2026.infrastructure.modeling.time_features import compute_sequence_stats, compute_sequence_time_buckets

    g = torch.Generator().manual_seed(1234)
    arrays: dict[str, np.ndarray] = {}

    # ---- norms: fp32 and bf16, power-of-two and ragged widths, 1 % outlier rows
    for tag, cols, dtype in (("f32_96", 96, torch.float32), ("f32_128", 128, torch.float32),
                             ("bf16_128", 128, torch.bfloat16), ("bf16_400", 400, torch.bfloat16),
                             ("f32_127", 127, torch.float32)):
        x = torch.randn(37, cols, generator=g)
        x[::11] *= 50.0
        w = 1.0 + 0.02 * torch.randn(cols, generator=g)
        b = 0.02 * torch.randn(cols, generator=g)
        x, w, b = x.to(dtype), w.to(dtype), b.to(dtype)
        arrays[f"norm_{tag}_x"], arrays[f"norm_{tag}_w"], arrays[f"norm_{tag}_b"] = _np(x), _np(w), _np(b)
        arrays[f"norm_{tag}_rms"] = _np(rms_norm(x, w, 1e-6, backend="torch"))
        arrays[f"norm_{tag}_ln"] = _np(layer_norm(x, w, b, 1e-6, backend="torch"))

    # ---- bag mean: padding ids, empty bags, bag of one
    table = torch.randn(53, 16, generator=g)
    table[0] = 0
    ids = torch.randint(0, 53, (29, 5), generator=g)
    ids[ids % 4 == 0] = 0
    ids[3] = 0
    arrays["bag_table"], arrays["bag_ids"] = _np(table), _np(ids)
    arrays["bag_out"] = _np(embedding_bag_mean(table, ids, backend="torch"))
    ids1 = torch.randint(0, 53, (31, 1), generator=g)
    arrays["bag1_ids"] = _np(ids1)
    arrays["bag1_out"] = _np(embedding_bag_mean(table, ids1, backend="torch"))

    # ---- attention through the torch dispatcher with the three mask families
    B, H, T, D = 3, 2, 24, 16
    q, k, v = (torch.randn(B, H, T, D, generator=g) / 4 for _ in range(3))
    lens = torch.tensor([24, 7, 13])
    arrays["attn_q"], arrays["attn_k"], arrays["attn_v"], arrays["attn_lens"] = _np(q), _np(k), _np(v), _np(lens)
    pad = make_padding_mask(lens, T)
    key_mask = (~pad)[:, None, None, :].expand(B, H, T, T)
    arrays["attn_out_keypad"] = _np(flash_attention(q, k, v, backend="torch", attn_mask=key_mask))
    plan = _plan_tilelang_flash_attention_mask(q, k, key_mask, is_causal=False)
    arrays["plan_keypad_lengths"] = _np(plan.key_lengths)
    arrays["attn_out_causal_nomask"] = _np(flash_attention(q, k, v, backend="torch", is_causal=True))
    cv = causal_valid_attention_mask(pad, H)
    arrays["attn_mask_causal_valid"] = _np(cv[:, 0])
    arrays["attn_out_causal_valid"] = _np(flash_attention(q, k, v, backend="torch", attn_mask=cv))
    plan = _plan_tilelang_flash_attention_mask(q, k, cv, is_causal=False)
    arrays["plan_causal_valid_lengths"] = _np(plan.key_lengths)
    arrays["plan_causal_valid_self"] = _np(plan.query_self_mask)
    ns = 5  # OneTrans layout: [sequence (prefix valid) | ns always-valid tokens]
    seq_lens = torch.tensor([19, 4, 0])
    pad_ns = torch.cat([make_padding_mask(seq_lens, T - ns), torch.zeros(B, ns, dtype=torch.bool)], dim=1)
    cv_ns = causal_valid_attention_mask(pad_ns, H)
    arrays["attn_ns_seq_lens"] = _np(seq_lens)
    arrays["attn_mask_ns"] = _np(cv_ns[:, 0])
    arrays["attn_out_ns"] = _np(flash_attention(q, k, v, backend="torch", attn_mask=cv_ns))

    # ---- integer helpers
    vals = torch.randint(-3, 40, (6, 17), generator=g)
    arrays["hash_in"] = _np(vals)
    arrays["hash_out_7"] = _np(hash_compress_ids(vals, 7))
    arrays["hash_out_0"] = _np(hash_compress_ids(vals, 0))

    Bq, Fq, Lq = 9, 2, 12
    seq = torch.randint(0, 4, (Bq, Fq, Lq), generator=g)
    seq_lengths = torch.tensor([12, 0, 1, 5, 12, 9, 3, 20, -2])
    ts = torch.randint(1, 10_000_000, (Bq, Lq), generator=g)
    ts[:, ::5] = 0
    req = torch.randint(5_000_000, 40_000_000, (Bq,), generator=g)
    arrays["seq_values"], arrays["seq_lengths"], arrays["seq_ts"], arrays["seq_req"] = _np(seq), _np(seq_lengths), _np(ts), _np(req)
    dv, dl, dt = deduplicate_sequence_events(seq, seq_lengths, ts)
    arrays["dedup_values"], arrays["dedup_lengths"], arrays["dedup_ts"] = _np(dv), _np(dl), _np(dt)
    arrays["seq_stats"] = _np(compute_sequence_stats(seq, seq_lengths, ts, req))
    arrays["seq_buckets"] = _np(compute_sequence_time_buckets(ts, req))
    gaps = torch.tensor([[0, 1, 4, 5, 6, 60, 61, 3600, 3601, 31536000, 31536001, 10**10]])
    arrays["bucket_edge_gaps"] = _np(gaps)
    arrays["bucket_edge_out"] = _np(compute_sequence_time_buckets(10**11 - gaps, torch.tensor([10**11])))

    tok = torch.randn(4, 6, 8, generator=g)
    pm = make_padding_mask(torch.tensor([6, 0, 3, 1]), 6)
    arrays["mm_tokens"], arrays["mm_mask"], arrays["mm_out"] = _np(tok), _np(pm), _np(masked_mean(tok, pm))
    arrays["sinus_9_16"] = _np(sinusoidal_positions(9, 16, torch.device("cpu")))

    labels = (torch.rand(200, generator=g) < 0.3).numpy().astype(np.float64)
    scores = torch.round(torch.rand(200, generator=g) * 50).numpy() / 50.0  # ties on purpose
    arrays["auc_labels"], arrays["auc_scores"] = labels, scores
    arrays["auc_value"] = np.array(binary_auc(labels, scores))

    np.savez_compressed(out, **arrays)
    print(f"wrote {out} ({out.stat().st_size} bytes, {len(arrays)} arrays)")


def make_onetrans(out: Path, root: Path, variant: str) -> None:
    from taac2026.domain.config import PCVRModelConfig, PCVRNSConfig
    from taac2026.domain.schema import PCVRSchema
    from taac2026.infrastructure.data.batches import PCVREntityInput, PCVRModelInput, PCVRSequenceInput
    from taac2026.infrastructure.experiments.module_loader import load_experiment_submodule
    from taac2026.infrastructure.modeling.model_contract import build_pcvr_model_specs

    model_module = load_experiment_submodule(root / "experiments" / "onetrans", "model")
    g = torch.Generator().manual_seed(99 if variant == "a" else 7)
    if variant == "a":  # the C1 shape in miniature: one id per field, one domain, no time buckets
        schema = PCVRSchema(
            format="raw_parquet",
            user_int=[[i + 1, 40 + i, 1] for i in range(4)],
            item_int=[[i + 10, 30, 1] for i in range(2)],
            user_dense=[[1, 4]],
            item_dense=[],
            seq={"seq_a": {"prefix": "seq_a", "ts_fid": 1, "features": [[1, 0], [2, 90]]}},
        )
        config = PCVRModelConfig(
            d_model=64, emb_dim=16, num_blocks=2, num_heads=2, hidden_mult=4, dropout_rate=0.0,
            use_time_buckets=False, seq_top_k=40, emb_skip_threshold=0,
            ns=PCVRNSConfig(grouping_strategy="singleton", tokenizer_type="rankmixer", user_tokens=2, item_tokens=1),
        )
        B, lens = 6, {"seq_a": (40, torch.tensor([40, 1, 17, 0, 33, 8]))}
    else:  # multi-id fields, two domains, time buckets, hashed high-cardinality tables, tail crop
        schema = PCVRSchema(
            format="raw_parquet",
            user_int=[[1, 25, 3], [2, 300, 1], [3, 12, 2]],
            item_int=[[7, 500, 2], [8, 9, 1]],
            user_dense=[[1, 3], [2, 2]],
            item_dense=[[5, 2]],
            seq={
                "seq_a": {"prefix": "seq_a", "ts_fid": 1, "features": [[1, 0], [2, 60], [3, 400]]},
                "seq_b": {"prefix": "seq_b", "ts_fid": 4, "features": [[4, 0], [5, 20]]},
            },
        )
        config = PCVRModelConfig(
            d_model=64, emb_dim=8, num_blocks=3, num_heads=2, hidden_mult=2, dropout_rate=0.0,
            use_time_buckets=True, seq_top_k=10, emb_skip_threshold=100,
            ns=PCVRNSConfig(grouping_strategy="singleton", tokenizer_type="rankmixer", user_tokens=3, item_tokens=2),
        )
        B, lens = 5, {"seq_a": (14, torch.tensor([14, 3, 0, 9, 12])), "seq_b": (6, torch.tensor([2, 6, 6, 0, 1]))}

    torch.manual_seed(0)
    model = model_module.PCVROneTrans(schema=schema, config=config).eval()
    specs = build_pcvr_model_specs(schema, config.ns)

    def entity(int_specs, dense_dim):
        cols = max(off + ln for _v, off, ln in int_specs)
        ints = torch.zeros(B, cols, dtype=torch.long)
        for vocab, off, ln in int_specs:
            ints[:, off : off + ln] = torch.randint(0, vocab + 3, (B, ln), generator=g)  # some ids beyond vocab: clamp path
        miss = torch.rand(B, cols, generator=g) < 0.2
        dense = torch.randn(B, dense_dim, generator=g)
        dmiss = torch.rand(B, dense_dim, generator=g) < 0.2
        return PCVREntityInput(ints, miss, dense, dmiss)

    user = entity(specs.user_int_feature_specs, specs.user_dense_dim)
    item = entity(specs.item_int_feature_specs, specs.item_dense_dim)
    req = torch.randint(20_000_000, 30_000_000, (B,), generator=g)
    sequences = {}
    for domain, vocabs in specs.seq_vocab_sizes.items():
        L, lengths = lens[domain]
        values = torch.zeros(B, len(vocabs), L, dtype=torch.long)
        for f, vocab in enumerate(vocabs):
            values[:, f] = torch.randint(1, min(vocab, 6) + 1, (B, L), generator=g)  # few distinct ids: duplicates
        values = torch.where((torch.arange(L)[None] < lengths[:, None])[:, None, :], values, torch.zeros_like(values))
        ts = req[:, None] - torch.randint(1, 5_000_000, (B, L), generator=g)
        ts = torch.where(torch.arange(L)[None] < lengths[:, None], ts, torch.zeros_like(ts))
        if variant == "a":
            ts = torch.zeros_like(ts)
        sequences[domain] = PCVRSequenceInput(values=values, lengths=lengths, timestamps=ts)
    inputs = PCVRModelInput(user=user, item=item, sequences=sequences, request_timestamp=req)
    with torch.no_grad():
        logits, embeddings = model.predict(inputs)

    arrays = {f"sd/{name}": _np(t) for name, t in model.state_dict().items()}
    spec = {
        "user_int_specs": [list(s) for s in specs.user_int_feature_specs],
        "item_int_specs": [list(s) for s in specs.item_int_feature_specs],
        "user_dense_dim": specs.user_dense_dim, "item_dense_dim": specs.item_dense_dim,
        "seq_vocab_sizes": specs.seq_vocab_sizes, "d_model": config.d_model, "emb_dim": config.emb_dim,
        "num_blocks": config.num_blocks, "num_heads": config.num_heads, "hidden_mult": config.hidden_mult,
        "seq_top_k": config.seq_top_k, "emb_skip_threshold": config.emb_skip_threshold,
        "num_time_buckets": model.sequence_tokenizers[sorted(specs.seq_vocab_sizes)[0]].time_embedding.num_embeddings
        if config.use_time_buckets else 0,
        "user_ns_tokens": config.ns.user_tokens, "item_ns_tokens": config.ns.item_tokens, "force_auto_split": True,
        "user_ns_groups": specs.user_ns_groups, "item_ns_groups": specs.item_ns_groups, "action_num": config.action_num,
    }
    arrays["spec_json"] = np.frombuffer(json.dumps(spec).encode(), dtype=np.uint8)
    for name, ent in (("user", user), ("item", item)):
        arrays[f"in/{name}/int_values"] = _np(ent.int_values)
        arrays[f"in/{name}/int_missing_mask"] = _np(ent.int_missing_mask)
        arrays[f"in/{name}/dense_values"] = _np(ent.dense_values)
        arrays[f"in/{name}/dense_missing_mask"] = _np(ent.dense_missing_mask)
    for domain, seq in sequences.items():
        arrays[f"in/seq/{domain}/values"] = _np(seq.values)
        arrays[f"in/seq/{domain}/lengths"] = _np(seq.lengths)
        arrays[f"in/seq/{domain}/timestamps"] = _np(seq.timestamps)
    arrays["in/request_timestamp"] = _np(req)
    arrays["out/logits"], arrays["out/embeddings"] = _np(logits), _np(embeddings)
    np.savez_compressed(out, **arrays)
    print(f"wrote {out} ({out.stat().st_size} bytes); logits {logits.flatten().tolist()}")


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--reference", type=Path, required=True, help="root of the reference checkout")
    args = parser.parse_args()
    _import_reference(args.reference)
    torch.set_num_threads(1)  # deterministic reduction order
    make_ops(HERE / "ops.npz")
    make_onetrans(HERE / "onetrans_a.npz", args.reference, "a")
    make_onetrans(HERE / "onetrans_b.npz", args.reference, "b")


if __name__ == "__main__":
    main()
