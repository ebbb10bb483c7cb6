"""Runs the reference's own ``PCVROneTrans`` as the checker and the timed CPU baseline
(TEST / BENCHMARK INFRASTRUCTURE, never imported by the product).

The reference (package ``taac2026`` plus ``experiments/onetrans``) is found, in this order, as a source
checkout named by ``TAAC2026_REFERENCE``, as the archive of compiled modules under ``oracle/_ref`` (see
``oracle/build_ref.py``; imported through the small finder below), or as a sibling ``reference/`` checkout.  ``orjson``, which the reference only
uses to read and write JSON files (src/taac2026/infrastructure/io/json.py:8-41), is replaced by a
stdlib-backed stand-in when it is not installed.

``build_model`` constructs the unmodified ``PCVROneTrans`` (experiments/onetrans/model.py:110-359) for a
``OneTransSpec`` the way the reference's package tests do (tests/unit/experiments/test_packages.py:49-77):
singleton grouping, rank-mixer NS tokenizers, dropout 0.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import json
import marshal
import os
import sys
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REF_DIR = HERE / "_ref"
_state: dict[str, object] = {"kind": None}


def _install_orjson_stand_in() -> None:
    if "orjson" in sys.modules:
        return
    try:
        import orjson  # noqa: F401
        return
    except ImportError:
        pass
    shim = types.ModuleType("orjson")
    shim.OPT_INDENT_2, shim.OPT_SORT_KEYS, shim.OPT_SERIALIZE_NUMPY, shim.OPT_NON_STR_KEYS = 1, 2, 4, 8
    shim.dumps = lambda obj, default=None, option=0: json.dumps(
        obj, default=default, indent=2 if option & 1 else None, sort_keys=bool(option & 2)).encode()
    shim.loads = json.loads
    shim.JSONDecodeError = json.JSONDecodeError
    sys.modules["orjson"] = shim


class _ArchiveImporter(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Imports the modules of ``oracle/_ref/reference_modules.bin``: module name -> (is package, marshalled code)."""

    def __init__(self, archive: Path) -> None:
        self.archive = archive
        self.table: dict[str, tuple[bool, bytes]] = marshal.loads(archive.read_bytes())

    def find_spec(self, fullname, path=None, target=None):
        entry = self.table.get(fullname)
        if entry is None:
            return None
        return importlib.util.spec_from_loader(fullname, self, origin=f"{self.archive}:{fullname}", is_package=entry[0])

    def create_module(self, spec):
        return None

    def exec_module(self, module) -> None:
        is_package, blob = self.table[module.__name__]
        module.__file__ = f"{self.archive}:{module.__name__}"
        if is_package:
            module.__path__ = []
        exec(marshal.loads(blob), module.__dict__)


def locate() -> tuple[str, Path] | None:
    """-> ("checkout" | "compiled", path) of the first usable form of the reference, or None."""
    env = os.environ.get("TAAC2026_REFERENCE")
    if env and (Path(env) / "src" / "taac2026").is_dir():
        return "checkout", Path(env)
    info = REF_DIR / "BUILD_INFO.json"
    if info.exists():
        try:
            meta = json.loads(info.read_text())
            if meta.get("magic") == importlib.util.MAGIC_NUMBER.hex() and (REF_DIR / meta.get("archive", "")).is_file():
                return "compiled", REF_DIR / meta["archive"]
        except (OSError, ValueError):
            pass
    sibling = HERE.parent.parent / "reference"
    if (sibling / "src" / "taac2026").is_dir():
        return "checkout", sibling
    return None


def available() -> bool:
    return locate() is not None


def import_reference() -> str:
    """Make ``taac2026`` and ``experiments.onetrans`` importable; returns "checkout" or "compiled"."""
    if _state["kind"] is not None:
        return str(_state["kind"])
    found = locate()
    if found is None:
        raise RuntimeError("the reference is not available: no checkout and no oracle/_ref (python -m oracle.build_ref)")
    kind, path = found
    _install_orjson_stand_in()
    if kind == "checkout":
        for entry in (path / "src", path):
            if str(entry) not in sys.path:
                sys.path.insert(0, str(entry))
    else:
        sys.meta_path.insert(0, _ArchiveImporter(path))
    importlib.import_module("taac2026.infrastructure.accelerators")
    _state["kind"] = kind
    return kind


def schema_and_config(spec: dict, **config_overrides):
    """(PCVRSchema, PCVRModelConfig) that make the reference build the model a ``OneTransSpec`` describes."""
    import_reference()
    from taac2026.domain.config import PCVRModelConfig, PCVRNSConfig
    from taac2026.domain.schema import PCVRSchema

    def int_fields(specs, first_fid):
        return [[first_fid + i, int(vocab), int(length)] for i, (vocab, _offset, length) in enumerate(specs)]

    seq = {}
    for domain in sorted(spec["seq_vocab_sizes"]):
        vocabs = spec["seq_vocab_sizes"][domain]
        seq[domain] = {"prefix": domain, "ts_fid": 1, "features": [[1, 0]] + [[i + 2, int(v)] for i, v in enumerate(vocabs)]}
    schema = PCVRSchema(
        format="raw_parquet",
        user_int=int_fields(spec["user_int_specs"], 1),
        item_int=int_fields(spec["item_int_specs"], 1001),
        user_dense=[[1, int(spec["user_dense_dim"])]] if spec["user_dense_dim"] > 0 else [],
        item_dense=[[1001, int(spec["item_dense_dim"])]] if spec["item_dense_dim"] > 0 else [],
        seq=seq,
    )
    kwargs = dict(
        d_model=spec["d_model"], emb_dim=spec["emb_dim"], num_blocks=spec["num_blocks"], num_heads=spec["num_heads"],
        hidden_mult=spec["hidden_mult"], dropout_rate=0.0, use_time_buckets=spec["num_time_buckets"] > 0,
        seq_top_k=spec["seq_top_k"], emb_skip_threshold=spec["emb_skip_threshold"], action_num=spec["action_num"],
        ns=PCVRNSConfig(grouping_strategy="singleton", tokenizer_type="rankmixer" if spec["force_auto_split"] else "group",
                        user_tokens=spec["user_ns_tokens"], item_tokens=spec["item_ns_tokens"]),
    )
    kwargs.update(config_overrides)
    return schema, PCVRModelConfig(**kwargs)


def build_model(spec: dict, *, seed: int | None = 0, state_dict: dict | None = None, device: str = "cpu",
                meta_init: bool = False, **config_overrides):
    """The reference's ``PCVROneTrans`` in eval mode.  ``seed`` seeds its own initialisation
    (``torch.manual_seed(seed)`` before construction = "random-init weights from seed 0");
    ``state_dict`` (fp32 tensors with the module's parameter names) replaces the parameters afterwards.
    ``meta_init=True`` constructs the module without allocating or initialising parameters and then
    adopts the tensors of ``state_dict`` as they are (for multi-GB tables)."""
    import_reference()
    model_module = importlib.import_module("experiments.onetrans.model")
    schema, config = schema_and_config(spec, **config_overrides)
    # the two runtime switches, set from the configuration exactly as `build_prediction_model` does before it
    # constructs the model (src/taac2026/application/evaluation/workflow.py:116-129): RMSNorm modules capture
    # their backend at construction, attention reads its backend at call time
    from taac2026.infrastructure.modeling import normalization as m_norm
    from taac2026.infrastructure.modeling import sequence as m_seq

    m_seq.configure_flash_attention_runtime(backend=config.flash_attention_backend)
    m_norm.configure_rms_norm_runtime(backend=config.rms_norm_backend, block_rows=config.rms_norm_block_rows)
    if meta_init:
        if state_dict is None:
            raise ValueError("meta_init needs a state_dict")
        with torch.device("meta"):
            model = model_module.PCVROneTrans(schema=schema, config=config)
        model.load_state_dict(state_dict, assign=True, strict=True)
        return model.eval()
    if seed is not None:
        torch.manual_seed(seed)
    model = model_module.PCVROneTrans(schema=schema, config=config)
    if state_dict is not None:
        model.load_state_dict(state_dict, strict=True)
    return model.to(device).eval()


def model_input(batch):
    """``taac_2026_b200.inputs.ModelInput`` (or any record with the same attributes) -> ``PCVRModelInput``."""
    import_reference()
    from taac2026.infrastructure.data.batches import PCVREntityInput, PCVRModelInput, PCVRSequenceInput

    def entity(e):
        return PCVREntityInput(e.int_values, e.int_missing_mask, e.dense_values, e.dense_missing_mask)

    sequences = {name: PCVRSequenceInput(values=s.values, lengths=s.lengths, timestamps=s.timestamps)
                 for name, s in batch.sequences.items()}
    return PCVRModelInput(user=entity(batch.user), item=entity(batch.item), sequences=sequences,
                          request_timestamp=batch.request_timestamp)


@torch.no_grad()
def predict(model, batch) -> tuple[torch.Tensor, torch.Tensor]:
    """(logits, pooled embeddings) of ``PCVROneTrans.predict`` (experiments/onetrans/model.py:354-359)."""
    return model.predict(model_input(batch))


__all__ = ["available", "build_model", "import_reference", "locate", "model_input", "predict", "schema_and_config"]
