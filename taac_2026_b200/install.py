"""Teach an importable checkout of the reference (package ``taac2026``) the ``"cuda"`` backend.

``install()`` wraps the reference's four operator dispatchers and its two runtime switches so that
``backend="cuda"`` reaches ``taac_2026_b200.ops``; every other backend value goes to the original
function untouched.  Nothing in the reference checkout is edited; ``uninstall()`` restores the originals.

What is wrapped (paths relative to the reference root):

* dispatchers — ``rms_norm`` (src/taac2026/infrastructure/accelerators/normalization/rms_norm.py:377),
  ``layer_norm`` (.../normalization/layer_norm.py:261), ``flash_attention``
  (.../attention/flash_attention.py:871), ``embedding_bag_mean`` (.../embedding/embedding_bag.py:439),
  including the names the modeling modules imported from them
  (modeling/normalization.py:11-12, modeling/sequence.py:12, modeling/embeddings.py:8-10);
* switches — ``configure_rms_norm_runtime`` (modeling/normalization.py:17-25),
  ``configure_flash_attention_runtime`` (modeling/sequence.py:22-25) and the backend checks in
  ``RMSNorm.__init__`` / ``LayerNorm.__init__`` (modeling/normalization.py:30-43, :55-66);
* the registered-kernel hook of ``embedding_bag_mean`` (embedding_bag.py:77-79), because the shared
  model code calls it without a ``backend=`` argument (modeling/embeddings.py:32).

``install(route_all=True)`` additionally maps every backend the workflows configure
(evaluation/workflow.py:120-125) to ``"cuda"``, which is how an unmodified CLI run is switched over
while the Pydantic literal sets (domain/config.py:35-38) still only know the reference's own names.
"""

from __future__ import annotations

import importlib
from typing import Any

import torch

from taac_2026_b200 import ops

_originals: list[tuple[Any, str, Any]] = []
_state = {"installed": False, "route_all": False}


def _patch(obj: Any, name: str, new: Any) -> None:
    _originals.append((obj, name, getattr(obj, name)))
    setattr(obj, name, new)


def _modules() -> dict[str, Any]:
    names = {
        "rms": "taac2026.infrastructure.accelerators.normalization.rms_norm",
        "ln": "taac2026.infrastructure.accelerators.normalization.layer_norm",
        "fa": "taac2026.infrastructure.accelerators.attention.flash_attention",
        "bag": "taac2026.infrastructure.accelerators.embedding.embedding_bag",
        "acc": "taac2026.infrastructure.accelerators",
        "m_norm": "taac2026.infrastructure.modeling.normalization",
        "m_seq": "taac2026.infrastructure.modeling.sequence",
        "m_emb": "taac2026.infrastructure.modeling.embeddings",
    }
    try:
        return {key: importlib.import_module(path) for key, path in names.items()}
    except ImportError as error:  # pragma: no cover - depends on the environment
        raise RuntimeError(f"the reference package taac2026 is not importable: {error}") from error


def install(*, route_all: bool = False) -> None:
    """Route ``backend="cuda"`` of the reference's operators to this library (idempotent)."""
    if _state["installed"]:
        _state["route_all"] = bool(route_all)
        return
    mods = _modules()
    _state["route_all"] = bool(route_all)

    def pick(backend: str) -> str:
        return "cuda" if (_state["route_all"] or backend == "cuda") else backend

    # ---- dispatchers
    ref_rms, ref_ln = mods["rms"].rms_norm, mods["ln"].layer_norm
    ref_fa, ref_bag = mods["fa"].flash_attention, mods["bag"].embedding_bag_mean

    def rms_norm(x, weight, eps=1e-6, *, backend, block_rows=None):
        if pick(backend) == "cuda":
            return ops.rms_norm(x, weight, eps, backend="cuda", block_rows=block_rows)
        return ref_rms(x, weight, eps, backend=backend, block_rows=block_rows)

    def layer_norm(x, weight, bias, eps=1e-5, *, backend, block_rows=None):
        if pick(backend) == "cuda":
            return ops.layer_norm(x, weight, bias, eps, backend="cuda", block_rows=block_rows)
        return ref_ln(x, weight, bias, eps, backend=backend, block_rows=block_rows)

    def flash_attention(q, k, v, *, backend, **kwargs):
        if pick(backend) == "cuda":
            return ops.flash_attention(q, k, v, backend="cuda", **kwargs)
        return ref_fa(q, k, v, backend=backend, **kwargs)

    def embedding_bag_mean(embedding_weight, values, *, backend="torch", block_rows=None, block_cols=None):
        if backend == "cuda":
            return ops.embedding_bag_mean(embedding_weight, values, backend="cuda")
        return ref_bag(embedding_weight, values, backend=backend, block_rows=block_rows, block_cols=block_cols)

    for holder, name, fn in (
        (mods["rms"], "rms_norm", rms_norm), (mods["ln"], "layer_norm", layer_norm),
        (mods["fa"], "flash_attention", flash_attention), (mods["bag"], "embedding_bag_mean", embedding_bag_mean),
        (mods["acc"], "rms_norm", rms_norm), (mods["acc"], "layer_norm", layer_norm),
        (mods["acc"], "flash_attention", flash_attention), (mods["acc"], "embedding_bag_mean", embedding_bag_mean),
        (mods["m_norm"], "rms_norm", rms_norm), (mods["m_norm"], "layer_norm", layer_norm),
        (mods["m_seq"], "flash_attention", flash_attention), (mods["m_emb"], "embedding_bag_mean", embedding_bag_mean),
    ):
        if hasattr(holder, name):
            _patch(holder, name, fn)

    # ---- switches
    m_norm, m_seq = mods["m_norm"], mods["m_seq"]
    ref_cfg_rms, ref_cfg_fa = m_norm.configure_rms_norm_runtime, m_seq.configure_flash_attention_runtime

    def configure_rms_norm_runtime(*, backend: str, block_rows: int) -> None:
        if pick(backend) != "cuda":
            return ref_cfg_rms(backend=backend, block_rows=block_rows)
        if int(block_rows) < 1:
            raise ValueError("rms_norm block_rows must be positive")
        m_norm._RMS_NORM_BACKEND.set("cuda")
        m_norm._RMS_NORM_BLOCK_ROWS.set(int(block_rows))

    def configure_flash_attention_runtime(*, backend: str) -> None:
        if pick(backend) != "cuda":
            return ref_cfg_fa(backend=backend)
        m_seq._FLASH_ATTENTION_BACKEND.set("cuda")

    _patch(m_norm, "configure_rms_norm_runtime", configure_rms_norm_runtime)
    _patch(m_seq, "configure_flash_attention_runtime", configure_flash_attention_runtime)

    def wrap_init(cls, default_backend):
        ref_init = cls.__init__

        def __init__(self, dim, eps=None, *, backend=None, block_rows=None):
            chosen = default_backend() if backend is None else backend
            kwargs = {} if eps is None else {"eps": eps}
            if block_rows is not None:
                kwargs["block_rows"] = block_rows
            if pick(chosen) == "cuda":
                ref_init(self, dim, backend="torch", **kwargs)  # the reference's check only knows its own names
                self.backend = "cuda"
            else:
                ref_init(self, dim, backend=chosen, **kwargs)

        _patch(cls, "__init__", __init__)

    wrap_init(m_norm.RMSNorm, lambda: m_norm.rms_norm_runtime_state()[0])
    wrap_init(m_norm.LayerNorm, lambda: "torch")

    # ---- embedding hook: the only way unmodified model code reaches the CUDA gather
    def bag_hook(weight: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
        if weight.device.type == "cuda" and ops.cuda_available() and ops.cuda_supported_floating_dtype(weight.dtype):
            return ops.embedding_bag_mean(weight, values, backend="cuda")
        return mods["bag"]._torch_embedding_bag_mean(weight, values)

    _originals.append((mods["bag"], "_embedding_bag_mean_kernel", mods["bag"]._embedding_bag_mean_kernel))
    mods["bag"].register_embedding_bag_mean_kernel(bag_hook)
    _state["installed"] = True


def uninstall() -> None:
    """Put every wrapped attribute of the reference back."""
    while _originals:
        obj, name, value = _originals.pop()
        setattr(obj, name, value)
    _state["installed"] = False
    _state["route_all"] = False


def spec_from_reference(schema, config):
    """``OneTransSpec`` for a reference ``PCVRSchema`` + ``PCVRModelConfig`` (the arguments of
    `PCVROneTrans(schema, config)`, experiments/onetrans/model.py:111-146)."""
    from taac2026.infrastructure.modeling.model_contract import build_pcvr_model_specs
    from taac2026.infrastructure.modeling.time_features import NUM_TIME_BUCKETS

    from taac_2026_b200.inputs import OneTransSpec

    specs = build_pcvr_model_specs(schema, config.ns)
    return OneTransSpec(
        user_int_specs=[tuple(s) for s in specs.user_int_feature_specs],
        item_int_specs=[tuple(s) for s in specs.item_int_feature_specs],
        user_dense_dim=specs.user_dense_dim, item_dense_dim=specs.item_dense_dim,
        seq_vocab_sizes=dict(specs.seq_vocab_sizes), d_model=config.d_model, emb_dim=config.emb_dim,
        num_blocks=config.num_blocks, num_heads=config.num_heads, hidden_mult=config.hidden_mult,
        seq_top_k=config.seq_top_k, emb_skip_threshold=config.emb_skip_threshold,
        num_time_buckets=NUM_TIME_BUCKETS if config.use_time_buckets else 0,
        user_ns_tokens=config.ns.user_tokens, item_ns_tokens=config.ns.item_tokens,
        force_auto_split=config.ns.tokenizer_type == "rankmixer", action_num=config.action_num,
        user_ns_groups=[list(g) for g in specs.user_ns_groups], item_ns_groups=[list(g) for g in specs.item_ns_groups],
    )


__all__ = ["install", "spec_from_reference", "uninstall"]
