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

* the backend literal of the configuration — ``RMSNormBackend`` / ``FlashAttentionBackend``,
  ``RMS_NORM_BACKEND_CHOICES`` / ``FLASH_ATTENTION_BACKEND_CHOICES`` and the two field validators of
  ``PCVRModelConfig`` (domain/config.py:35-38, :309-321) — so that
  ``PCVRModelConfig(rms_norm_backend="cuda", flash_attention_backend="cuda")`` and
  ``--model.rms_norm_backend cuda`` validate;
* ``resolved_rms_norm_backend`` / ``resolved_layer_norm_backend`` / ``resolved_flash_attention_backend`` /
  ``resolved_embedding_bag_mean_backend`` in every namespace that exports them, and the operator benchmark
  (application/benchmarking/pcvr_tilelang_ops_benchmark.py:20-38, :123-130, :253-430): ``cuda`` joins its
  ``SUPPORTED_BACKENDS`` and its four ``_prepare_*_callable`` helpers hand out this library's kernels for it, so
  ``taac-benchmark-pcvr-tilelang-ops --backends torch,cuda`` times them next to the reference's own.

``install(route_all=True)`` additionally maps every backend the workflows configure
(evaluation/workflow.py:120-125) to ``"cuda"``: an unmodified CLI run is switched over without touching its
configuration.  Under autograd the norms and attention stay on this library where its backward kernels take the
shape (norm rows of whole 16-byte pieces, at most 1024 16-bit columns; attention up to 4096 rows); other shapes go
back to the reference's own dispatcher (torch backend).
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

    def wants_grad(*tensors) -> bool:
        return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)

    def rms_norm(x, weight, eps=1e-6, *, backend, block_rows=None):
        if pick(backend) == "cuda":
            # the norms are differentiable here for rows the backward kernels take; for other shapes a caller that
            # trains gets the reference's torch path when everything was routed here wholesale, and the operator's
            # own refusal when it asked for "cuda" itself
            if backend != "cuda" and wants_grad(x, weight) and not (x.is_cuda and ops.norm_backward_supported(x)):
                return ref_rms(x, weight, eps, backend="torch", block_rows=block_rows)
            return ops.rms_norm(x, weight, eps, backend="cuda", block_rows=block_rows)
        return ref_rms(x, weight, eps, backend=backend, block_rows=block_rows)

    def layer_norm(x, weight, bias, eps=1e-5, *, backend, block_rows=None):
        if pick(backend) == "cuda":
            if backend != "cuda" and wants_grad(x, weight, bias) and not (x.is_cuda and ops.norm_backward_supported(x)):
                return ref_ln(x, weight, bias, eps, backend="torch", block_rows=block_rows)
            return ops.layer_norm(x, weight, bias, eps, backend="cuda", block_rows=block_rows)
        return ref_ln(x, weight, bias, eps, backend=backend, block_rows=block_rows)

    def flash_attention(q, k, v, *, backend, **kwargs):
        if pick(backend) == "cuda":
            if backend != "cuda" and wants_grad(q, k, v) and not (q.is_cuda and ops.attention_backward_supported(q, k)):
                return ref_fa(q, k, v, backend="torch", **kwargs)
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

    _install_resolvers(mods)
    _install_config_literal()
    _install_benchmark_cli()

    # ---- embedding hook: the only way unmodified model code reaches the CUDA gather
    def bag_hook(weight: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
        if weight.device.type == "cuda" and ops.cuda_available() and ops.cuda_supported_floating_dtype(weight.dtype):
            return ops.embedding_bag_mean(weight, values, backend="cuda")
        return mods["bag"]._torch_embedding_bag_mean(weight, values)

    _originals.append((mods["bag"], "_embedding_bag_mean_kernel", mods["bag"]._embedding_bag_mean_kernel))
    mods["bag"].register_embedding_bag_mean_kernel(bag_hook)
    _state["installed"] = True


def _install_resolvers(mods: dict[str, Any]) -> None:
    """``resolved_*_backend(..., "cuda")`` answers "cuda" (after this library's own availability and dtype checks)
    in the operator modules, their packages and the accelerators namespace; other names go to the original."""
    holders = [mods["acc"]]
    for path in ("normalization", "attention", "embedding"):
        try:
            holders.append(importlib.import_module(f"taac2026.infrastructure.accelerators.{path}"))
        except ImportError:  # pragma: no cover - layout of another reference version
            pass

    def wrap(owner: Any, name: str, ours: Any, position: int) -> None:
        original = getattr(owner, name)

        def resolved(*args, **kwargs):
            backend = kwargs.get("backend", args[position] if len(args) > position else None)
            if backend == "cuda":
                call_kwargs = {k: v for k, v in kwargs.items() if k != "backend"}
                return ours(*args[:position], "cuda", *args[position + 1:], **call_kwargs)
            return original(*args, **kwargs)

        resolved.__name__ = name
        for holder in [owner, *holders]:
            if getattr(holder, name, None) is original:
                _patch(holder, name, resolved)

    wrap(mods["rms"], "resolved_rms_norm_backend", ops.resolved_rms_norm_backend, 1)
    wrap(mods["ln"], "resolved_layer_norm_backend", ops.resolved_layer_norm_backend, 1)
    wrap(mods["fa"], "resolved_flash_attention_backend", ops.resolved_flash_attention_backend, 3)
    wrap(mods["bag"], "resolved_embedding_bag_mean_backend", ops.resolved_embedding_bag_mean_backend, 2)


def _install_config_literal() -> None:
    """Teach the configuration layer the literal: the two ``Literal`` aliases, the two ``*_CHOICES`` tuples that
    the field validators read at call time, and the two field annotations of ``PCVRModelConfig`` (rebuilt so that
    pydantic's own literal check accepts it as well)."""
    from typing import Literal

    try:
        cfg = importlib.import_module("taac2026.domain.config")
    except ImportError:  # pragma: no cover
        return
    rms_choices = tuple(dict.fromkeys((*cfg.RMS_NORM_BACKEND_CHOICES, "cuda")))
    fa_choices = tuple(dict.fromkeys((*cfg.FLASH_ATTENTION_BACKEND_CHOICES, "cuda")))
    _patch(cfg, "RMS_NORM_BACKEND_CHOICES", rms_choices)
    _patch(cfg, "FLASH_ATTENTION_BACKEND_CHOICES", fa_choices)
    _patch(cfg, "RMSNormBackend", Literal[rms_choices])          # type: ignore[valid-type]
    _patch(cfg, "FlashAttentionBackend", Literal[fa_choices])    # type: ignore[valid-type]
    model = cfg.PCVRModelConfig
    changed = []
    for field_name, literal in (("rms_norm_backend", cfg.RMSNormBackend), ("flash_attention_backend", cfg.FlashAttentionBackend)):
        field = model.model_fields.get(field_name)
        if field is None:
            continue
        changed.append((field_name, field.annotation, model.__annotations__.get(field_name)))
        field.annotation = literal
        model.__annotations__[field_name] = literal
    if changed:
        model.model_rebuild(force=True)
        _config_undo.append((model, changed))


def _install_benchmark_cli() -> None:
    """`taac-benchmark-pcvr-tilelang-ops --backends ...,cuda`: the CLI module's backend list and its four helpers
    that turn (backend, tensors) into (callable, resolved name, compile seconds)."""
    import time

    try:
        bench = importlib.import_module("taac2026.application.benchmarking.pcvr_tilelang_ops_benchmark")
    except ImportError:  # pragma: no cover - the CLI's own dependencies (tyro, rich) may be absent
        return
    _patch(bench, "SUPPORTED_BACKENDS", tuple(dict.fromkeys((*bench.SUPPORTED_BACKENDS, "cuda"))))

    def timed_compile(build):
        started = time.perf_counter()
        kernel = build()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return kernel, time.perf_counter() - started

    ref_rms, ref_ln = bench._prepare_rms_norm_callable, bench._prepare_layer_norm_callable
    ref_fa, ref_bag = bench._prepare_flash_attention_callable, bench._prepare_embedding_bag_mean_callable

    def prepare_rms(*, backend, args, device, x, weight):
        if backend != "cuda":
            return ref_rms(backend=backend, args=args, device=device, x=x, weight=weight)
        ops.clear_rms_norm_kernel_cache()
        kernel, sec = timed_compile(lambda: ops.compile_rms_norm_kernel(x, weight, args.eps, block_rows=args.block_rows))
        return (lambda: kernel(x, weight)), "cuda", sec

    def prepare_ln(*, backend, args, device, x, weight, bias):
        if backend != "cuda":
            return ref_ln(backend=backend, args=args, device=device, x=x, weight=weight, bias=bias)
        ops.clear_layer_norm_kernel_cache()
        kernel, sec = timed_compile(lambda: ops.compile_layer_norm_kernel(x, weight, bias, args.eps, block_rows=args.block_rows))
        return (lambda: kernel(x, weight, bias)), "cuda", sec

    def prepare_fa(*, backend, args, device, q, k, v):
        if backend != "cuda":
            return ref_fa(backend=backend, args=args, device=device, q=q, k=k, v=v)
        ops.clear_flash_attention_kernel_cache()
        kernel, sec = timed_compile(lambda: ops.compile_flash_attention_kernel(q, k, v, is_causal=args.is_causal))
        key_lengths = torch.full((q.shape[0],), k.shape[2], dtype=torch.int32, device=q.device)
        return (lambda: kernel(q, k, v, key_lengths)), "cuda", sec

    def prepare_bag(*, backend, args, device, embedding_weight, values):
        if backend != "cuda":
            return ref_bag(backend=backend, args=args, device=device, embedding_weight=embedding_weight, values=values)
        ops.clear_embedding_bag_mean_kernel_cache()
        kernel, sec = timed_compile(lambda: ops.compile_embedding_bag_mean_kernel(embedding_weight, values))
        return (lambda: kernel(embedding_weight, values)), "cuda", sec

    _patch(bench, "_prepare_rms_norm_callable", prepare_rms)
    _patch(bench, "_prepare_layer_norm_callable", prepare_ln)
    _patch(bench, "_prepare_flash_attention_callable", prepare_fa)
    _patch(bench, "_prepare_embedding_bag_mean_callable", prepare_bag)


_config_undo: list[tuple[Any, list[tuple[str, Any, Any]]]] = []


def uninstall() -> None:
    """Put every wrapped attribute of the reference back."""
    while _config_undo:
        model, changed = _config_undo.pop()
        for field_name, annotation, class_annotation in changed:
            model.model_fields[field_name].annotation = annotation
            if class_annotation is not None:
                model.__annotations__[field_name] = class_annotation
        model.model_rebuild(force=True)
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
