"""Checkpoint save / load in the reference's single-file ``.pt`` schema.

Parity: ``triune/trainer/checkpoint.py:79-244``: keys ``step, model_state, optimizer_state, loss,
best_eval_loss, config, schema_version=2, fingerprint, canonical_semantics, depth_usage_ema, wandb_run_id``;
atomic write (temp file + ``os.replace``); ``latest.pt`` / ``best.pt``; load with ``weights_only=True`` only, the
schema-v2 fingerprint (nested by category, compact JSON, SHA-256) with a gate that reports the differing
``category.key`` entries, tolerance for optimizer-only mismatches on a weights-only load, the critical-key
comparison for files without a fingerprint, and stripping of ``_orig_mod.`` prefixes. Model state uses the reference's per-expert / per-projection key names, so files
written by either project load in the other.
"""

from __future__ import annotations

import hashlib
import json
import os
import tempfile
from typing import Any, Dict, Optional

import torch

SCHEMA_VERSION = 2

# Schema-v2 fingerprint: the canonical semantics are nested by category, serialised with sort_keys and the compact
# separators (",", ":"), and hashed with SHA-256. The table is the file-format contract of the reference
# (``triune/trainer/checkpoint.py:19-42``): a file written by either project must hash to the same value in the other.
_MODEL_SPEC = (
    ("architecture", ("hidden_dim", "num_layers", "num_heads", "head_dim", "vocab_size")),
    ("attention", ("head_dim", "use_rope", "rope_max_seq_len")),
    ("moe", ("num_experts", "top_k", "shared_expert", "shared_scale", "capacity_multiplier")),
    ("hierarchy", ("router_prefix_layers", "reflex_exit_layer", "limbic_exit_layer", "target_depth_dist")),
    ("precision", ("use_fp4", "use_fp8")),
)
_OPTIMIZER_SPEC = (("optimizer", ("use_muon", "muon_lr", "galore", "galore_rank")),)
FINGERPRINT_SPEC = _MODEL_SPEC + _OPTIMIZER_SPEC
MODEL_CATEGORIES = tuple(c for c, _ in _MODEL_SPEC)
# Without a stored fingerprint (files older than schema 2) these keys are compared one by one.
_LEGACY_CRITICAL_KEYS = ("hidden_dim", "num_layers", "num_heads", "head_dim", "vocab_size", "num_experts", "top_k",
                         "shared_expert", "router_prefix_layers", "reflex_exit_layer", "limbic_exit_layer")
# Architecture keys of this framework that the reference's table does not carry; stored beside the fingerprint
# (``arch_extras``) and compared on load when both sides have them.
_EXTRA_KEYS = ("expert_hidden", "dense_hidden")


def _canon(config: Dict[str, Any], spec) -> Dict[str, Any]:
    out: Dict[str, Any] = {"schema_version": SCHEMA_VERSION}
    for category, keys in spec:
        out[category] = {k: (list(v) if isinstance(v := config.get(k), tuple) else v) for k in keys}
    return out


def canonical_semantics(config: Dict[str, Any]) -> Dict[str, Any]:
    """``{"schema_version": 2, category: {key: value}}`` over every fingerprint category (missing keys are None)."""
    return _canon(config, FINGERPRINT_SPEC)


def _digest(canon: Dict[str, Any]) -> str:
    return hashlib.sha256(json.dumps(canon, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()


def fingerprint(config: Dict[str, Any]) -> str:
    """SHA-256 over the schema-v2 canonical semantics (model and optimizer categories)."""
    return _digest(canonical_semantics(config))


def model_fingerprint(config: Dict[str, Any]) -> str:
    """The same hash over the model categories only (what a weights-only load has to agree on)."""
    return _digest(_canon(config, _MODEL_SPEC))


# the reference's names of the same things (``triune/trainer/checkpoint.py:29-76``)
MODEL_FINGERPRINT_KEYS = {c: list(k) for c, k in _MODEL_SPEC}
OPTIMIZER_FINGERPRINT_KEYS = {c: list(k) for c, k in _OPTIMIZER_SPEC}
compute_model_fingerprint = model_fingerprint
extract_canonical_semantics = canonical_semantics
compute_checkpoint_fingerprint = fingerprint


def safe_torch_load(path, map_location="cpu"):
    """``torch.load(..., weights_only=True)`` and nothing else: a checkpoint path can come from an API request, so a
    file that needs the unrestricted unpickler is refused (the error says which type it wanted). Types that are
    known to be harmless can be allow-listed by the caller with ``torch.serialization.add_safe_globals``."""
    return torch.load(path, map_location=map_location, weights_only=True)


def _semantic_mismatches(saved: Dict[str, Any], current: Dict[str, Any], categories) -> list:
    out = []
    for category, keys in FINGERPRINT_SPEC:
        if category not in categories:
            continue
        s_cat, c_cat = saved.get(category) or {}, current.get(category) or {}
        for k in keys:
            if s_cat.get(k) != c_cat.get(k):
                out.append(f"{category}.{k}: saved={s_cat.get(k)} vs current={c_cat.get(k)}")
    return out


def check_compatibility(ck: Dict[str, Any], config: Dict[str, Any], load_optimizer: bool, path: str = "") -> None:
    """The fingerprint gate of ``load_checkpoint`` (``triune/trainer/checkpoint.py:158-244``). Raises ``ValueError``
    naming every differing ``category.key``. A weights-only load tolerates differences in the optimizer category."""
    saved_fp, saved_cfg = ck.get("fingerprint"), ck.get("config") or {}
    if saved_fp is not None:
        current_fp = fingerprint(config)
        if saved_fp != current_fp:
            saved_canon = ck.get("canonical_semantics")
            if not (isinstance(saved_canon, dict) and any(isinstance(saved_canon.get(c), dict) for c in MODEL_CATEGORIES)):
                saved_canon = canonical_semantics(saved_cfg)  # flat or missing record: rebuild from the stored config
            cats = MODEL_CATEGORIES + (("optimizer",) if load_optimizer else ())
            diff = _semantic_mismatches(saved_canon, canonical_semantics(config), cats)
            if diff or load_optimizer:
                lines = "\n".join(f"  - {m}" for m in diff) if diff else "  - non-semantic configuration variation"
                raise ValueError(f"checkpoint architecture mismatch for {path}\nsaved fingerprint:   {saved_fp}\n"
                                 f"current fingerprint: {current_fp}\nchanged parameters:\n{lines}")
    elif saved_cfg:
        diff = [f"{k}: saved={saved_cfg.get(k)} vs current={config.get(k)}" for k in _LEGACY_CRITICAL_KEYS
                if saved_cfg.get(k) is not None and config.get(k) is not None and saved_cfg.get(k) != config.get(k)]
        if diff:
            raise ValueError(f"checkpoint architecture mismatch for {path}:\n" + "\n".join(f"  - {m}" for m in diff))
    extras = ck.get("arch_extras") or {}
    diff = [f"{k}: saved={extras[k]} vs current={config[k]}" for k in _EXTRA_KEYS
            if extras.get(k) is not None and config.get(k) is not None and extras[k] != config[k]]
    if diff:
        raise ValueError(f"checkpoint architecture mismatch for {path}:\n" + "\n".join(f"  - {m}" for m in diff))


def _atomic_save(obj, path: str) -> None:
    d = os.path.dirname(os.path.abspath(path)) or "."
    os.makedirs(d, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=d, suffix=".tmp")
    os.close(fd)
    try:
        torch.save(obj, tmp)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def _plain(v):
    if isinstance(v, dict):
        return {k: _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


def save_checkpoint(path: str, model, optimizer=None, step: int = 0, loss: float = 0.0, best_eval_loss: float = float("inf"),
                    config: Optional[Dict[str, Any]] = None, depth_usage_ema=None, wandb_run_id=None) -> str:
    config = dict(config or {})
    arch = getattr(model, "model_config", None)  # the architecture travels with the weights, apart from the run config
    arch = _plain(arch.to_dict()) if arch is not None and hasattr(arch, "to_dict") else None
    sd = {k.replace("_orig_mod.", ""): v.detach().cpu() for k, v in model.state_dict().items()}
    payload = {
        "step": int(step), "model_state": sd,
        "optimizer_state": _to_cpu(optimizer.state_dict()) if optimizer is not None else None,
        "loss": float(loss), "best_eval_loss": float(best_eval_loss), "config": _plain(config),
        "schema_version": SCHEMA_VERSION, "fingerprint": fingerprint(config), "architecture": arch,
        "canonical_semantics": canonical_semantics(config),
        "arch_extras": {k: config.get(k) for k in _EXTRA_KEYS if config.get(k) is not None},
        "depth_usage_ema": list(depth_usage_ema) if depth_usage_ema is not None else None,
        "wandb_run_id": wandb_run_id,
    }
    _atomic_save(payload, path)
    return path


def _to_cpu(obj):
    if torch.is_tensor(obj):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


def save_latest(ckpt_dir: str, **kw) -> str:
    return save_checkpoint(os.path.join(ckpt_dir, "latest.pt"), **kw)


def save_best(ckpt_dir: str, **kw) -> str:
    return save_checkpoint(os.path.join(ckpt_dir, "best.pt"), **kw)


def load_checkpoint(path: str, model=None, optimizer=None, config: Optional[Dict[str, Any]] = None, strict: bool = True,
                    map_location="cpu") -> Dict[str, Any]:
    ck = safe_torch_load(path, map_location=map_location)
    if "model_state" not in ck and "model" in ck:
        ck["model_state"] = ck["model"]
    if config is not None:
        check_compatibility(ck, config, load_optimizer=optimizer is not None, path=str(path))
    if model is not None:
        sd = {k.replace("_orig_mod.", ""): v for k, v in ck["model_state"].items()}
        model.load_state_dict(sd, strict=strict)
    if optimizer is not None and ck.get("optimizer_state") is not None:
        try:
            optimizer.load_state_dict(ck["optimizer_state"])
        except Exception as e:  # weights-only resume is allowed
            ck["optimizer_load_error"] = str(e)
    if optimizer is not None and hasattr(optimizer, "arena"):
        optimizer.arena.rebind()
        if ck.get("optimizer_load_error") or ck.get("optimizer_state") is None:
            optimizer.arena.sync_master_from_params()
    return ck
