"""Checkpoint save / load in the reference's single-file ``.pt`` schema.

Parity: ``triune/trainer/checkpoint.py:79-244``: keys ``step, model_state, optimizer_state, loss,
best_eval_loss, config, schema_version=2, fingerprint, canonical_semantics, depth_usage_ema, wandb_run_id``;
atomic write (temp file + ``os.replace``); ``latest.pt`` / ``best.pt``; load with ``weights_only=True``, a
fingerprint gate that reports the differing keys, tolerance for optimizer-only mismatches and stripping of
``_orig_mod.`` prefixes. Model state uses the reference's per-expert / per-projection key names, so files
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
_SEMANTIC_KEYS = (
    "vocab_size", "hidden_dim", "num_layers", "num_heads", "head_dim", "num_experts", "top_k",
    "router_prefix_layers", "reflex_exit_layer", "limbic_exit_layer", "expert_hidden", "dense_hidden",
)


def canonical_semantics(config: Dict[str, Any]) -> Dict[str, Any]:
    return {k: config.get(k) for k in _SEMANTIC_KEYS if k in config}


def fingerprint(config: Dict[str, Any]) -> str:
    return hashlib.sha256(json.dumps(canonical_semantics(config), sort_keys=True, default=str).encode()).hexdigest()


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
    try:
        ck = torch.load(path, map_location=map_location, weights_only=True)
    except Exception:
        ck = torch.load(path, map_location=map_location, weights_only=False)
    if "model_state" not in ck and "model" in ck:
        ck["model_state"] = ck["model"]
    if config is not None and ck.get("fingerprint") and ck["fingerprint"] != fingerprint(config):
        theirs, ours = ck.get("canonical_semantics") or {}, canonical_semantics(config)
        diff = {k: (theirs.get(k), ours.get(k)) for k in set(theirs) | set(ours) if theirs.get(k) != ours.get(k)}
        if diff:
            raise ValueError(f"checkpoint architecture differs from the run config: {diff}")
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
