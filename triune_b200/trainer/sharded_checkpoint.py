"""Rank-local checkpoints of tensor- / expert-parallel models and their merge into the canonical single file.

Every rank of a sharded model writes ONE file with the slices it owns, each recorded under the key the *unsharded*
model uses in its ``state_dict`` (the reference's key layout: ``q_proj`` / ``k_proj`` / ``v_proj`` / ``g_proj``,
``gate_proj`` / ``up_proj`` / ``down_proj``, ``experts.{e}.{0,2}.{weight,bias}``;
``triune/trainer/checkpoint.py:79-98`` for the payload). Nothing is gathered at save time, so saving costs no
collective and no rank ever holds the whole model. ``merge_shards`` (``python -m triune_b200 checkpoint merge``) reads
the shard files one after another on the host and assembles the single-file checkpoint that ``load_checkpoint`` and
the inference entry points read. ``load_sharded`` resumes a sharded run from its own shard files without a merge.

A piece is ``(key, dim, start, stop, full, tensor)``: ``tensor`` is the slice ``[start, stop)`` along ``dim`` of the
full parameter whose size along that dimension is ``full``; ``dim is None`` means a whole tensor (replicated
parameters are written by shard 0 only; an expert owned by one rank is written by that rank).
"""

from __future__ import annotations

import glob
import os
import re
from typing import Any, Dict, Iterator, List, Optional, Tuple

import torch
import torch.nn as nn

from .checkpoint import (SCHEMA_VERSION, _atomic_save, _plain, _to_cpu, canonical_semantics, fingerprint,
                         safe_torch_load)

FORMAT = "triune_b200.sharded.v1"
Piece = Tuple[str, Optional[int], int, int, int, torch.Tensor]


def _sharded_modules(model: nn.Module):
    for name, mod in model.named_modules():
        if hasattr(mod, "checkpoint_pieces"):
            yield name, mod


def shard_position(model: nn.Module) -> Tuple[int, int]:
    """(rank, world) of this process inside the sharding group of the first sharded module (0, 1 if none)."""
    for _, mod in _sharded_modules(model):
        ctx = getattr(mod, "tp", None) or getattr(mod, "ep", None)
        if ctx is not None:
            return int(ctx.rank), int(ctx.world)
    return 0, 1


def collect_pieces(model: nn.Module) -> Tuple[List[Piece], Dict[str, torch.Tensor]]:
    """(sharded pieces, replicated tensors) of ``model``; all tensors are views of the live parameters."""
    pieces: List[Piece] = []
    handled: List[str] = []
    replicated: Dict[str, torch.Tensor] = {}
    for name, mod in _sharded_modules(model):
        prefix = name + "." if name else ""
        handled.append(prefix)
        pieces.extend(mod.checkpoint_pieces(prefix))
        for key, t in mod.checkpoint_replicated(prefix).items():
            replicated[key] = t
    for key, t in model.state_dict().items():
        key = key.replace("_orig_mod.", "")
        if not any(key.startswith(p) for p in handled):
            replicated[key] = t
    return pieces, replicated


def shard_path(ckpt_dir: str, rank: int, world: int) -> str:
    return os.path.join(ckpt_dir, f"shard-{rank:05d}-of-{world:05d}.pt")


def save_sharded(ckpt_dir: str, model: nn.Module, optimizer=None, step: int = 0, loss: float = 0.0,
                 config: Optional[Dict[str, Any]] = None, position: Optional[Tuple[int, int]] = None) -> str:
    """Write this rank's shard file. With data-parallel replicas of a sharded model only ONE replica calls this.
    The optimizer state is stored as this rank's own ``state_dict`` (it resumes on the same layout; it is not merged)."""
    rank, world = position if position is not None else shard_position(model)
    pieces, replicated = collect_pieces(model)
    os.makedirs(ckpt_dir, exist_ok=True)
    config = dict(config or {})
    arch = getattr(model, "model_config", None) or getattr(model, "cfg", None)
    arch = _plain(arch.to_dict()) if arch is not None and hasattr(arch, "to_dict") else None
    payload = {
        "format": FORMAT, "rank": rank, "world": world, "step": int(step), "loss": float(loss),
        "pieces": [(k, d, int(s), int(e), int(f), t.detach().cpu().clone()) for k, d, s, e, f, t in pieces],
        "replicated": {k: v.detach().cpu().clone() for k, v in replicated.items()} if rank == 0 else {},
        "optimizer_state": _to_cpu(optimizer.state_dict()) if optimizer is not None else None,
        "config": _plain(config), "architecture": arch,
    }
    path = shard_path(ckpt_dir, rank, world)
    _atomic_save(payload, path)
    return path


def _shard_files(ckpt_dir: str) -> List[str]:
    files = sorted(glob.glob(os.path.join(ckpt_dir, "shard-*-of-*.pt")))
    if not files:
        raise FileNotFoundError(f"no shard files in {ckpt_dir}")
    worlds = {int(re.search(r"-of-(\d+)\.pt$", f).group(1)) for f in files}
    if len(worlds) != 1:
        raise ValueError(f"{ckpt_dir} mixes shard sets of different sizes: {sorted(worlds)}")
    world = worlds.pop()
    ranks = [int(re.search(r"shard-(\d+)-of-", os.path.basename(f)).group(1)) for f in files]
    if sorted(ranks) != list(range(world)):
        raise ValueError(f"{ckpt_dir}: expected shards 0..{world - 1}, found {sorted(ranks)}")
    return files


def merge_shards(ckpt_dir: str, out_path: Optional[str] = None) -> Dict[str, Any]:
    """Assemble the canonical single-file checkpoint from all shard files of ``ckpt_dir``. Returns the payload (and
    writes it to ``out_path`` when given). Every sliced parameter must be covered exactly once."""
    state: Dict[str, torch.Tensor] = {}
    covered: Dict[str, int] = {}
    full_of: Dict[str, int] = {}
    meta: Dict[str, Any] = {}
    for f in _shard_files(ckpt_dir):
        sh = safe_torch_load(f)
        if sh.get("format") != FORMAT:
            raise ValueError(f"{f} is not a shard file of this format")
        if sh["rank"] == 0:
            meta = {k: sh.get(k) for k in ("step", "loss", "config", "architecture")}
            for k, v in sh["replicated"].items():
                state[k] = v
        for key, dim, start, stop, full, t in sh["pieces"]:
            if dim is None:
                if key in state:
                    raise ValueError(f"{key} is written by more than one shard")
                state[key] = t
                continue
            if key not in state:
                shape = list(t.shape)
                shape[dim] = full
                state[key] = torch.zeros(shape, dtype=t.dtype)
                covered[key], full_of[key] = 0, full
            idx = [slice(None)] * state[key].dim()
            idx[dim] = slice(start, stop)
            state[key][tuple(idx)] = t
            covered[key] += stop - start
    bad = [k for k, n in covered.items() if n != full_of[k]]
    if bad:
        raise ValueError(f"incomplete or overlapping shards for {bad[:4]}")
    config = meta.get("config") or {}
    payload = {
        "step": int(meta.get("step") or 0), "model_state": state, "optimizer_state": None,
        "loss": float(meta.get("loss") or 0.0), "best_eval_loss": float("inf"), "config": config,
        "schema_version": SCHEMA_VERSION, "fingerprint": fingerprint(config), "architecture": meta.get("architecture"),
        "canonical_semantics": canonical_semantics(config), "arch_extras": {}, "depth_usage_ema": None, "wandb_run_id": None,
        "merged_from": {"dir": os.path.basename(os.path.normpath(ckpt_dir)), "shards": len(_shard_files(ckpt_dir))},
    }
    if out_path:
        _atomic_save(payload, out_path)
    return payload


@torch.no_grad()
def load_sharded(ckpt_dir: str, model: nn.Module, optimizer=None, position: Optional[Tuple[int, int]] = None) -> Dict[str, Any]:
    """Resume a sharded model from its own shard file (same parallel layout as at save time)."""
    rank, world = position if position is not None else shard_position(model)
    sh = safe_torch_load(shard_path(ckpt_dir, rank, world))
    pieces, replicated = collect_pieces(model)
    saved = {(k, d, s, e): t for k, d, s, e, _, t in sh["pieces"]}
    for k, d, s, e, _, view in pieces:
        if (k, d, s, e) not in saved:
            raise KeyError(f"shard {rank} has no slice {k}[{s}:{e}] (a different parallel layout?)")
        view.copy_(saved[(k, d, s, e)].to(view.device, view.dtype))
    rep = sh["replicated"] if rank == 0 else safe_torch_load(shard_path(ckpt_dir, 0, world))["replicated"]
    for k, view in replicated.items():
        if k in rep:
            view.copy_(rep[k].to(view.device, view.dtype))
    if optimizer is not None and sh.get("optimizer_state") is not None:
        optimizer.load_state_dict(sh["optimizer_state"])
    if optimizer is not None and hasattr(optimizer, "arena"):
        optimizer.arena.rebind()
        if sh.get("optimizer_state") is None:
            optimizer.arena.sync_master_from_params()
    return {"step": sh["step"], "loss": sh["loss"], "config": sh["config"]}
