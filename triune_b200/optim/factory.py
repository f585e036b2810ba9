"""Optimizer factory (reference: ``triune/optim/factory.py:12-40``): config dict -> CentroidSteer or AdamW."""

from __future__ import annotations

from typing import Any, Dict

import torch

from .centroid import CentroidSteerOptimizer


def build_optimizer(model: torch.nn.Module, config: Dict[str, Any]):
    kind = str(config.get("optimizer", "centroid_steer" if config.get("galore", True) else "adamw")).lower()
    lr = float(config.get("lr", 1e-4))
    betas = tuple(config.get("betas", (0.9, 0.95)))
    wd = float(config.get("weight_decay", 0.05))
    if kind in ("centroid_steer", "centroid", "galore"):
        return CentroidSteerOptimizer(
            model, lr=lr, betas=betas, weight_decay=wd, rank=int(config.get("galore_rank", 256)),
            update_gap=int(config.get("galore_update_gap", 200)), steer_scale=float(config.get("steer_scale", 0.2)),
            steer_update_gap=int(config.get("steer_update_gap", 10)), expert_lr=config.get("galore_lr"),
            expert_betas=tuple(config.get("galore_betas", (0.9, 0.999))),
            expert_wd=float(config.get("galore_weight_decay", 0.05)), use_muon=bool(config.get("use_muon", True)),
            muon_lr=config.get("muon_lr"), muon_momentum=float(config.get("muon_momentum", 0.95)),
            muon_weight_decay=float(config.get("muon_weight_decay", 0.01)),
            muon_ns_steps=int(config.get("ns_steps", config.get("muon_ns_steps", 3))),
            use_triangular_core=bool(config.get("use_triangular_core", True)),
            core_mask_mode=str(config.get("core_mask_mode", "full")), grad_clip=config.get("grad_clip"),
        )
    if kind == "muon":
        return CentroidSteerOptimizer(model, lr=lr, betas=betas, weight_decay=wd, use_triangular_core=False,
                                      steer_scale=0.0, grad_clip=config.get("grad_clip"),
                                      muon_ns_steps=int(config.get("ns_steps", 3)))
    return torch.optim.AdamW(model.parameters(), lr=lr, betas=betas, weight_decay=wd)
