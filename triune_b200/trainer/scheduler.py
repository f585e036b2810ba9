"""Learning-rate schedule (reference: ``triune/trainer/scheduler.py:4-37``): linear warm-up, cosine decay to
``min_lr``, and a fresh cycle (without warm-up) each time ``cycle_steps`` is passed."""

from __future__ import annotations

import math
from typing import Any, Dict


def lr_schedule(config: Dict[str, Any], step: int) -> float:
    lr, min_lr = float(config.get("lr", 1e-4)), float(config.get("min_lr", 1e-6))
    warmup = int(config.get("warmup_steps", 500))
    total = int(config.get("cycle_steps", config.get("total_steps", 50_000)))
    if step < warmup:
        return lr * (step + 1) / max(1, warmup)
    span = max(1, total - warmup)
    pos = step - warmup
    if pos >= span:
        pos = pos % span
    return min_lr + 0.5 * (lr - min_lr) * (1.0 + math.cos(math.pi * pos / span))


def set_optimizer_lr(optimizer, lr: float, expert_lr=None) -> None:
    if hasattr(optimizer, "set_lr"):
        optimizer.set_lr(lr, expert_lr=expert_lr)
        return
    for g in optimizer.param_groups:
        g["lr"] = lr
