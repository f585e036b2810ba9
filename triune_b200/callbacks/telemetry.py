"""Per-step telemetry callback (reference: ``triune/callbacks/telemetry.py``): loss terms, router target, device memory."""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import torch

from .base import Callback


class TelemetryCallback(Callback):
    def __init__(self, broadcast_fn: Optional[Callable[[Dict[str, Any]], None]] = None, max_history: int = 10000):
        self.broadcast_fn = broadcast_fn
        self.history: List[Dict[str, Any]] = []
        self.max_history = max_history

    def on_step_end(self, trainer: Any, step: int, logs: Dict[str, Any]) -> None:
        dev = getattr(trainer, "device", None)
        gb = torch.cuda.memory_allocated(dev) / 2**30 if dev is not None and dev.type == "cuda" else 0.0

        def val(k):
            v = logs.get(k)
            return float(v) if torch.is_tensor(v) else v

        payload = {"step": step, "loss": val("loss"), "lm_loss": val("lm_loss"), "router_loss": val("router_loss"),
                   "target_router": logs.get("target_router"), "vram_gb": round(gb, 3)}
        self.history.append(payload)
        if len(self.history) > self.max_history:
            del self.history[: len(self.history) - self.max_history]
        if self.broadcast_fn:
            self.broadcast_fn(payload)
