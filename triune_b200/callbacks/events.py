"""Event emitter for live logs, loss curves and generated tokens (reference: ``triune/callbacks/events.py``)."""

from __future__ import annotations

import logging
import time
from collections import defaultdict
from typing import Any, Callable, Dict, List

log = logging.getLogger(__name__)


class EventEmitter:
    def __init__(self):
        self._listeners: Dict[str, List[Callable]] = defaultdict(list)

    def on(self, event_name: str, listener: Callable) -> None:
        self._listeners[event_name].append(listener)

    def off(self, event_name: str, listener: Callable) -> None:
        if listener in self._listeners.get(event_name, ()):
            self._listeners[event_name].remove(listener)

    def emit(self, event_name: str, *args: Any, **kwargs: Any) -> None:
        for fn in list(self._listeners.get(event_name, ())):
            try:
                fn(*args, **kwargs)
            except Exception as err:  # a broken listener must not stop training
                log.warning("listener error for %r: %s", event_name, err)

    def _stamp(self, event, **payload):
        payload["timestamp"] = time.time()
        self.emit(event, payload)

    def emit_node_start(self, node_id: str, node_type: str, params: Dict[str, Any]) -> None:
        self._stamp("on_node_start", node_id=node_id, node_type=node_type, params=params)

    def emit_token_generate(self, token: str, step: int) -> None:
        self._stamp("on_token_generate", token=token, step=step)

    def emit_loss_update(self, step: int, loss: float, lm_loss: float = 0.0, router_loss: float = 0.0) -> None:
        self._stamp("on_loss_update", step=step, loss=loss, lm_loss=lm_loss, router_loss=router_loss)

    def emit_vram_update(self, allocated_gb: float, reserved_gb: float, total_gb: float) -> None:
        self._stamp("on_vram_update", allocated_gb=allocated_gb, reserved_gb=reserved_gb, total_gb=total_gb)


global_emitter = EventEmitter()
