"""Trainer lifecycle callbacks (reference: ``triune/callbacks/base.py``)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional

_EVENTS = ("on_train_begin", "on_train_end", "on_step_begin", "on_step_end", "on_eval_begin", "on_eval_end")


class Callback:
    def on_train_begin(self, trainer: Any) -> None: ...
    def on_train_end(self, trainer: Any) -> None: ...
    def on_step_begin(self, trainer: Any, step: int) -> None: ...
    def on_step_end(self, trainer: Any, step: int, logs: Dict[str, Any]) -> None: ...
    def on_eval_begin(self, trainer: Any) -> None: ...
    def on_eval_end(self, trainer: Any, eval_loss: float) -> None: ...


class CallbackList(Callback):
    """Fans every event out to its members, in registration order."""

    def __init__(self, callbacks: Optional[List[Callback]] = None):
        self.callbacks: List[Callback] = list(callbacks or [])

    def add(self, callback: Callback) -> None:
        self.callbacks.append(callback)


def _fan_out(name):
    def dispatch(self, *args, **kwargs):
        for cb in self.callbacks:
            getattr(cb, name)(*args, **kwargs)

    dispatch.__name__ = name
    return dispatch


for _n in _EVENTS:
    setattr(CallbackList, _n, _fan_out(_n))
