"""Process-signal handling for training runs (reference: ``triune/trainer/callbacks.py``): SIGINT / SIGTERM save the
latest checkpoint once, then raise ``KeyboardInterrupt`` so the training loop unwinds normally."""

from __future__ import annotations

import signal
from typing import Callable


def install_checkpoint_signal_handlers(save_latest: Callable[[], object], signals=(signal.SIGINT, signal.SIGTERM)):
    """Returns the previous handlers so a caller can restore them."""
    state = {"saving": False}
    previous = {}

    def handler(signum, frame):
        if not state["saving"]:  # a second signal during the save must not start a second save
            state["saving"] = True
            try:
                save_latest()
            finally:
                state["saving"] = False
        raise KeyboardInterrupt

    for s in signals:
        try:
            previous[s] = signal.signal(s, handler)
        except (ValueError, OSError):  # not the main thread / not supported on this platform
            pass
    return previous


def restore_signal_handlers(previous) -> None:
    for s, h in previous.items():
        try:
            signal.signal(s, h)
        except (ValueError, OSError):
            pass
