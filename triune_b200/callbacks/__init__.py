from .base import Callback, CallbackList
from .events import EventEmitter, global_emitter
from .telemetry import TelemetryCallback

__all__ = ["Callback", "CallbackList", "TelemetryCallback", "EventEmitter", "global_emitter"]
