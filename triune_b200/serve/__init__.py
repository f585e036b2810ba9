"""Serving API: FastAPI app, OpenAI-style chat completions, session recurrent state, request queue."""

from .engine_state import EngineState, get_state, reset_state
from .srsm import ServingRequestQueue, SessionRecurrentStateManager

__all__ = ["EngineState", "get_state", "reset_state", "ServingRequestQueue", "SessionRecurrentStateManager", "create_app", "run_server"]


def create_app(*a, **k):
    from .server import create_app as f

    return f(*a, **k)


def run_server(*a, **k):
    from .server import run_server as f

    return f(*a, **k)
