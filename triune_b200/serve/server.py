"""FastAPI application factory and launcher.

Parity (``triune/api/server.py:57-221``): ``/healthz`` that touches neither PyTorch nor the model; a middleware that
lets loopback clients through and requires ``Authorization: Bearer $TRIUNE_API_TOKEN`` (at least 32 characters,
constant-time comparison) from anyone else on ``/v1`` and ``/api`` paths; binding to a non-loopback interface refuses to
start without that token and TLS certificate + key files; the single-page Studio (``triune_b200/studio``, or ``static_dir``) mounted under ``/static`` and served at ``/``.
"""

from __future__ import annotations

import hmac
from contextlib import asynccontextmanager
import ipaddress
import os
from pathlib import Path
from typing import Optional

MIN_TOKEN_CHARS = 32


def _is_loopback(host: Optional[str]) -> bool:
    if host in ("testclient", "localhost"):
        return True
    try:
        return host is not None and ipaddress.ip_address(host).is_loopback
    except ValueError:
        return False


@asynccontextmanager
async def lifespan(app):
    """Nothing to start (models load on request); on shutdown a training run that is still going is asked to stop and
    joined, so that the process does not exit with the trainer half-way through a checkpoint."""
    yield
    from .engine_state import get_state

    state = get_state()
    if state.train_status.get("running"):
        state.stop_training()


def create_app(static_dir: Optional[str] = None):
    import fastapi
    from fastapi.responses import FileResponse, JSONResponse

    from .routes import router

    app = fastapi.FastAPI(title="Triune B200 server", description="Serving, training control and telemetry API", version="1.0.0",
                          lifespan=lifespan)

    @app.get("/healthz", include_in_schema=False)
    async def healthz():
        return {"status": "ok", "service": "triune-b200"}

    @app.middleware("http")
    async def restrict_remote_api(request, call_next):
        if request.url.path.startswith(("/v1/", "/api/")) and not _is_loopback(request.client.host if request.client else None):
            token = os.environ.get("TRIUNE_API_TOKEN", "")
            if len(token) < MIN_TOKEN_CHARS:
                return JSONResponse(status_code=503, content={"detail": f"Remote API is unavailable: configure TRIUNE_API_TOKEN with at least {MIN_TOKEN_CHARS} characters."})
            scheme, _, cred = request.headers.get("authorization", "").partition(" ")
            if scheme.lower() != "bearer" or not hmac.compare_digest(cred.encode(), token.encode()):
                return JSONResponse(status_code=401, headers={"WWW-Authenticate": "Bearer"},
                                    content={"detail": "A valid bearer token is required for remote API access."})
        return await call_next(request)

    app.include_router(router)
    from .routes_shell import shell_router

    app.include_router(shell_router)
    # the packaged single-page Studio (chat, training control, graph canvas, fine-tuning, system) unless another directory is given
    root = Path(static_dir) if static_dir else Path(__file__).resolve().parent.parent / "studio"
    if root is not None and root.is_dir() and (root / "index.html").is_file():
        from fastapi.staticfiles import StaticFiles

        app.mount("/static", StaticFiles(directory=str(root)), name="static")
        no_cache = {"Cache-Control": "no-cache, no-store, must-revalidate", "Pragma": "no-cache", "Expires": "0"}

        @app.get("/")
        async def index():
            return FileResponse(str(root / "index.html"), headers=no_cache)

        @app.get("/{full_path:path}")
        async def spa(full_path: str):
            try:
                cand = (root / full_path).resolve(strict=True)
                cand.relative_to(root.resolve())  # never serve anything outside the static root
                if cand.is_file():
                    return FileResponse(str(cand), headers=no_cache)
            except (OSError, RuntimeError, ValueError):
                pass
            return FileResponse(str(root / "index.html"), headers=no_cache)

    return app


def check_bind_policy(host: str) -> dict:
    """Raises unless ``host`` is loopback or both a long token and TLS files are configured; returns uvicorn TLS kwargs."""
    cert, key = os.environ.get("TRIUNE_TLS_CERTFILE", ""), os.environ.get("TRIUNE_TLS_KEYFILE", "")
    if not _is_loopback(host):
        if len(os.environ.get("TRIUNE_API_TOKEN", "")) < MIN_TOKEN_CHARS:
            raise RuntimeError(f"Binding to a remote interface requires TRIUNE_API_TOKEN with at least {MIN_TOKEN_CHARS} characters.")
        if not (cert and key and Path(cert).is_file() and Path(key).is_file()):
            raise RuntimeError("Binding to a remote interface requires valid TRIUNE_TLS_CERTFILE and TRIUNE_TLS_KEYFILE files; "
                               "alternatively keep the server on loopback behind an authenticated HTTPS proxy.")
    return {"ssl_certfile": cert or None, "ssl_keyfile": key or None}


def run_server(host: str = "127.0.0.1", port: int = 8000, static_dir: Optional[str] = None, log_level: str = "info") -> None:
    import threading

    import uvicorn

    tls = check_bind_policy(host)

    class SafeServer(uvicorn.Server):
        def install_signal_handlers(self) -> None:  # signal handlers can only be installed from the main thread
            if threading.current_thread() is threading.main_thread():
                super().install_signal_handlers()

    SafeServer(uvicorn.Config(app=create_app(static_dir), host=host, port=port, log_level=log_level, **tls)).run()
