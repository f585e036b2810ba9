"""Local launcher: start (or find) the API server on this machine and open its page.

What it does, in order: if the wanted port already answers ``/healthz`` as this service, reuse that server; if another
program holds the port, move to the next free one; otherwise start ``python -m triune_b200 serve`` as a child process,
wait until it is healthy, then open the default browser on it (unless told not to) and stay in the foreground until
interrupted, at which point the child is stopped. There is no embedded web view and no GUI toolkit here: the page is
whatever the server mounts from ``--static-dir`` plus its HTTP API.

Covers the launcher part of the reference's desktop shell (``triune/desktop.py:22-62`` port and liveness probes,
``:118-385`` launch flow); its WSL interpreter discovery and Windows host are specific to that shell and not built.
"""

from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time
import urllib.error
import urllib.request
from typing import List, Optional

SERVICE_NAME = "triune-b200"


def port_in_use(port: int, host: str = "127.0.0.1") -> bool:
    """True when something listens on the port. Decided by trying to bind it, so a listener whose accept queue is full
    (and which therefore does not answer a probe connection) still counts."""
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        try:
            s.bind((host, port))
        except OSError:
            return True
    return False


def find_free_port(start: int = 8000, attempts: int = 20, host: str = "127.0.0.1") -> int:
    """The first port at or after ``start`` that nothing listens on."""
    for port in range(start, start + attempts):
        if not port_in_use(port, host):
            return port
    raise RuntimeError(f"no free port in [{start}, {start + attempts})")


def server_alive(port: int, host: str = "127.0.0.1", timeout: float = 1.0) -> bool:
    """True when the port answers ``/healthz`` as this service (and not as some other program)."""
    try:
        with urllib.request.urlopen(f"http://{host}:{port}/healthz", timeout=timeout) as r:
            return json.loads(r.read().decode()).get("service") == SERVICE_NAME
    except (urllib.error.URLError, OSError, ValueError):
        return False


def wait_for_server(port: int, host: str = "127.0.0.1", timeout: float = 60.0, proc: Optional[subprocess.Popen] = None) -> bool:
    """Poll until the server is healthy, the child has exited, or the time is up."""
    end = time.monotonic() + timeout
    while time.monotonic() < end:
        if server_alive(port, host):
            return True
        if proc is not None and proc.poll() is not None:
            return False
        time.sleep(0.2)
    return False


def server_command(port: int, host: str = "127.0.0.1", model: Optional[str] = None, static_dir: Optional[str] = None,
                   precision: Optional[str] = None) -> List[str]:
    cmd = [sys.executable, "-m", "triune_b200", "serve", "--host", host, "--port", str(port)]
    if model:
        cmd += ["--model", model]
    if precision:
        cmd += ["--precision", precision]
    if static_dir:
        cmd += ["--static-dir", static_dir]
    return cmd


class DesktopSession:
    """A running (or reused) server: ``url``, ``port``, and the child process if this session started one."""

    def __init__(self, port: int, host: str, proc: Optional[subprocess.Popen], reused: bool):
        self.port, self.host, self.proc, self.reused = port, host, proc, reused

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}/"

    def stop(self, grace: float = 5.0) -> None:
        """Stop the child this session started (a reused server is left alone)."""
        if self.proc is None or self.proc.poll() is not None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=grace)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            self.proc.wait(timeout=grace)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()


def start_session(port: int = 8000, host: str = "127.0.0.1", model: Optional[str] = None, static_dir: Optional[str] = None,
                  precision: Optional[str] = None, startup_timeout: float = 120.0, quiet: bool = False) -> DesktopSession:
    """Find or start the server and return once it is healthy."""
    say = (lambda *_: None) if quiet else (lambda m: print(f"[launcher] {m}", flush=True))
    if port_in_use(port, host):
        if server_alive(port, host):
            say(f"using the server that already runs on http://{host}:{port}/")
            return DesktopSession(port, host, None, True)
        moved = find_free_port(port + 1, host=host)
        say(f"port {port} belongs to another program; using {moved}")
        port = moved
    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    out = subprocess.DEVNULL if quiet else None
    proc = subprocess.Popen(server_command(port, host, model, static_dir, precision), env=env, stdout=out, stderr=out)
    if not wait_for_server(port, host, startup_timeout, proc):
        code = proc.poll()
        DesktopSession(port, host, proc, False).stop()
        raise RuntimeError(f"the server did not come up on port {port}" + (f" (exit code {code})" if code is not None else ""))
    say(f"server ready on http://{host}:{port}/")
    return DesktopSession(port, host, proc, False)


def launch_desktop_app(port: int = 8000, use_browser: bool = True, host: str = "127.0.0.1", model: Optional[str] = None,
                       static_dir: Optional[str] = None, precision: Optional[str] = None, block: bool = True) -> DesktopSession:
    """Start or reuse the server, open the page, and (``block``) stay until Ctrl-C or until the server exits."""
    session = start_session(port, host, model, static_dir, precision)
    if use_browser:
        import webbrowser

        try:
            webbrowser.open(session.url)
        except Exception as e:  # a headless machine has no browser to open
            print(f"[launcher] no browser could be opened ({e}); the page is at {session.url}", flush=True)
    if not block:
        return session
    try:
        while session.proc is None or session.proc.poll() is None:
            time.sleep(0.5)
            if session.proc is None and not server_alive(session.port, session.host):
                break
    except KeyboardInterrupt:
        pass
    finally:
        session.stop()
    return session
