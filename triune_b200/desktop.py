"""Local launcher: start (or find) the API server on this machine and open its page.

What it does, in order: if the wanted port already answers ``/healthz`` as this service, reuse that server; if another
program holds the port, move to the next free one; otherwise start ``python -m triune_b200 serve`` as a child process,
wait until it is healthy, then open the default browser on it (unless told not to) and stay in the foreground until
interrupted, at which point the child is stopped. There is no embedded web view and no GUI toolkit here: the page is
the packaged Studio (or whatever ``--static-dir`` names) plus the HTTP API.

On a Windows host without a CUDA build of PyTorch the server can run inside WSL 2 instead (``allow_wsl``): the
launcher looks for a Python interpreter there that can import this package and sees a GPU, translates the workspace
path, and starts ``python -m triune_b200 serve`` through ``wsl.exe``; WSL forwards the guest's loopback port to the
host, so the page opens on the same URL. All of that goes through an injectable command runner, so it is tested
without Windows.

Covers the launcher of the reference's desktop shell (``triune/desktop.py:22-62`` port and liveness probes, ``:64-116``
WSL interpreter discovery and path translation, ``:118-385`` launch flow); its WPF host window is not built.
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
from typing import Callable, List, Optional, Sequence, Tuple

SERVICE_NAME = "triune-b200"

# (argv, timeout seconds) -> (exit code, stdout); the one place the WSL helpers touch the system
Runner = Callable[[Sequence[str], float], Tuple[int, str]]


def _run(argv: Sequence[str], timeout: float = 8.0) -> Tuple[int, str]:
    try:
        flags = getattr(subprocess, "CREATE_NO_WINDOW", 0) if sys.platform == "win32" else 0
        r = subprocess.run(list(argv), capture_output=True, text=True, timeout=timeout, creationflags=flags)
        return r.returncode, r.stdout
    except (OSError, subprocess.SubprocessError):
        return 127, ""


def to_wsl_path(path: str) -> str:
    """``C:\\Users\\me\\repo`` -> ``/mnt/c/Users/me/repo``; UNC paths into a distribution (``\\\\wsl$\\Ubuntu\\home\\me`` or
    ``\\\\wsl.localhost\\...``) -> the path inside it; POSIX paths are returned unchanged."""
    p = str(path)
    low = p.lower()
    for prefix in ("\\\\wsl$\\", "\\\\wsl.localhost\\"):
        if low.startswith(prefix):
            rest = p[len(prefix):].split("\\", 1)
            return "/" + (rest[1].replace("\\", "/") if len(rest) > 1 else "")
    if len(p) >= 2 and p[1] == ":" and p[0].isalpha():
        return f"/mnt/{p[0].lower()}" + p[2:].replace("\\", "/")
    return p.replace("\\", "/")


def find_wsl_python(workspace: Optional[str] = None, candidates: Sequence[str] = (), run: Runner = _run) -> Optional[dict]:
    """An interpreter inside the default WSL distribution that can serve this package, or None.

    Tried in order: ``$TRIUNE_WSL_PYTHON``, ``candidates``, ``~/venvs/triune/bin/python``, ``~/.venv/bin/python``, the
    workspace's own ``.venv``, then ``python3`` on the guest's PATH. A candidate counts when it exists, imports torch,
    and (with ``workspace``) finds the package there. Returns ``{"python", "cuda", "torch", "workspace"}``; candidates
    that see a GPU are preferred over ones that do not."""
    code, _ = run(["wsl.exe", "--status"], 5.0)
    if code != 0:
        return None
    ws = to_wsl_path(workspace) if workspace else None
    tried: List[str] = [c for c in (os.environ.get("TRIUNE_WSL_PYTHON"), *candidates) if c]
    code, home = run(["wsl.exe", "-e", "sh", "-c", "printf %s \"$HOME\""], 5.0)
    home = home.strip() if code == 0 else ""
    if home:
        tried += [f"{home}/venvs/triune/bin/python", f"{home}/.venv/bin/python"]
    if ws:
        tried.append(f"{ws}/.venv/bin/python")
    code, which = run(["wsl.exe", "-e", "sh", "-c", "command -v python3"], 5.0)
    if code == 0 and which.strip():
        tried.append(which.strip().splitlines()[0])
    probe = ("import json,sys\n"
             "try:\n import torch; t=torch.__version__; c=bool(torch.cuda.is_available())\n"
             "except Exception: t=None; c=False\n"
             "ok=True\n"
             "if len(sys.argv)>1:\n sys.path.insert(0, sys.argv[1])\n"
             " try: import triune_b200\n except Exception: ok=False\n"
             "print(json.dumps({'torch':t,'cuda':c,'package':ok}))")
    best = None
    seen = set()
    for py in tried:
        if py in seen:
            continue
        seen.add(py)
        if run(["wsl.exe", "-e", "test", "-x", py], 3.0)[0] != 0:
            continue
        code, out = run(["wsl.exe", "-e", py, "-c", probe] + ([ws] if ws else []), 60.0)
        if code != 0:
            continue
        try:
            info = json.loads(out.strip().splitlines()[-1])
        except (ValueError, IndexError):
            continue
        if not info.get("torch") or not info.get("package", True):
            continue
        found = {"python": py, "cuda": bool(info.get("cuda")), "torch": info["torch"], "workspace": ws}
        if found["cuda"]:
            return found
        best = best or found
    return best


def wsl_server_command(wsl: dict, port: int, model: Optional[str] = None, precision: Optional[str] = None) -> List[str]:
    """``wsl.exe`` command line that serves on the guest's loopback (forwarded to the host by WSL; never a wildcard bind)."""
    inner = [wsl["python"], "-m", "triune_b200", "serve", "--host", "127.0.0.1", "--port", str(int(port))]
    if model:
        inner += ["--model", model]
    if precision:
        inner += ["--precision", precision]
    cmd = ["wsl.exe"]
    if wsl.get("workspace"):
        cmd += ["--cd", wsl["workspace"]]
    return cmd + ["-e"] + inner


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


def _local_cuda() -> bool:
    try:
        import torch

        return bool(torch.cuda.is_available())
    except Exception:
        return False


def start_session(port: int = 8000, host: str = "127.0.0.1", model: Optional[str] = None, static_dir: Optional[str] = None,
                  precision: Optional[str] = None, startup_timeout: float = 120.0, quiet: bool = False,
                  allow_wsl: bool = False, run: Runner = _run, popen=subprocess.Popen, platform: str = sys.platform) -> DesktopSession:
    """Find or start the server and return once it is healthy. With ``allow_wsl`` on a Windows host whose own PyTorch
    sees no GPU, the server is started inside WSL 2 when an interpreter there can serve this package."""
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
    cmd = server_command(port, host, model, static_dir, precision)
    if allow_wsl and platform == "win32" and not _local_cuda():
        wsl = find_wsl_python(root, run=run)
        if wsl is not None:
            say(f"starting the server inside WSL 2 with {wsl['python']} (torch {wsl['torch']}, GPU {'yes' if wsl['cuda'] else 'no'})")
            cmd = wsl_server_command(wsl, port, model, precision)
        else:
            say("no usable interpreter was found inside WSL 2; starting the server on this host")
    proc = popen(cmd, env=env, stdout=out, stderr=out)
    if not wait_for_server(port, host, startup_timeout, proc):
        code = proc.poll()
        DesktopSession(port, host, proc, False).stop()
        raise RuntimeError(f"the server did not come up on port {port}" + (f" (exit code {code})" if code is not None else ""))
    say(f"server ready on http://{host}:{port}/")
    return DesktopSession(port, host, proc, False)


def launch_desktop_app(port: int = 8000, use_browser: bool = True, host: str = "127.0.0.1", model: Optional[str] = None,
                       static_dir: Optional[str] = None, precision: Optional[str] = None, block: bool = True,
                       allow_wsl: bool = False) -> DesktopSession:
    """Start or reuse the server, open the page, and (``block``) stay until Ctrl-C or until the server exits."""
    session = start_session(port, host, model, static_dir, precision, allow_wsl=allow_wsl)
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
