"""Installer: set this framework up on a machine, as a plan of steps that can be shown before it is run.

``python -m triune_b200 install [--venv DIR] [--find-links WHEELS] [--offline] [--no-build] [--no-shortcuts] [--dry-run]``

What it does: looks at the machine (operating system, WSL, NVIDIA driver and GPUs through ``nvidia-smi``, ``nvcc``,
the interpreter's version), decides what this machine can run (the sm_100a kernels need Linux, an NVIDIA GPU of
compute capability 10.x and the CUDA compiler; anything else gets the PyTorch reference paths and is told so), and
produces an ordered list of steps: create a virtual environment, install PyTorch and the Python dependencies (from an
index, or from a local wheel directory with ``--offline`` / ``--find-links``), build the CUDA extensions in-tree,
generate the launcher bundle for this platform, and verify the result by importing the package and running one tiny
CPU forward pass in the new environment. ``--dry-run`` prints the plan and changes nothing.

Every external command goes through one injectable runner, so the planner and the executor are tested on a CPU box
with a fake runner. Counterpart in the reference: ``studio/installer/installer.py`` (hardware profile, virtual
environment, accelerator-specific PyTorch wheels, desktop shortcuts, health check) with its ``install_studio.sh`` /
``install_studio.bat`` front ends; the wheel choice here is a single one (CUDA 12.x builds of PyTorch for Blackwell),
because this framework targets one GPU family.
"""

from __future__ import annotations

import json
import platform
import shutil
import subprocess
import sys
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

WORKSPACE_ROOT = Path(__file__).resolve().parent.parent
MIN_PYTHON = (3, 10)
# what the package imports at run time; the serving extras are optional and listed apart
CORE_REQUIREMENTS = ("numpy", "pyyaml", "einops", "tqdm", "psutil", "pybind11", "ninja")
SERVE_REQUIREMENTS = ("fastapi", "uvicorn", "pydantic")
EXTRA_REQUIREMENTS = ("tokenizers", "safetensors", "pyarrow", "transformers")
TORCH_INDEX = "https://download.pytorch.org/whl/cu128"

# (argv, cwd, timeout) -> (exit code, combined output)
Runner = Callable[[Sequence[str], Optional[str], float], Tuple[int, str]]


def system_runner(argv: Sequence[str], cwd: Optional[str] = None, timeout: float = 3600.0) -> Tuple[int, str]:
    try:
        r = subprocess.run(list(argv), cwd=cwd, capture_output=True, text=True, timeout=timeout)
        return r.returncode, (r.stdout or "") + (r.stderr or "")
    except FileNotFoundError:
        return 127, f"{argv[0]}: not found"
    except subprocess.TimeoutExpired:
        return 124, f"{argv[0]}: timed out after {timeout:.0f} s"
    except OSError as e:
        return 126, f"{argv[0]}: {e}"


@dataclass
class MachineProfile:
    os_type: str = ""
    arch: str = ""
    python: Tuple[int, int] = (0, 0)
    is_wsl: bool = False
    gpus: List[Dict[str, Any]] = field(default_factory=list)  # name, memory_gb, compute_capability
    driver: Optional[str] = None
    nvcc: Optional[str] = None  # release string, e.g. "12.9"
    notes: List[str] = field(default_factory=list)

    @property
    def blackwell(self) -> bool:
        return any(str(g.get("compute_capability", "")).startswith("10.") for g in self.gpus)

    @property
    def can_build_kernels(self) -> bool:
        return self.os_type == "Linux" and self.blackwell and self.nvcc is not None

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.update(blackwell=self.blackwell, can_build_kernels=self.can_build_kernels)
        return d


def probe_machine(run: Runner = system_runner, os_type: Optional[str] = None, proc_version: Optional[str] = None) -> MachineProfile:
    m = MachineProfile(os_type=os_type or platform.system(), arch=platform.machine(), python=tuple(sys.version_info[:2]))
    if m.os_type == "Linux":
        if proc_version is None:
            try:
                proc_version = Path("/proc/version").read_text(encoding="utf-8", errors="replace")
            except OSError:
                proc_version = ""
        m.is_wsl = "microsoft" in proc_version.lower()
    code, out = run(["nvidia-smi", "--query-gpu=name,memory.total,driver_version,compute_cap", "--format=csv,noheader,nounits"], None, 10.0)
    if code == 0:
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 2:
                try:
                    mem = round(float(parts[1]) / 1024.0, 1)
                except ValueError:
                    continue
                m.gpus.append({"name": parts[0], "memory_gb": mem, "compute_capability": parts[3] if len(parts) > 3 else ""})
                if len(parts) > 2:
                    m.driver = parts[2]
    code, out = run(["nvcc", "--version"], None, 10.0)
    if code == 0:
        for tok in out.replace(",", " ").split():
            if tok[:1].isdigit() and "." in tok and "release" in out:
                m.nvcc = tok
                break
    if m.python < MIN_PYTHON:
        m.notes.append(f"Python {m.python[0]}.{m.python[1]} is older than the supported {MIN_PYTHON[0]}.{MIN_PYTHON[1]}")
    if not m.gpus:
        m.notes.append("no NVIDIA GPU was found: the PyTorch reference paths run on the CPU; the CUDA kernels are not built")
    elif not m.blackwell:
        m.notes.append("the GPUs here are not compute capability 10.x: the sm_100a kernels do not run on them; PyTorch paths are used")
    elif m.os_type != "Linux":
        m.notes.append("the kernels are built and run on Linux (on Windows: inside WSL 2)")
    elif m.nvcc is None:
        m.notes.append("nvcc was not found: install the CUDA toolkit (12.8 or newer) to build the sm_100a kernels")
    return m


@dataclass
class Step:
    name: str
    argv: List[str]
    why: str
    cwd: Optional[str] = None
    optional: bool = False  # a failure is reported but does not stop the installation
    timeout: float = 3600.0


def venv_python(venv: Path, os_type: str) -> Path:
    return venv / ("Scripts/python.exe" if os_type == "Windows" else "bin/python")


def plan_install(machine: MachineProfile, venv: Optional[Path] = None, find_links: Optional[str] = None, offline: bool = False,
                 build: bool = True, shortcuts: bool = True, extras: bool = True, base_python: str = sys.executable,
                 workspace: Path = WORKSPACE_ROOT) -> List[Step]:
    """The ordered steps for this machine. Without ``venv`` the current interpreter is used as it is."""
    steps: List[Step] = []
    py = base_python
    if venv is not None:
        py = str(venv_python(venv, machine.os_type))
        if Path(py).exists():
            steps.append(Step("check-venv", [py, "-c", "import sys; print(sys.prefix)"], "the environment exists already"))
        else:
            # offline without wheels the environment has to see the packages that are installed already
            steps.append(Step("create-venv", [base_python, "-m", "venv"] + (["--system-site-packages"] if offline and not find_links else []) + [str(venv)],
                              "an isolated interpreter for the framework"))
    pip = [py, "-m", "pip", "install", "--disable-pip-version-check"]
    src = (["--no-index"] if offline else []) + (["--find-links", find_links] if find_links else [])
    if offline and not find_links:
        steps.append(Step("check-torch", [py, "-c", "import torch; print(torch.__version__)"],
                          "offline without a wheel directory: PyTorch must be present already"))
    else:
        steps.append(Step("install-torch", pip + src + (["--index-url", TORCH_INDEX] if not offline and not find_links else []) + ["torch"],
                          "PyTorch built for CUDA 12.8+ (Blackwell)" if machine.gpus else "PyTorch (CPU paths only on this machine)"))
        steps.append(Step("install-core", pip + src + list(CORE_REQUIREMENTS), "run-time dependencies of the package"))
        steps.append(Step("install-serve", pip + src + list(SERVE_REQUIREMENTS), "the HTTP server and Studio page", optional=True))
        if extras:
            steps.append(Step("install-extras", pip + src + list(EXTRA_REQUIREMENTS),
                              "tokenizer files, safetensors, parquet corpora, foreign checkpoints", optional=True))
    if build and machine.can_build_kernels:
        steps.append(Step("build-kernels", [py, "-m", "triune_b200", "native"], "compile the sm_100a CUDA extensions in-tree",
                          cwd=str(workspace), timeout=7200.0))
    if shortcuts:
        target = {"Linux": "linux", "Darwin": "macos", "Windows": "windows"}.get(machine.os_type)
        if target:
            steps.append(Step("launcher", [py, "-m", "triune_b200", "package", "--target", target],
                              "launcher bundle for this platform (start the server, open the Studio page)", cwd=str(workspace), optional=True))
    verify = ("import torch, triune_b200\n"
              "from triune_b200.models.zoo import load_model\n"
              "m = load_model('default', vocab_size=64, hidden_dim=32, num_layers=4, num_heads=1, head_dim=32, num_experts=2,\n"
              "               router_prefix_layers=1, reflex_exit_layer=2, limbic_exit_layer=3)\n"
              "y = m(torch.randint(0, 64, (1, 8)), force_depth=2)[0]\n"
              "assert y.shape == (1, 8, 64) and torch.isfinite(y).all()\n"
              "print('ok', torch.__version__, 'cuda' if torch.cuda.is_available() else 'cpu')\n")
    steps.append(Step("verify", [py, "-c", verify], "import the package and run one tiny forward pass", cwd=str(workspace), timeout=600.0))
    return steps


def run_plan(steps: Sequence[Step], run: Runner = system_runner, say: Callable[[str], None] = print, dry_run: bool = False) -> Dict[str, Any]:
    """Run the steps in order; a failing required step stops the run. Returns a record of what happened."""
    record: List[Dict[str, Any]] = []
    ok = True
    for k, st in enumerate(steps, 1):
        say(f"[{k}/{len(steps)}] {st.name}: {st.why}")
        if dry_run:
            say("      " + " ".join(_quote(a) for a in st.argv))
            record.append({"step": st.name, "status": "planned"})
            continue
        code, out = run(st.argv, st.cwd, st.timeout)
        tail = "\n".join(out.strip().splitlines()[-6:])
        if code == 0:
            record.append({"step": st.name, "status": "done"})
            continue
        record.append({"step": st.name, "status": "failed" if not st.optional else "skipped", "exit_code": code, "output": tail})
        say(f"      {'warning' if st.optional else 'error'}: exit code {code}\n{_indent(tail)}")
        if not st.optional:
            ok = False
            break
    return {"ok": ok, "dry_run": dry_run, "steps": record}


def _quote(a: str) -> str:
    return a if a and all(c.isalnum() or c in "-_./:=+,@" for c in a) else json.dumps(a)


def _indent(text: str, pad: str = "      ") -> str:
    return "\n".join(pad + l for l in text.splitlines())


def install(venv: Optional[str] = None, find_links: Optional[str] = None, offline: bool = False, build: bool = True,
            shortcuts: bool = True, extras: bool = True, dry_run: bool = False, run: Runner = system_runner,
            say: Callable[[str], None] = print) -> Dict[str, Any]:
    machine = probe_machine(run)
    say(f"machine: {machine.os_type} {machine.arch}{' (WSL)' if machine.is_wsl else ''}, Python {machine.python[0]}.{machine.python[1]}, "
        f"GPUs: {', '.join(g['name'] for g in machine.gpus) or 'none'}, driver {machine.driver or '-'}, nvcc {machine.nvcc or '-'}")
    for n in machine.notes:
        say("note: " + n)
    if machine.python < MIN_PYTHON:
        return {"ok": False, "machine": machine.to_dict(), "steps": [], "error": machine.notes[0]}
    steps = plan_install(machine, Path(venv).expanduser() if venv else None, find_links, offline, build, shortcuts, extras)
    out = run_plan(steps, run, say, dry_run)
    out["machine"] = machine.to_dict()
    if out["ok"] and not dry_run:
        say("installed. Start with:  python -m triune_b200 desktop    (or: python -m triune_b200 serve)")
    return out


def write_bootstrap_scripts(out_dir: Path, workspace: Path = WORKSPACE_ROOT) -> Dict[str, str]:
    """``install.sh`` and ``install.bat``: find a Python, then hand over to ``python -m triune_b200 install``. On Windows
    the script prefers WSL 2 when it has one (the kernels build there) and falls back to a CPU installation on the host."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    sh = f"""#!/usr/bin/env sh
# Installs the framework that lives in {workspace.name}/ into a virtual environment next to it.
set -e
HERE="$(cd "$(dirname "$0")" && pwd)"
ROOT="${{TRIUNE_ROOT:-$HERE/..}}"
PY="${{PYTHON:-}}"
if [ -z "$PY" ]; then
  for c in python3.12 python3.11 python3.10 python3 python; do
    if command -v "$c" >/dev/null 2>&1; then PY="$c"; break; fi
  done
fi
[ -n "$PY" ] || {{ echo "No Python interpreter was found (3.10 or newer is needed)." >&2; exit 1; }}
cd "$ROOT"
exec "$PY" -m triune_b200 install --venv "${{TRIUNE_VENV:-$ROOT/.venv}}" "$@"
"""
    bat = f"""@echo off
rem Installs the framework that lives in {workspace.name}\\ . With WSL 2 present the installation runs inside it (GPU kernels);
rem otherwise a CPU installation is made with the Python of this host.
setlocal
set "ROOT=%~dp0.."
wsl.exe --status >nul 2>&1
if %ERRORLEVEL%==0 (
  for /f "usebackq delims=" %%p in (`wsl.exe wslpath -a "%ROOT%"`) do set "WROOT=%%p"
  wsl.exe --cd "%WROOT%" -e sh dist/install.sh %*
  exit /b %ERRORLEVEL%
)
where py >nul 2>&1 && (set "PY=py -3") || (set "PY=python")
cd /d "%ROOT%"
%PY% -m triune_b200 install --venv "%ROOT%\\.venv" %*
exit /b %ERRORLEVEL%
"""
    p_sh, p_bat = out_dir / "install.sh", out_dir / "install.bat"
    p_sh.write_text(sh, encoding="utf-8", newline="\n")
    p_sh.chmod(0o755)
    p_bat.write_text(bat, encoding="utf-8", newline="\r\n")
    return {"sh": str(p_sh), "bat": str(p_bat)}


def uninstall(venv: str, dist_dir: Optional[str] = None, dry_run: bool = False) -> Dict[str, Any]:
    """Remove what ``install`` created: the virtual environment (only if it is one) and the generated launcher bundles."""
    removed, kept = [], []
    v = Path(venv).expanduser()
    if (v / "pyvenv.cfg").is_file():
        removed.append(str(v))
        if not dry_run:
            shutil.rmtree(v)
    elif v.exists():
        kept.append(f"{v} (no pyvenv.cfg: not a virtual environment, left alone)")
    d = Path(dist_dir).expanduser() if dist_dir else WORKSPACE_ROOT / "dist"
    for name in ("linux", "macos", "windows", "install.sh", "install.bat"):
        t = d / name
        if t.exists():
            removed.append(str(t))
            if not dry_run:
                shutil.rmtree(t) if t.is_dir() else t.unlink()
    return {"removed": removed, "kept": kept, "dry_run": dry_run}
