"""Launcher bundles for the three desktop platforms, generated as plain files (no compiler, no installer toolchain).

Each bundle is a small directory the platform's shell knows how to start, whose only job is to find a Python
interpreter and run ``python -m triune_b200 desktop``:

* Linux: an AppDir (``AppRun``, a ``.desktop`` entry, an icon) that AppImage tools can wrap as is;
* macOS: an ``.app`` directory (``Info.plist`` + ``Contents/MacOS/launcher``);
* Windows: a ``.cmd`` launcher next to a PowerShell script that creates a Start-menu shortcut to it.

The bundles point at the source tree they were generated from (``workspace``) and fall back to the directory they sit
in, so a copied tree keeps working. Covers the reference's ``triune/packaging.py:42-297`` (which builds a WPF host and
installers around its Studio front-end; neither exists here, so those parts are not reproduced).
"""

from __future__ import annotations

import os
import stat
from pathlib import Path
from typing import Any, Dict

APP_NAME = "Triune B200"
APP_ID = "triune-b200"
WORKSPACE_ROOT = Path(__file__).resolve().parent.parent

ICON_SVG = """<svg xmlns="http://www.w3.org/2000/svg" viewBox="0 0 96 96">
<rect width="96" height="96" rx="18" fill="#10151c"/>
<path d="M48 14 L80 70 H16 Z" fill="none" stroke="#76b900" stroke-width="6" stroke-linejoin="round"/>
<circle cx="48" cy="52" r="7" fill="#76b900"/>
</svg>
"""


def _write(path: Path, text: str, executable: bool = False) -> Path:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(text, encoding="utf-8")
    if executable:
        path.chmod(path.stat().st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
    return path


def _posix_launcher(workspace: Path, up: str) -> str:
    """A bash launcher: the recorded workspace if it still exists, else ``up`` levels above the script."""
    return f"""#!/usr/bin/env bash
set -e
ROOT="{workspace.as_posix()}"
if [ ! -d "$ROOT/triune_b200" ]; then
    ROOT="$(cd "$(dirname "$0")/{up}" && pwd)"
fi
export PYTHONPATH="$ROOT${{PYTHONPATH:+:$PYTHONPATH}}"
for PY in "$ROOT/.venv/bin/python" "$(command -v python3 || true)" "$(command -v python || true)"; do
    if [ -n "$PY" ] && [ -x "$PY" ]; then
        exec "$PY" -m triune_b200 desktop "$@"
    fi
done
echo "{APP_NAME}: no Python interpreter found" >&2
exit 127
"""


def build_linux_bundle(workspace: Path = WORKSPACE_ROOT, out_dir: Path | None = None) -> Dict[str, Any]:
    out = Path(out_dir) if out_dir else workspace / "dist" / "linux"
    appdir = out / f"{APP_ID}.AppDir"
    run = _write(appdir / "AppRun", _posix_launcher(workspace, "../../.."), executable=True)
    _write(appdir / "usr" / "bin" / APP_ID, _posix_launcher(workspace, "../../../../.."), executable=True)
    entry = _write(appdir / f"{APP_ID}.desktop", "\n".join([
        "[Desktop Entry]", "Type=Application", f"Name={APP_NAME}", f"Exec={APP_ID}", f"Icon={APP_ID}",
        "Categories=Development;Science;", "Terminal=true", ""]))
    _write(appdir / "usr" / "share" / "applications" / f"{APP_ID}.desktop", entry.read_text())
    _write(appdir / f"{APP_ID}.svg", ICON_SVG)
    _write(appdir / "usr" / "share" / "icons" / "hicolor" / "scalable" / "apps" / f"{APP_ID}.svg", ICON_SVG)
    return {"platform": "linux", "bundle": str(appdir), "entry": str(run)}


def build_macos_bundle(workspace: Path = WORKSPACE_ROOT, out_dir: Path | None = None) -> Dict[str, Any]:
    out = Path(out_dir) if out_dir else workspace / "dist" / "macos"
    app = out / f"{APP_NAME}.app"
    launcher = _write(app / "Contents" / "MacOS" / "launcher", _posix_launcher(workspace, "../../../../.."), executable=True)
    _write(app / "Contents" / "Info.plist", f"""<?xml version="1.0" encoding="UTF-8"?>
<!DOCTYPE plist PUBLIC "-//Apple//DTD PLIST 1.0//EN" "http://www.apple.com/DTDs/PropertyList-1.0.dtd">
<plist version="1.0"><dict>
<key>CFBundleName</key><string>{APP_NAME}</string>
<key>CFBundleIdentifier</key><string>org.{APP_ID}.launcher</string>
<key>CFBundleExecutable</key><string>launcher</string>
<key>CFBundlePackageType</key><string>APPL</string>
<key>CFBundleShortVersionString</key><string>1.0</string>
<key>LSMinimumSystemVersion</key><string>11.0</string>
</dict></plist>
""")
    _write(app / "Contents" / "Resources" / f"{APP_ID}.svg", ICON_SVG)
    return {"platform": "macos", "bundle": str(app), "entry": str(launcher)}


def build_windows_bundle(workspace: Path = WORKSPACE_ROOT, out_dir: Path | None = None) -> Dict[str, Any]:
    out = Path(out_dir) if out_dir else workspace / "dist" / "windows"
    win_root = str(workspace).replace("/", "\\")
    cmd = _write(out / f"{APP_ID}.cmd", "\r\n".join([
        "@echo off", "setlocal", f'set "ROOT={win_root}"', 'if not exist "%ROOT%\\triune_b200" set "ROOT=%~dp0..\\.."',
        'set "PYTHONPATH=%ROOT%;%PYTHONPATH%"',
        'if exist "%ROOT%\\.venv\\Scripts\\python.exe" ("%ROOT%\\.venv\\Scripts\\python.exe" -m triune_b200 desktop %* & exit /b %ERRORLEVEL%)',
        "where py >nul 2>nul && (py -3 -m triune_b200 desktop %* & exit /b %ERRORLEVEL%)",
        "python -m triune_b200 desktop %*", "exit /b %ERRORLEVEL%", ""]))
    _write(out / "install-shortcut.ps1", "\r\n".join([
        "$target = Join-Path $PSScriptRoot '" + f"{APP_ID}.cmd" + "'",
        "$menu = [Environment]::GetFolderPath('Programs')",
        "$link = (New-Object -ComObject WScript.Shell).CreateShortcut((Join-Path $menu '" + f"{APP_NAME}.lnk" + "'))",
        "$link.TargetPath = $target", "$link.WorkingDirectory = $PSScriptRoot", "$link.Save()", ""]))
    return {"platform": "windows", "bundle": str(out), "entry": str(cmd)}


def build_native_targets(target: str = "all", workspace: Path = WORKSPACE_ROOT, out_dir: Path | None = None) -> Dict[str, Any]:
    """Generate the bundle(s) for ``target``: linux, macos, windows or all. Returns one record per platform."""
    t = target.lower().strip()
    builders = {"linux": build_linux_bundle, "macos": build_macos_bundle, "windows": build_windows_bundle}
    alias = {"mac": "macos", "darwin": "macos", "win": "windows", "win32": "windows"}
    t = alias.get(t, t)
    if t != "all" and t not in builders:
        raise ValueError(f"unknown packaging target {target!r}: linux, macos, windows or all")
    base = Path(out_dir) if out_dir else None
    res = {}
    for name, fn in builders.items():
        if t in ("all", name):
            res[name] = fn(Path(workspace), base / name if base else None)
    return res


# the reference's names of the same builders and of the icon (``triune/packaging.py:20-283``)
TRIUNE_SVG_ICON = ICON_SVG
build_linux_native = build_linux_bundle
build_macos_native = build_macos_bundle
build_windows_native = build_windows_bundle
