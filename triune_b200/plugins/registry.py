"""Plugin registry with signed manifests (thin version of ``triune/plugins/*.py`` and ``triune/modules/manager.py``).

A plugin is a directory with ``plugin.json`` (``name``, ``version``, ``entry`` Python file, ``sha256`` of that file and an
optional ``signature`` = HMAC-SHA256 of ``name|version|sha256`` under a key the operator configures in
``TRIUNE_PLUGIN_KEY``). Loading verifies the digest always and the signature whenever a key is configured (unsigned
plugins are refused then), imports the entry file and calls its ``register(registry)``, through which the plugin adds
DAG node types. Nothing is downloaded or executed at discovery time.
"""

from __future__ import annotations

import hashlib
import hmac
import importlib.util
import json
import os
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional


class PluginError(RuntimeError):
    pass


@dataclass
class PluginInfo:
    name: str
    version: str
    path: Path
    entry: str
    sha256: str
    signature: Optional[str] = None
    loaded: bool = False
    nodes: List[str] = field(default_factory=list)


def file_sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def sign_manifest(name: str, version: str, sha256: str, key: str) -> str:
    return hmac.new(key.encode(), f"{name}|{version}|{sha256}".encode(), hashlib.sha256).hexdigest()


class PluginRegistry:
    def __init__(self, key: Optional[str] = None):
        self.key = key if key is not None else os.environ.get("TRIUNE_PLUGIN_KEY") or None
        self.plugins: Dict[str, PluginInfo] = {}

    def discover(self, directory) -> List[PluginInfo]:
        out = []
        for man in sorted(Path(directory).glob("*/plugin.json")):
            try:
                m = json.loads(man.read_text())
                info = PluginInfo(m["name"], str(m.get("version", "0")), man.parent, m["entry"], m["sha256"], m.get("signature"))
            except (OSError, ValueError, KeyError):
                continue
            self.plugins.setdefault(info.name, info)
            out.append(info)
        return out

    def verify(self, info: PluginInfo) -> None:
        entry = (info.path / info.entry).resolve()
        if info.path.resolve() not in entry.parents:
            raise PluginError(f"{info.name}: entry file escapes the plugin directory")
        if not entry.is_file() or not hmac.compare_digest(file_sha256(entry), info.sha256):
            raise PluginError(f"{info.name}: entry file digest does not match the manifest")
        if self.key:
            if not info.signature or not hmac.compare_digest(sign_manifest(info.name, info.version, info.sha256, self.key), info.signature):
                raise PluginError(f"{info.name}: missing or invalid signature")

    def register_node(self, info: PluginInfo):
        from ..execution import dag

        def reg(name, inputs, outputs, description="", optional=()):
            full = f"{info.name}.{name}"
            info.nodes.append(full)
            return dag.register_node(full, inputs, outputs, description, optional)

        return reg

    def load(self, name: str) -> PluginInfo:
        info = self.plugins.get(name)
        if info is None:
            raise PluginError(f"unknown plugin {name!r}")
        if info.loaded:
            return info
        self.verify(info)
        spec = importlib.util.spec_from_file_location(f"triune_plugin_{info.name}", info.path / info.entry)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        if not hasattr(mod, "register"):
            raise PluginError(f"{info.name}: entry file defines no register(registry)")
        mod.register(type("PluginAPI", (), {"register_node": staticmethod(self.register_node(info)), "info": info})())
        info.loaded = True
        return info

    def list(self) -> List[Dict[str, Any]]:
        return [{"name": p.name, "version": p.version, "path": str(p.path), "loaded": p.loaded, "nodes": p.nodes,
                 "signed": bool(p.signature)} for p in self.plugins.values()]
