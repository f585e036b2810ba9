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


def _is_curated_copy(info: "PluginInfo") -> bool:
    """True when the plugin's entry file is byte for byte the one of a module shipped in ``plugins/curated``."""
    try:
        from .curated import curated_path

        shipped = curated_path(info.name) / info.entry
        return shipped.is_file() and hmac.compare_digest(file_sha256(shipped), file_sha256(info.path / info.entry))
    except (KeyError, OSError):
        return False


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

        bare = _is_curated_copy(info)

        def reg(name, inputs, outputs, description="", optional=()):
            full = f"{info.name}.{name}"
            info.nodes.append(full)
            deco = dag.register_node(full, inputs, outputs, description, optional)
            if not bare:
                return deco
            # modules that ship with the framework also answer to the plain node name, which is what saved graphs use
            info.nodes.append(name)
            plain = dag.register_node(name, inputs, outputs, description, optional)
            return lambda fn: plain(deco(fn))

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


_SCAFFOLD = '''"""Plugin {name}: registers DAG nodes. Edit, then re-sign the manifest (the digest covers this file)."""


def register(api):
    @api.register_node("echo", {{"value": "any"}}, {{"out": "any"}}, "returns its input unchanged")
    def echo(inputs, params, context):
        return {{"out": inputs.get("value")}}
'''


def write_manifest(plugin_dir, key: Optional[str] = None) -> Dict[str, Any]:
    """(Re)compute the entry file's digest, sign when a key is given (or configured in ``TRIUNE_PLUGIN_KEY``) and write
    ``plugin.json``. Run after every edit of the entry file. Same job as the reference's
    ``scripts/sign_plugin_manifest.py``."""
    d = Path(plugin_dir)
    man_path = d / "plugin.json"
    man = json.loads(man_path.read_text()) if man_path.is_file() else {"name": d.name, "version": "0.1.0", "entry": "plugin.py"}
    entry = (d / man["entry"]).resolve()
    if d.resolve() not in entry.parents or not entry.is_file():
        raise PluginError(f"{man.get('name', d.name)}: entry file {man['entry']!r} is missing or outside the plugin directory")
    man["sha256"] = file_sha256(entry)
    key = key if key is not None else os.environ.get("TRIUNE_PLUGIN_KEY") or None
    if key:
        man["signature"] = sign_manifest(man["name"], str(man["version"]), man["sha256"], key)
    else:
        man.pop("signature", None)
    man_path.write_text(json.dumps(man, indent=2) + "\n")
    return man


def create_plugin(directory, name: str, key: Optional[str] = None, version: str = "0.1.0") -> Path:
    """Scaffold ``directory/name`` with an entry file that registers one node, and a (signed) manifest."""
    if not name.replace("_", "").replace("-", "").isalnum():
        raise PluginError("plugin names are letters, digits, '-' and '_'")
    d = Path(directory) / name
    if d.exists():
        raise PluginError(f"{d} already exists")
    d.mkdir(parents=True)
    (d / "plugin.py").write_text(_SCAFFOLD.format(name=name))
    (d / "plugin.json").write_text(json.dumps({"name": name, "version": version, "entry": "plugin.py"}))
    write_manifest(d, key)
    return d
