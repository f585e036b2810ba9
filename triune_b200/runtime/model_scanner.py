"""Discovery of models on the local machine.

Parity (``triune/runtime/model_scanner.py:92-1196``): walks the usual locations (working directory checkpoints, the
Hugging Face hub cache, Ollama's store, LM Studio / vLLM style folders, loose GGUF files, NVFP4 disk caches, LoRA adapter
folders) and classifies what it finds with size, format and, where cheaply available, architecture facts read from the
file headers (never loading weights).
"""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional

DEFAULT_ROOTS = ("checkpoints_full", "checkpoints", "models", "adapters", "exports", "~/.cache/huggingface/hub", "~/.ollama/models",
                 "~/.cache/lm-studio/models", "~/.lmstudio/models", "~/.cache/triune_b200/nvfp4", "/usr/share/ollama/.ollama/models")
_SKIP_DIRS = {".git", "__pycache__", "node_modules", ".venv", "venv", "site-packages"}


def _size(path: Path) -> int:
    if path.is_file():
        return path.stat().st_size
    return sum(f.stat().st_size for f in path.rglob("*") if f.is_file())


def _hf_dir_info(d: Path) -> Dict[str, Any]:
    info: Dict[str, Any] = {}
    try:
        cfg = json.loads((d / "config.json").read_text())
        for k in ("model_type", "architectures", "hidden_size", "hidden_dim", "num_hidden_layers", "num_layers", "vocab_size",
                  "num_attention_heads", "num_key_value_heads", "num_local_experts", "num_experts", "torch_dtype"):
            if k in cfg:
                info[k] = cfg[k]
    except (OSError, ValueError):
        pass
    return info


def classify(path: Path) -> Optional[Dict[str, Any]]:
    """One entry for a file or directory that is a model artefact, else None."""
    try:
        if path.is_file():
            suf = path.suffix.lower()
            if suf == ".gguf":
                from .gguf_loader import read_gguf_directory

                entry = {"kind": "gguf", "format": "GGUF"}
                try:
                    d = read_gguf_directory(path, load_tokenizer_arrays=False)
                    m = d["metadata"]
                    arch = m.get("general.architecture")
                    entry.update(architecture=arch, name=m.get("general.name"), tensors=len(d["tensors"]),
                                 layers=m.get(f"{arch}.block_count"), hidden_size=m.get(f"{arch}.embedding_length"))
                except Exception as e:
                    entry["error"] = str(e)
                return {**entry, "path": str(path), "size_bytes": path.stat().st_size}
            if suf in (".pt", ".pth", ".ckpt") and path.stat().st_size > 4096:
                return {"kind": "checkpoint", "format": "torch", "path": str(path), "size_bytes": path.stat().st_size}
            return None
        if (path / "manifest.json").is_file() and (path / "layers").is_dir():
            m = json.loads((path / "manifest.json").read_text())
            return {"kind": "nvfp4_cache", "format": m.get("format", "nvfp4"), "path": str(path), "layers": m.get("num_layers"),
                    "source": m.get("source"), "size_bytes": _size(path)}
        if (path / "adapter_config.json").is_file():
            m = json.loads((path / "adapter_config.json").read_text())
            return {"kind": "lora_adapter", "format": "peft", "path": str(path), "rank": m.get("r"), "base_model": m.get("base_model_name_or_path"),
                    "size_bytes": _size(path)}
        if (path / "config.json").is_file() and (any(path.glob("*.safetensors")) or any(path.glob("pytorch_model*.bin"))):
            info = _hf_dir_info(path)
            kind = "triune_hf_bundle" if info.get("model_type") == "triune" else "hf_model"
            return {"kind": kind, "format": "safetensors" if any(path.glob("*.safetensors")) else "bin", "path": str(path),
                    "size_bytes": _size(path), **info}
    except OSError:
        return None
    return None


def _ollama_entries(root: Path) -> List[Dict[str, Any]]:
    out = []
    man = root / "manifests"
    if not man.is_dir():
        return out
    for f in man.rglob("*"):
        if not f.is_file():
            continue
        try:
            layers = json.loads(f.read_text()).get("layers", [])
        except (OSError, ValueError):
            continue
        for layer in layers:
            if str(layer.get("mediaType", "")).endswith("image.model"):
                blob = root / "blobs" / str(layer.get("digest", "")).replace(":", "-")
                parts = f.relative_to(man).parts
                out.append({"kind": "ollama", "format": "GGUF", "name": f"{'/'.join(parts[1:-1])}:{parts[-1]}", "path": str(blob),
                            "size_bytes": int(layer.get("size", 0)), "exists": blob.is_file()})
    return out


def scan_models(roots: Optional[Iterable[str]] = None, max_depth: int = 4, limit: int = 2000) -> Dict[str, Any]:
    found: List[Dict[str, Any]] = []
    seen = set()
    for r in (roots or DEFAULT_ROOTS):
        root = Path(os.path.expanduser(str(r)))
        if not root.exists():
            continue
        if (root / "manifests").is_dir() and (root / "blobs").is_dir():
            found.extend(_ollama_entries(root))
            continue
        stack = [(root, 0)]
        while stack and len(found) < limit:
            d, depth = stack.pop()
            key = str(d.resolve()) if d.exists() else str(d)
            if key in seen:
                continue
            seen.add(key)
            e = classify(d)
            if e is not None:
                found.append(e)
                if d.is_dir():
                    continue  # a model directory is one entry; do not list its shards again
            if d.is_dir() and depth < max_depth:
                try:
                    for c in sorted(d.iterdir()):
                        if c.name in _SKIP_DIRS or c.name.startswith("."):
                            if c.name != ".cache":
                                continue
                        stack.append((c, depth + 1))
                except OSError:
                    pass
    by_kind: Dict[str, int] = {}
    for e in found:
        by_kind[e["kind"]] = by_kind.get(e["kind"], 0) + 1
    return {"models": found, "counts": by_kind, "total_bytes": sum(int(e.get("size_bytes", 0)) for e in found)}


# ---------------------------------------------------------------------------------------------------- a local Ollama daemon
OLLAMA_URL = "http://127.0.0.1:11434"


def _loopback(url: str) -> bool:
    from urllib.parse import urlparse

    host = (urlparse(url).hostname or "").lower()
    return host in ("127.0.0.1", "localhost", "::1")


def query_ollama_running_tags(base_url: str = OLLAMA_URL, timeout: float = 0.4) -> List[str]:
    """Model tags a local Ollama daemon offers (``GET /api/tags``); an empty list when nothing answers on the loopback
    address. Only loopback URLs are contacted (``triune/runtime/model_scanner.py:213-286`` of the reference)."""
    import urllib.request

    if not _loopback(base_url):
        return []
    try:
        with urllib.request.urlopen(base_url.rstrip("/") + "/api/tags", timeout=timeout) as r:
            data = json.loads(r.read().decode("utf-8", "replace"))
    except (OSError, ValueError):
        return []
    return [str(m.get("name")) for m in data.get("models", []) if isinstance(m, dict) and m.get("name")]


def stream_ollama_chat(model: str, messages: List[Dict[str, str]], base_url: str = OLLAMA_URL, options: Optional[Dict[str, Any]] = None,
                       timeout: float = 120.0):
    """Yield the text pieces of a chat answered by a local Ollama daemon (``POST /api/chat`` with ``stream: true``: one
    JSON object per line). Raises ``ConnectionError`` when the daemon does not answer; refuses non-loopback URLs."""
    import urllib.request

    if not _loopback(base_url):
        raise ValueError("only a daemon on the loopback address is contacted")
    body = json.dumps({"model": model, "messages": messages, "stream": True, **({"options": options} if options else {})}).encode()
    req = urllib.request.Request(base_url.rstrip("/") + "/api/chat", data=body, headers={"Content-Type": "application/json"}, method="POST")
    try:
        resp = urllib.request.urlopen(req, timeout=timeout)
    except OSError as e:
        raise ConnectionError(f"no Ollama daemon answers at {base_url}: {e}") from e
    with resp:
        for raw in resp:
            line = raw.decode("utf-8", "replace").strip()
            if not line:
                continue
            try:
                obj = json.loads(line)
            except ValueError:
                continue
            if obj.get("error"):
                raise RuntimeError(str(obj["error"]))
            piece = (obj.get("message") or {}).get("content")
            if piece:
                yield piece
            if obj.get("done"):
                break
