"""Discovery of models on the local machine.

Parity (``triune/runtime/model_scanner.py:92-1196``): walks the usual locations (working directory checkpoints, the
Hugging Face hub cache, Ollama's store, LM Studio / vLLM style folders, loose GGUF files, NVFP4 disk caches, LoRA adapter
folders) and classifies what it finds with size, format and, where cheaply available, architecture facts read from the
file headers (never loading weights).
"""

from __future__ import annotations

import json
import os
import struct
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


# ---------------------------------------------------------------------------------------------------- shapes of models on disk
def resolve_ollama_host(base_url: Optional[str] = None) -> str:
    """Base URL of the local Ollama daemon: the argument, else ``$OLLAMA_HOST``, else the default; a scheme is added when
    missing and a trailing slash removed."""
    host = (base_url or os.environ.get("OLLAMA_HOST") or OLLAMA_URL).strip()
    if not host.startswith(("http://", "https://")):
        host = "http://" + host
    return host.rstrip("/")


def parse_gguf_header(gguf_path, max_kv: int = 96) -> Optional[Dict[str, Any]]:
    """Architecture figures of a GGUF file read from its header only (no tensor data): ``architecture``, ``name``,
    ``num_layers``, ``hidden_dim``, ``num_heads``, ``num_kv_heads``, ``ffn_dim``, ``vocab_size``, ``context_length``,
    ``quantization`` (the most common tensor type) and ``tensors``. None when the file is not GGUF or cannot be read.
    ``max_kv`` is accepted for the reference's signature; the whole key/value table is read (token arrays skipped)."""
    from .gguf_loader import hf_config_from_gguf, read_gguf_directory

    try:
        d = read_gguf_directory(gguf_path, load_tokenizer_arrays=False)
    except (OSError, ValueError, struct.error):
        return None
    meta = d["metadata"]
    cfg = hf_config_from_gguf(meta)
    types: Dict[int, int] = {}
    for t in d["tensors"].values():
        if len(t["shape"]) >= 2:
            types[t["type"]] = types.get(t["type"], 0) + 1
    names = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K",
             14: "Q6_K", 15: "Q8_K", 30: "BF16"}
    top = max(types, key=types.get) if types else None
    arch = cfg["architecture"]
    has = lambda k: meta.get(f"{arch}.{k}") is not None  # noqa: E731
    return {"architecture": arch, "name": meta.get("general.name"), "num_layers": cfg["num_hidden_layers"] if has("block_count") else None,
            "hidden_dim": cfg["hidden_size"] if has("embedding_length") else None,
            "num_heads": cfg["num_attention_heads"] if has("attention.head_count") else None, "num_kv_heads": cfg["num_key_value_heads"],
            "ffn_dim": cfg["intermediate_size"] if has("feed_forward_length") else None, "vocab_size": cfg["vocab_size"],
            "context_length": cfg["max_position_embeddings"], "quantization": names.get(top, None if top is None else f"type{top}"),
            "tensors": len(d["tensors"])}


def scan_pc_models(extra_paths: Optional[List[str]] = None, *, include_wsl: bool = True, max_depth: int = 4,
                   installed_modules: Optional[List[Dict[str, Any]]] = None) -> Dict[str, Any]:
    """``scan_models`` over the default places plus ``extra_paths``, in the report shape of the reference
    (``triune/runtime/model_scanner.py:489-700``): every entry gets an ``id`` (``ollama:<tag>`` for Ollama models, else
    ``<kind>:<path>``), GGUF entries their header figures, Ollama entries whether the daemon lists them. ``include_wsl``
    adds the Linux homes visible from a Windows host (``\\\\wsl$``); ``installed_modules`` are listed as they are."""
    import time

    t0 = time.perf_counter()
    roots = [str(r) for r in DEFAULT_ROOTS] + [str(p) for p in (extra_paths or [])]
    if include_wsl and os.name == "nt":
        roots += [str(h / ".ollama" / "models") for d in Path(r"\\wsl$").glob("*") for h in (d / "home").glob("*")]
    rep = scan_models(roots, max_depth=max_depth)
    live = {t.lower() for t in query_ollama_running_tags()}
    models, seen = [], set()
    for e in rep["models"]:
        e = dict(e)
        if e["kind"] == "ollama":
            e["id"] = f"ollama:{e['name']}".lower()
            e["live"] = e["name"].lower() in live
        else:
            e["id"] = f"{e['kind']}:{e['path']}"
        if e["id"] in seen:
            continue
        seen.add(e["id"])
        if e.get("format") == "GGUF" and Path(e["path"]).is_file():
            head = parse_gguf_header(e["path"])
            if head:
                e.update({k: v for k, v in head.items() if v is not None and k not in e})
        e.setdefault("name", Path(e["path"]).name)
        models.append(e)
    for m in installed_modules or []:
        models.append({**m, "kind": "module", "id": f"module:{m.get('id') or m.get('name')}"})
    return {"models": models, "counts": rep["counts"], "total_bytes": rep["total_bytes"], "scanned_roots": roots,
            "ollama_live_tags": sorted(live), "scan_time_ms": round((time.perf_counter() - t0) * 1e3, 2)}


def inspect_model_spec_for_upgrade(raw_source: str, *, checkpoint_arch_fn=None, fallback_spec: Optional[Dict[str, Any]] = None):
    """(layers, hidden size, heads, FFN size, vocabulary size, label) of whatever ``raw_source`` names: ``ollama:<tag>``,
    a GGUF file, a ``.pt`` / ``.safetensors`` file, an NVFP4 cache or Hugging Face directory; None when it cannot be read.
    Used to size a model before converting it (``triune/runtime/model_scanner.py:1069-1230`` of the reference, which
    also asks the Hugging Face hub about repository ids; that needs the network and is left out here)."""
    raw = str(raw_source or "").strip()
    if not raw:
        return None

    def out(layers, hidden, heads, ffn, vocab, label):
        hidden = int(hidden or 1024)
        return (int(layers or 24), hidden, int(heads or max(1, hidden // 64)), int(ffn or 4 * hidden), int(vocab or 32000), label)

    if raw.lower().startswith("ollama:"):
        from .gguf_loader import resolve_ollama_gguf_blob

        blob = resolve_ollama_gguf_blob(raw[len("ollama:"):])
        if blob is None:
            return None
        head = parse_gguf_header(blob)
        if not head:
            return None
        return out(head["num_layers"], head["hidden_dim"], head["num_heads"], head["ffn_dim"], head["vocab_size"],
                   f"Ollama ({raw[len('ollama:'):]} · {head.get('quantization') or 'GGUF'})")
    p = Path(raw).expanduser()
    if p.is_file() and p.suffix.lower() == ".gguf":
        head = parse_gguf_header(p)
        if head and (head["num_layers"] or head["hidden_dim"]):
            return out(head["num_layers"], head["hidden_dim"], head["num_heads"], head["ffn_dim"], head["vocab_size"],
                       f"{str(head['architecture']).upper()} GGUF ({p.name})")
        return None
    if p.is_file() and p.suffix.lower() == ".safetensors":
        from ..export.safetensors_io import read_header as read_safetensors_header

        try:
            shapes = {k: tuple(v["shape"]) for k, v in read_safetensors_header(p).items() if k != "__metadata__"}
        except (OSError, ValueError, KeyError):
            return None
        return _spec_from_shapes(shapes, f"Saved SafeTensors ({p.name})", out)
    if p.is_file() and p.suffix.lower() in (".pt", ".pth", ".bin", ".ckpt"):
        import torch

        try:
            ck = torch.load(p, map_location="cpu", weights_only=True)
        except Exception:
            return None
        if isinstance(ck, dict) and checkpoint_arch_fn is not None:
            try:
                _, arch = checkpoint_arch_fn(ck, fallback_spec or {})
                cfg = ck.get("config") if isinstance(ck.get("config"), dict) else {}
                return out(arch.get("num_layers"), arch.get("hidden_dim"), arch.get("num_heads"), cfg.get("ffn_dim"), arch.get("vocab_size"),
                           f"Saved Checkpoint ({p.name})")
            except Exception:
                pass
        sd = ck.get("model_state", ck.get("model", ck)) if isinstance(ck, dict) else {}
        shapes = {k: tuple(v.shape) for k, v in sd.items() if hasattr(v, "shape")} if isinstance(sd, dict) else {}
        return _spec_from_shapes(shapes, f"Saved Checkpoint ({p.name})", out) if shapes else None
    if p.is_dir():
        if (p / "manifest.json").is_file():
            try:
                m = json.loads((p / "manifest.json").read_text())
                cfg = m.get("config") or {}
                return out(m.get("num_layers") or cfg.get("num_hidden_layers"), cfg.get("hidden_size"), cfg.get("num_attention_heads"),
                           cfg.get("intermediate_size"), cfg.get("vocab_size"), f"NVFP4 cache ({p.name})")
            except (OSError, ValueError):
                return None
        info = _hf_dir_info(p)
        if info:
            try:
                cfg = json.loads((p / "config.json").read_text())
            except (OSError, ValueError):
                cfg = {}
            return out(info.get("num_hidden_layers") or info.get("num_layers"), info.get("hidden_size") or info.get("hidden_dim"),
                       info.get("num_attention_heads"), cfg.get("intermediate_size") or cfg.get("ffn_dim"), info.get("vocab_size"),
                       f"{str(info.get('model_type') or 'hf').upper()} ({p.name})")
    return None


def _spec_from_shapes(shapes: Dict[str, tuple], label: str, out):
    """Sizes of a decoder from the names and shapes of its tensors: layers from the highest block index, vocabulary and
    width from the embedding matrix, FFN size from the first gate / up / fc1 / expert weight."""
    import re

    idx = [int(m.group(1)) for k in shapes if (m := re.match(r"(?:model\.layers|transformer\.h|layers)\.(\d+)\.", k))]
    emb = next((s for k, s in shapes.items() if "embed" in k and len(s) == 2), None)
    vocab, hidden = (emb if emb else (32000, 384))
    ffn = next((max(s) for k, s in shapes.items() if len(s) >= 2 and any(t in k for t in ("gate_proj", "up_proj", "fc1", "experts.0.0", ".w1"))), None)
    return out(max(idx) + 1 if idx else 8, hidden, None, ffn, vocab, label)
