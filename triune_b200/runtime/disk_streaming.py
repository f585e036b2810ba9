"""NVFP4 disk cache and disk -> host -> device layer streaming for models far larger than memory.

Parity (``triune/runtime/disk_streaming.py:192-805``): ``build_nvfp4_disk_cache`` converts a Hugging Face safetensors
checkpoint shard by shard (the unquantised model never exists in memory) into one safetensors file per layer holding
packed E2M1 weights + scales, a root file (embeddings, norms, head) in bf16, and ``manifest.json`` (version 1);
``DiskNVFP4StreamingEngine`` builds the model skeleton without allocating weights, keeps the root resident and streams
layers NVMe -> pinned host -> device with a one-worker prefetch thread; for QLoRA the backward pass re-stages the
forward-time packed weights.

Differences: scales are true NVFP4 (E4M3 per 16 + fp32 per tensor); packing runs in the quantise kernel on the GPU;
a staged layer is a flat pinned byte buffer moved with one asynchronous copy and decoded by the dequantise kernel on
the side stream, so the next layer's copy and decode overlap the current layer's compute; with 180 GB of HBM the engine
keeps as many decoded layers resident as ``resident_budget_gb`` allows before it starts evicting.
"""

from __future__ import annotations

import json
import os
import re
import shutil
import threading
from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..export.safetensors_io import load_file, read_header, save_file
from ..models.quant_linear import PROTECTED

MANIFEST_VERSION = 1
_AUX_FILES = ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json", "special_tokens_map.json",
              "vocab.json", "merges.txt", "tokenizer.model")
_LAYER_RE = re.compile(r"^(.*?(?:layers|h|blocks))\.(\d+)\.(.+)$")


def default_nvfp4_cache_dir(model_id_or_dir, hadamard: bool = True) -> Path:
    name = re.sub(r"[^A-Za-z0-9_.-]+", "--", str(model_id_or_dir).strip("/"))
    return Path.home() / ".cache" / "triune_b200" / "nvfp4" / f"{name}{'-had' if hadamard else ''}"


def _discover_weight_map(model_dir: Path) -> Dict[str, Path]:
    idx = model_dir / "model.safetensors.index.json"
    if idx.is_file():
        wm = json.loads(idx.read_text())["weight_map"]
        return {k: model_dir / v for k, v in wm.items()}
    out: Dict[str, Path] = {}
    for f in sorted(model_dir.glob("*.safetensors")):
        for k in read_header(str(f)):
            if k != "__metadata__":
                out[k] = f
    if not out:
        raise FileNotFoundError(f"no safetensors weights under {model_dir}")
    return out


class _ShardReader:
    """Reads single tensors out of safetensors shards without loading the shard."""

    def __init__(self):
        self._headers: Dict[Path, Tuple[dict, int]] = {}

    def get(self, shard: Path, key: str) -> torch.Tensor:
        import struct

        from ..export.safetensors_io import _RD

        if shard not in self._headers:
            with open(shard, "rb") as f:
                (n,) = struct.unpack("<Q", f.read(8))
                self._headers[shard] = (json.loads(f.read(n)), 8 + n)
        header, base = self._headers[shard]
        info = header[key]
        b, e = info["data_offsets"]
        with open(shard, "rb") as f:
            f.seek(base + b)
            buf = bytearray(f.read(e - b))
        dt = _RD[info["dtype"]]
        return torch.frombuffer(buf, dtype=torch.uint8).view(dt).reshape(info["shape"]) if e > b else torch.empty(info["shape"], dtype=dt)


def _quantisable(key: str, t: torch.Tensor, protect: bool) -> bool:
    if t.dim() != 2 or not t.is_floating_point() or t.shape[1] % 16 != 0 or not key.endswith("weight"):
        return False
    low = key.lower()
    if protect and (any(p in low for p in PROTECTED) or "norm" in low or ("gate" in low and t.numel() < 65536 and "gate_proj" not in low)):
        return False
    return min(t.shape) >= 16


def _pack(t: torch.Tensor, hadamard: bool, device: torch.device):
    p, s, ts = ops.nvfp4_quantize(t.to(device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32), hadamard=hadamard)
    return p.cpu().contiguous(), s.cpu().contiguous(), ts.reshape(1).float().cpu()


def build_nvfp4_disk_cache(model_id_or_dir, cache_dir=None, *, hadamard: bool = True, protect_sensitive: bool = True,
                           quantize_lm_head: bool = False, device: Optional[str] = None, force: bool = False) -> Dict[str, Any]:
    """Returns the manifest (also written to ``<cache_dir>/manifest.json``)."""
    model_dir = Path(model_id_or_dir)
    if not model_dir.is_dir():
        raise FileNotFoundError(f"{model_id_or_dir} is not a local model directory (hub downloads need network access)")
    target = Path(cache_dir) if cache_dir is not None else default_nvfp4_cache_dir(model_id_or_dir, hadamard)
    mpath = target / "manifest.json"
    if mpath.is_file() and not force:
        old = json.loads(mpath.read_text())
        if old.get("version") == MANIFEST_VERSION and bool(old.get("hadamard")) == bool(hadamard) and old.get("num_layers", 0) > 0 \
                and bool(old.get("quantize_lm_head", False)) == bool(quantize_lm_head):
            return old
    (target / "layers").mkdir(parents=True, exist_ok=True)
    for f in _AUX_FILES:
        if (model_dir / f).is_file():
            shutil.copy2(model_dir / f, target / f)
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    wmap = _discover_weight_map(model_dir)
    reader = _ShardReader()
    layers: Dict[int, Dict[str, Path]] = {}
    root: Dict[str, Path] = {}
    prefix = None
    for k, shard in wmap.items():
        m = _LAYER_RE.match(k)
        if m:
            prefix = prefix or m.group(1)
            layers.setdefault(int(m.group(2)), {})[m.group(3)] = shard
        else:
            root[k] = shard
    raw_bytes = packed_bytes = 0
    tied = False
    if (model_dir / "config.json").is_file():
        tied = bool(json.loads((model_dir / "config.json").read_text()).get("tie_word_embeddings", False))

    def convert(items: Dict[str, Path], full_prefix: str, allow_quant) -> Tuple[Dict[str, torch.Tensor], List[str]]:
        nonlocal raw_bytes, packed_bytes
        out: Dict[str, torch.Tensor] = {}
        qmods: List[str] = []
        for sub, shard in items.items():
            t = reader.get(shard, f"{full_prefix}{sub}")
            raw_bytes += t.numel() * t.element_size()
            if allow_quant(sub, t):
                p, s, ts = _pack(t, hadamard, dev)
                stem = sub[: -len(".weight")]
                out[f"{stem}.packed_weight"], out[f"{stem}.block_scales"], out[f"{stem}.tensor_scale"] = p, s.view(torch.uint8), ts
                qmods.append(stem)
            else:
                out[sub] = (t.to(torch.bfloat16) if t.is_floating_point() else t).contiguous()
        packed_bytes += sum(v.numel() * v.element_size() for v in out.values())
        return out, qmods

    root_t, root_q = convert(root, "", lambda k, t: quantize_lm_head and k == "lm_head.weight" and not tied and _quantisable("x.weight", t, False))
    save_file(root_t, str(target / "root.safetensors"))
    layer_files, layer_q = [], []
    for i in sorted(layers):
        lt, lq = convert(layers[i], f"{prefix}.{i}.", lambda k, t: _quantisable(k, t, protect_sensitive))
        rel = f"layers/layer_{i:04d}.safetensors"
        save_file(lt, str(target / rel))
        layer_files.append(rel)
        layer_q.append(lq)
    manifest = {"version": MANIFEST_VERSION, "source": str(model_dir), "format": "nvfp4-e2m1-e4m3x16-fp32", "hadamard": bool(hadamard),
                "quantize_lm_head": bool(quantize_lm_head), "layer_prefix": prefix, "num_layers": len(layer_files),
                "layer_files": layer_files, "quantized_modules": layer_q, "root_file": "root.safetensors",
                "root_quantized_modules": root_q, "raw_bytes": raw_bytes, "packed_bytes": packed_bytes,
                "compression": round(raw_bytes / max(1, packed_bytes), 3), "tie_word_embeddings": tied}
    mpath.write_text(json.dumps(manifest, indent=2))
    return manifest


def describe_cache(cache_dir) -> Dict[str, Any]:
    m = json.loads((Path(cache_dir) / "manifest.json").read_text())
    size = sum(f.stat().st_size for f in Path(cache_dir).rglob("*.safetensors"))
    return {**{k: m[k] for k in ("version", "source", "format", "hadamard", "num_layers", "compression")}, "bytes_on_disk": size}


class DiskNVFP4StreamingEngine:
    """Serves layer weights out of an NVFP4 disk cache.

    ``layer_state(i)`` returns a ``{name: tensor}`` dict on the device: quantised matrices decoded to ``dtype`` (or left
    packed as ``(packed, scales, tensor_scale)`` when ``keep_packed``), everything else as stored. The next layers are
    read and uploaded by a worker thread on a side stream while the caller computes.
    """

    def __init__(self, cache_dir, device, dtype: torch.dtype = torch.bfloat16, prefetch: int = 1, resident_budget_gb: float = 0.0,
                 keep_packed: bool = False, pin_memory: Optional[bool] = None):
        self.dir = Path(cache_dir)
        self.manifest = json.loads((self.dir / "manifest.json").read_text())
        if self.manifest.get("version") != MANIFEST_VERSION:
            raise ValueError(f"unsupported cache manifest version {self.manifest.get('version')}")
        self.device, self.dtype = torch.device(device), dtype
        self.cuda = self.device.type == "cuda"
        self.pin = self.cuda if pin_memory is None else pin_memory
        self.keep_packed, self.prefetch = keep_packed, max(0, prefetch)
        self.num_layers = int(self.manifest["num_layers"])
        self.hadamard = bool(self.manifest["hadamard"])
        self.budget = int(resident_budget_gb * 2**30)
        self._resident: "OrderedDict[int, Dict[str, Any]]" = OrderedDict()
        self._resident_bytes = 0
        self._pending: Dict[int, Future] = {}
        self._pool = ThreadPoolExecutor(max_workers=1, thread_name_prefix="nvfp4-prefetch")
        self._stream = torch.cuda.Stream(self.device) if self.cuda else None
        self._lock = threading.Lock()
        self.telemetry = {"disk_bytes": 0, "h2d_bytes": 0, "layers_loaded": 0, "cache_hits": 0, "evictions": 0}

    # ------------------------------------------------------------------ root
    def root_state(self) -> Dict[str, torch.Tensor]:
        sd = load_file(str(self.dir / self.manifest["root_file"]))
        return self._to_device(sd, set(self.manifest.get("root_quantized_modules", [])))[0]

    # ------------------------------------------------------------------ layers
    def _read(self, i: int) -> Dict[str, torch.Tensor]:
        path = self.dir / self.manifest["layer_files"][i]
        sd = load_file(str(path))
        self.telemetry["disk_bytes"] += path.stat().st_size
        if self.pin:
            sd = {k: v.pin_memory() for k, v in sd.items()}
        return sd

    def _to_device(self, sd: Dict[str, torch.Tensor], qmods) -> Tuple[Dict[str, Any], int]:
        out: Dict[str, Any] = {}
        nbytes = 0
        done = set()
        for stem in qmods:
            p = sd[f"{stem}.packed_weight"].to(self.device, non_blocking=True)
            s = sd[f"{stem}.block_scales"].to(self.device, non_blocking=True).view(torch.float8_e4m3fn)
            t = sd[f"{stem}.tensor_scale"].to(self.device, non_blocking=True).reshape(())
            self.telemetry["h2d_bytes"] += p.numel() + s.numel() + 4
            if self.keep_packed:
                out[f"{stem}.weight"] = (p, s, t)
                nbytes += p.numel() + s.numel()
            else:
                w = ops.nvfp4_dequantize(p, s, t, self.dtype)  # rotated weights stay rotated: the consumer rotates activations
                out[f"{stem}.weight"] = w
                nbytes += w.numel() * w.element_size()
            done.update((f"{stem}.packed_weight", f"{stem}.block_scales", f"{stem}.tensor_scale"))
        for k, v in sd.items():
            if k in done:
                continue
            t = v.to(self.device, non_blocking=True)
            t = t.to(self.dtype) if t.is_floating_point() else t
            out[k] = t
            nbytes += t.numel() * t.element_size()
            self.telemetry["h2d_bytes"] += v.numel() * v.element_size()
        return out, nbytes

    def _load(self, i: int):
        sd = self._read(i)
        qmods = self.manifest["quantized_modules"][i]
        if self._stream is not None:
            with torch.cuda.stream(self._stream):
                out, nbytes = self._to_device(sd, qmods)
                ev = torch.cuda.Event()
                ev.record(self._stream)
            return out, nbytes, ev, sd  # sd kept alive until the copies are known to be done
        out, nbytes = self._to_device(sd, qmods)
        return out, nbytes, None, None

    def _schedule(self, i: int) -> None:
        if 0 <= i < self.num_layers and i not in self._resident and i not in self._pending:
            self._pending[i] = self._pool.submit(self._load, i)

    def layer_state(self, i: int, direction: int = 1) -> Dict[str, Any]:
        """State of layer ``i``; schedules layers ``i + direction * (1..prefetch)`` in the background."""
        with self._lock:
            if i in self._resident:
                self._resident.move_to_end(i)
                self.telemetry["cache_hits"] += 1
                state = self._resident[i]
            else:
                self._schedule(i)
                out, nbytes, ev, _keep = self._pending.pop(i).result()
                if ev is not None:
                    torch.cuda.current_stream(self.device).wait_event(ev)
                self.telemetry["layers_loaded"] += 1
                state = out
                self._resident[i] = out
                self._resident_bytes += nbytes
                out["__nbytes__"] = nbytes
                while self._resident_bytes > max(self.budget, nbytes) and len(self._resident) > 1:
                    j, old = self._resident.popitem(last=False)
                    if j == i:  # never evict what we are about to hand out
                        self._resident[j] = old
                        self._resident.move_to_end(j, last=False)
                        break
                    self._resident_bytes -= old.get("__nbytes__", 0)
                    self.telemetry["evictions"] += 1
            for k in range(1, self.prefetch + 1):
                self._schedule(i + direction * k)
        return {k: v for k, v in state.items() if k != "__nbytes__"}

    def release_all(self) -> None:
        with self._lock:
            for f in self._pending.values():
                f.cancel()
            self._pending.clear()
            self._resident.clear()
            self._resident_bytes = 0

    def close(self) -> None:
        self.release_all()
        self._pool.shutdown(wait=True)

    # ------------------------------------------------------------------ forward helper for HF-style decoder stacks
    @torch.no_grad()
    def run_layers(self, layer_module: nn.Module, hidden: torch.Tensor, layer_prefix_strip: str = "", **layer_kwargs) -> torch.Tensor:
        """Run ``hidden`` through every cached layer using ONE module instance whose parameters are re-pointed at the
        streamed tensors layer after layer (the skeleton never owns weights of its own)."""
        params = dict(layer_module.named_parameters())
        for i in range(self.num_layers):
            state = self.layer_state(i)
            for name, p in params.items():
                w = state.get(name)
                if w is None or isinstance(w, tuple):
                    raise KeyError(f"layer {i} of the cache has no dense tensor for parameter {name!r}")
                p.data = w
            out = layer_module(hidden, **layer_kwargs)
            hidden = out[0] if isinstance(out, tuple) else out
        return hidden


# ---------------------------------------------------------------------------------------------------- a whole model on top of a cache
def resolve_hf_model_dir(model_id_or_dir, *, local_files_only: bool = False) -> Path:
    """The local directory of a Hugging Face model: the argument when it is a directory, else the snapshot of that
    repository id in the local hub cache. Nothing is downloaded (``triune/runtime/disk_streaming.py:50-78`` of the
    reference falls through to a download; here a model that is not on disk is a ``FileNotFoundError``)."""
    p = Path(model_id_or_dir).expanduser()
    if p.is_dir():
        return p
    hub = Path(os.environ.get("HF_HUB_CACHE") or Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface")) / "hub")
    snaps = hub / ("models--" + str(model_id_or_dir).replace("/", "--")) / "snapshots"
    if snaps.is_dir():
        for snap in sorted(snaps.iterdir(), key=lambda d: d.stat().st_mtime, reverse=True):
            if any(snap.glob("*.safetensors")) or (snap / "model.safetensors.index.json").is_file():
                return snap
    raise FileNotFoundError(f"{model_id_or_dir} is neither a local directory nor a snapshot in {hub} (downloads need network access)")


class _RotateIn(nn.Module):
    """A linear layer whose weight was quantised in the rotated basis: rotate the input the same way (the 16-point
    Walsh-Hadamard transform of every group of 16 features is its own inverse up to the scale both sides carry)."""

    def __init__(self, inner: nn.Linear):
        super().__init__()
        self.inner = inner

    @property
    def weight(self):
        return self.inner.weight

    @property
    def bias(self):
        return self.inner.bias

    def forward(self, x):
        from ..ops import reference as ref

        return self.inner(ref.fwht16(x.float()).to(x.dtype))


def load_disk_streamed_model(model_or_cache_dir, *, cache_dir=None, device=None, hadamard: bool = True, protect_sensitive: bool = True,
                             quantize_lm_head: bool = False, activation_checkpointing: bool = True, async_prefetch: bool = True,
                             pin_memory: bool = False, local_files_only: bool = False):
    """-> (model, engine, cache directory). A Hugging Face causal LM whose decoder layers exist only as an NVFP4 cache on
    disk: the model is created without storage, the root tensors (embeddings, final norm, head) are loaded to ``device``,
    and every decoder layer gets its weights from the ``DiskNVFP4StreamingEngine`` for the duration of its forward pass
    (decoded to bf16; the next layer is read in the background) and gives them back afterwards, so device memory holds
    one or two layers at a time. Inference only: the layers' weights are not parameters that an optimizer could update
    (``activation_checkpointing`` is accepted for the reference's signature). The cache is built first when the argument
    is a model directory (``triune/runtime/disk_streaming.py:696-800`` of the reference)."""
    from transformers import AutoConfig, AutoModelForCausalLM

    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    cand = Path(model_or_cache_dir).expanduser()
    if (cand / "manifest.json").is_file():
        cache = cand
    else:
        src = resolve_hf_model_dir(model_or_cache_dir, local_files_only=local_files_only)
        cache = Path(cache_dir) if cache_dir is not None else default_nvfp4_cache_dir(src, hadamard)
        build_nvfp4_disk_cache(src, cache, hadamard=hadamard, protect_sensitive=protect_sensitive, quantize_lm_head=quantize_lm_head)
    engine = DiskNVFP4StreamingEngine(cache, dev, dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                                      prefetch=1 if async_prefetch else 0, pin_memory=pin_memory and dev.type == "cuda")
    man = engine.manifest
    cfg = AutoConfig.from_pretrained(str(cache))
    with torch.device("meta"):
        try:
            model = AutoModelForCausalLM.from_config(cfg, dtype=engine.dtype)
        except TypeError:
            model = AutoModelForCausalLM.from_config(cfg, torch_dtype=engine.dtype)
    layers = model
    for part in str(man["layer_prefix"]).split("."):
        layers = getattr(layers, part)
    layers = list(layers)
    for lay in layers:  # the layers never hold storage of their own
        lay.requires_grad_(False)
    root = engine.root_state()
    if man.get("tie_word_embeddings") and "lm_head.weight" not in root:
        emb = next((v for k, v in root.items() if k.endswith("embed_tokens.weight") or k.endswith("wte.weight")), None)
        if emb is not None:
            root["lm_head.weight"] = emb
    inside = tuple(f"{man['layer_prefix']}.{i}." for i in range(len(layers)))
    missing = [k for k, v in model.state_dict().items() if v.is_meta and k not in root and not k.startswith(inside)]
    model.load_state_dict(root, strict=False, assign=True)
    for name, buf in list(model.named_buffers()):  # rotary tables and the like are computed, not stored: make them again
        if buf.is_meta:
            owner = model.get_submodule(name.rpartition(".")[0]) if "." in name else model
            fresh = type(owner)(config=cfg) if "rotary" in type(owner).__name__.lower() else None
            if fresh is None:
                raise RuntimeError(f"buffer {name} has no stored value in the cache and cannot be recomputed")
            owner.register_buffer(name.rpartition(".")[2], getattr(fresh, name.rpartition(".")[2]).to(dev), persistent=False)
    if missing:
        raise RuntimeError(f"the cache holds no value for: {missing[:5]}")
    rotated = bool(man.get("hadamard"))

    def wrap(i: int, layer: nn.Module):
        inner_forward = layer.forward
        qmods = list(man["quantized_modules"][i])

        def forward(*args, **kwargs):
            state = engine.layer_state(i)
            held = []
            for key, value in state.items():
                owner_name, _, leaf = key.rpartition(".")
                owner = layer.get_submodule(owner_name) if owner_name else layer
                if isinstance(owner, _RotateIn):
                    owner = owner.inner
                held.append((owner, leaf, owner._parameters.get(leaf), leaf in owner._parameters))
                if leaf in owner._parameters:
                    owner._parameters[leaf] = nn.Parameter(value, requires_grad=False)
                else:
                    owner._buffers[leaf] = value
            try:
                return inner_forward(*args, **kwargs)
            finally:
                for owner, leaf, old, is_param in held:
                    if is_param:
                        owner._parameters[leaf] = old
                if engine.budget <= 0:
                    with engine._lock:
                        engine._resident.pop(i, None)
                        engine._resident_bytes = sum(s.get("__nbytes__", 0) for s in engine._resident.values())

        if rotated:
            for stem in qmods:
                parent_name, _, leaf = stem.rpartition(".")
                parent = layer.get_submodule(parent_name) if parent_name else layer
                lin = getattr(parent, leaf)
                if isinstance(lin, nn.Linear):
                    setattr(parent, leaf, _RotateIn(lin))
        layer.forward = forward

    for i, lay in enumerate(layers):
        wrap(i, lay)
    model.eval()
    model._disk_streaming_engine = engine
    model._layer_streaming_active = True
    return model, engine, cache
