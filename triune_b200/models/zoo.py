"""Model specs, the preset zoo, the architecture registry and the unified model loader.

Parity: ``ModelSpec`` / ``CANONICAL_MODEL_SPECS`` / ``get_model_spec`` / ``build_model_from_spec`` /
``register_model`` (``triune/model/base.py:18-461``) and ``load_model`` (``triune/model/zoo.py:18-93``): eleven
canonical presets nano ... 70b plus legacy aliases; ``get_model_spec`` clamps the layer hierarchy
(``0 < prefix < reflex < limbic < L``, at least 4 layers), reconciles ``hidden_dim = heads * head_dim`` and normalises
the precision string; ``load_model`` resolves ``.json`` config -> checkpoint -> registry -> preset -> Hugging Face.

Difference: large models are materialised directly in bf16 on the target device (``device=`` argument) instead of
being built on the host with patched ``reset_parameters`` and copied through a bounce buffer; a 70B preset is ~140 GB
in bf16 and fits one B200.
"""

from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Tuple, Type

import torch
import torch.nn as nn

from ..config import MODEL_PRESETS, ModelConfig, build_config, model_config_from_flat

MODEL_REGISTRY: Dict[str, Type[nn.Module]] = {}


def register_model(name: str) -> Callable[[Type[nn.Module]], Type[nn.Module]]:
    """Class decorator: ``@register_model("my-arch")`` makes ``load_model("my-arch", **kw)`` construct it."""

    def deco(cls):
        MODEL_REGISTRY[name.lower()] = cls
        return cls

    return deco


@dataclass
class ModelSpec:
    model_id: str = "triune-small"
    name: str = "Triune-Small"
    vocab_size: int = 32000
    hidden_dim: int = 256
    num_layers: int = 6
    num_heads: int = 4
    head_dim: int = 64
    num_experts: int = 4
    experts_routed: int = 4
    experts_shared: int = 1
    router_prefix_layers: int = 1
    reflex_exit_layer: int = 2
    limbic_exit_layer: int = 4
    target_depth_dist: Tuple[float, float, float] = (0.50, 0.30, 0.20)
    balance_coef: float = 0.3
    depth_mode: str = "dynamic"
    precision: str = "bf16"
    use_fp4: bool = False
    use_fp8: bool = False
    streaming_fp8_weights: bool = False
    use_layer_streaming: bool = False
    chunk_size: int = 1
    recommended_batch: int = 4
    recommended_seq: int = 64
    tier: str = "Production Baseline"
    params_label: str = ""
    extra_config: Dict[str, Any] = field(default_factory=dict)

    def to_model_config(self) -> ModelConfig:
        extra = {k: v for k, v in self.extra_config.items() if k in ModelConfig.__dataclass_fields__}
        kw = dict(vocab_size=self.vocab_size, hidden_dim=self.hidden_dim, num_layers=self.num_layers,
                  num_heads=self.num_heads, head_dim=self.head_dim, num_experts=self.num_experts,
                  shared_expert=self.experts_shared >= 1, router_prefix_layers=self.router_prefix_layers,
                  reflex_exit_layer=self.reflex_exit_layer, limbic_exit_layer=self.limbic_exit_layer,
                  target_depth_dist=tuple(self.target_depth_dist), balance_coef=self.balance_coef,
                  use_fp4=self.use_fp4, use_fp8=self.use_fp8)
        kw.update(extra)
        return ModelConfig(**kw)

    def compute_exact_params(self) -> Tuple[int, int]:
        """(total parameters, parameters touched per token) of the TriuneTransformer this spec builds."""
        return self.to_model_config().param_count()

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        total, active = self.compute_exact_params()
        d.update(preset_id=self.model_id, params=self.params_label or _label(total), total_params=total,
                 active_params=active)
        return d

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "ModelSpec":
        names = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in data.items() if k in names}
        for alt in ("preset_id", "model_name"):
            if "model_id" not in kw and alt in data:
                kw["model_id"] = str(data[alt])
        if isinstance(kw.get("target_depth_dist"), list):
            kw["target_depth_dist"] = tuple(float(x) for x in kw["target_depth_dist"])
        derived = {"params", "total_params", "active_params", "preset_id", "model_name"}
        kw.setdefault("extra_config", {k: v for k, v in data.items() if k not in names and k not in derived})
        return cls(**kw)


def _label(n: int) -> str:
    return f"{n / 1e9:.2f}B params" if n >= 1e9 else f"{n / 1e6:.1f}M params"


_RECOMMENDED = {  # preset -> (batch, seq, tier, streaming)
    "triune-nano": (8, 128, "Edge / Drafter", False), "triune-small": (4, 64, "Production Baseline", False),
    "triune-base": (16, 2048, "Research Baseline", False), "triune-medium": (16, 2048, "Research", False),
    "triune-large": (16, 2048, "Research", False), "triune-1b": (8, 2048, "Workstation", False),
    "triune-3b": (8, 2048, "Workstation", False), "triune-7b": (4, 2048, "Single accelerator", False),
    "triune-14b": (4, 2048, "Single accelerator", False), "triune-32b": (2, 2048, "Single accelerator, streamed optimizer", True),
    "triune-70b": (1, 2048, "Layer-streamed", True),
}


def _spec_from_preset(pid: str, cfg: ModelConfig) -> ModelSpec:
    b, s, tier, stream = _RECOMMENDED.get(pid, (4, 2048, "Custom", False))
    spec = ModelSpec(model_id=pid, name="", vocab_size=cfg.vocab_size, hidden_dim=cfg.hidden_dim, num_layers=cfg.num_layers,
                     num_heads=cfg.num_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts,
                     experts_routed=cfg.num_experts, experts_shared=1 if cfg.shared_expert else 0,
                     router_prefix_layers=cfg.router_prefix_layers, reflex_exit_layer=cfg.reflex_exit_layer,
                     limbic_exit_layer=cfg.limbic_exit_layer, target_depth_dist=tuple(cfg.target_depth_dist),
                     balance_coef=cfg.balance_coef, recommended_batch=b, recommended_seq=s, tier=tier,
                     use_layer_streaming=stream)
    total, _ = spec.compute_exact_params()
    spec.params_label = _label(total)
    spec.name = f"{pid.replace('triune-', 'Triune-').title()} ({spec.params_label.split()[0]}, {cfg.num_layers}L / {cfg.hidden_dim}D / {cfg.num_experts}E)"
    return spec


_CANONICAL_IDS = ("triune-nano", "triune-small", "triune-base", "triune-medium", "triune-large", "triune-1b", "triune-3b",
                  "triune-7b", "triune-14b", "triune-32b", "triune-70b")
CANONICAL_MODEL_SPECS: Dict[str, ModelSpec] = {
    pid: _spec_from_preset(pid, MODEL_PRESETS["triune-1.5b" if pid == "triune-1b" else pid]) for pid in _CANONICAL_IDS
}

LEGACY_PRESET_ALIASES: Dict[str, str] = {
    "triune-micro": "triune-nano", "triune-drafter": "triune-nano", "triune-code-moe": "triune-base",
    "triune-math-gla": "triune-base", "triune-multimodal": "triune-base", "triune-1.5b": "triune-1b",
    "triune-2.5b": "triune-3b", "triune-3.0b": "triune-3b", "triune-moe": "triune-7b", "triune-7.0b": "triune-7b",
    "triune-14.5b": "triune-14b", "triune-32.0b": "triune-32b", "triune-34b": "triune-32b", "triune-34.5b": "triune-32b",
    "triune-70.0b": "triune-70b", "triune-71b": "triune-70b", "triune-71.0b": "triune-70b",
}


def _normalise_precision(p: str) -> str:
    p = str(p).lower()
    if any(t in p for t in ("fp8", "e4m3", "e5m2")):
        return "fp8"
    if any(t in p for t in ("fp4", "nf4", "int4")):
        return "fp4"
    if "32" in p:
        return "fp32"
    if "16" in p and "bf" not in p:
        return "fp16"
    return "bf16"


def get_model_spec(preset_id: Optional[str] = None, **overrides: Any) -> ModelSpec:
    raw = (preset_id or "triune-small").lower()
    pid = LEGACY_PRESET_ALIASES.get(raw, raw)
    base = CANONICAL_MODEL_SPECS.get(pid, CANONICAL_MODEL_SPECS["triune-small"])
    d = asdict(base)
    if raw in CANONICAL_MODEL_SPECS:
        d["model_id"] = raw
    elif preset_id:
        d["model_id"] = preset_id
        if raw not in LEGACY_PRESET_ALIASES:
            d["name"] = f"Triune-Custom ({preset_id})"
    d.update({k: v for k, v in overrides.items() if v is not None})
    L = max(4, int(d["num_layers"]))
    prefix = max(1, min(int(d["router_prefix_layers"]), max(1, L - 3)))
    reflex = max(prefix + 1, min(int(d["reflex_exit_layer"]), max(prefix + 1, L - 2)))
    limbic = max(reflex + 1, min(int(d["limbic_exit_layer"]), max(reflex + 1, L - 1)))
    heads, hd, hidden = max(1, int(d["num_heads"])), max(1, int(d["head_dim"])), int(d["hidden_dim"])
    if hidden != heads * hd:
        if "hidden_dim" in overrides and "head_dim" not in overrides and hidden % heads == 0:
            hd = hidden // heads
        else:
            hidden = heads * hd
    prec = _normalise_precision(d.get("precision", "bf16"))
    if overrides.get("precision") is not None:
        fp8, fp4 = bool(overrides.get("use_fp8", prec == "fp8")), bool(overrides.get("use_fp4", prec == "fp4"))
    else:
        fp4, fp8 = bool(d.get("use_fp4") or prec == "fp4"), bool(d.get("use_fp8") or prec == "fp8")
    d.update(num_layers=L, router_prefix_layers=prefix, reflex_exit_layer=reflex, limbic_exit_layer=limbic, num_heads=heads,
             head_dim=hd, hidden_dim=hidden, num_experts=max(1, int(d["num_experts"])), use_fp4=fp4, use_fp8=fp8,
             precision="fp8" if fp8 else ("fp4" if fp4 else prec))
    spec = ModelSpec.from_dict(d)
    spec.params_label = _label(spec.compute_exact_params()[0])
    return spec


def build_model_from_spec(spec: ModelSpec, device=None, dtype: Optional[torch.dtype] = None) -> nn.Module:
    """Build the TriuneTransformer a spec describes. Models of 150M parameters or more are created in bf16 (unless the
    spec says fp32) directly on ``device`` so no fp32 host copy ever exists."""
    from .transformer import TriuneTransformer

    spec = get_model_spec(spec.model_id, **{k: v for k, v in asdict(spec).items() if k != "model_id"})
    total, _ = spec.compute_exact_params()
    if dtype is None and total >= 150_000_000 and spec.precision != "fp32":
        dtype = torch.bfloat16
    old = torch.get_default_dtype()
    try:
        if dtype is not None:
            torch.set_default_dtype(dtype)
        if device is not None:
            with torch.device(device):
                model = TriuneTransformer.from_config(spec.to_model_config())
        else:
            model = TriuneTransformer.from_config(spec.to_model_config())
    finally:
        torch.set_default_dtype(old)
    model.spec = spec
    return model


def _load_state(path: Path) -> Dict[str, Any]:
    from ..trainer.checkpoint import safe_torch_load

    return safe_torch_load(path)


def load_model(model_name_or_path, **kwargs: Any) -> nn.Module:
    """Resolution order: ``.json`` config file, checkpoint file, registered architecture, canonical preset (or alias),
    ``models/configs/<name>.json`` next to the package, ``default``, then Hugging Face ``AutoModelForCausalLM``."""
    from .factory import build_model

    name = str(model_name_or_path).lower()
    path = Path(str(model_name_or_path))
    if path.is_file() and path.suffix.lower() == ".json":
        return build_model(build_config({**json.loads(path.read_text(encoding="utf-8")), **kwargs}))
    if path.is_file():
        ck = _load_state(path)
        saved = (ck.get("config") or {}) if isinstance(ck, dict) else {}
        sd = ck["model_state"] if isinstance(ck, dict) and "model_state" in ck else ck
        sd = {k.removeprefix("_orig_mod."): v for k, v in sd.items()}
        if all(k in saved for k in ("hidden_dim", "num_layers", "num_heads")):
            try:
                model = build_model(build_config({**saved, **kwargs}))
                model.load_state_dict(sd)
                return model
            except Exception:
                pass  # stale or partial config: fall through and read the architecture off the tensors
        from ..inference import load_checkpoint_model

        return load_checkpoint_model(str(path))[0]
    if name in MODEL_REGISTRY:
        return MODEL_REGISTRY[name](**kwargs)
    if name in CANONICAL_MODEL_SPECS or name in LEGACY_PRESET_ALIASES:
        device, dtype = kwargs.pop("device", None), kwargs.pop("dtype", None)
        return build_model_from_spec(get_model_spec(name, **kwargs), device=device, dtype=dtype)
    if name in MODEL_PRESETS:
        return build_model(name)
    cand = Path(__file__).resolve().parent.parent / "configs" / f"{name}.json"
    if not path.suffix and cand.is_file():
        return build_model(build_config({**json.loads(cand.read_text(encoding="utf-8")), **kwargs}))
    if name in ("default", "none", ""):
        return build_model(build_config(kwargs))
    try:
        if not (path.is_dir() or "/" in str(model_name_or_path)):
            raise FileNotFoundError("not a local directory and not an 'org/name' hub id")
        from transformers import AutoModelForCausalLM

        return AutoModelForCausalLM.from_pretrained(str(model_name_or_path), **kwargs)
    except Exception as exc:
        raise ValueError(f"model {model_name_or_path!r} is not a checkpoint, a registered architecture, a JSON config or "
                         f"a preset ({sorted(CANONICAL_MODEL_SPECS)}); Hugging Face loading failed with: {exc}") from exc


def list_models() -> Dict[str, Dict[str, Any]]:
    out = {k: v.to_dict() for k, v in CANONICAL_MODEL_SPECS.items()}
    out.update({k: {"registered": True, "class": c.__name__} for k, c in MODEL_REGISTRY.items()})
    return out
