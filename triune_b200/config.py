"""Typed configuration objects, model presets and the flat run-config dictionary.

Parity notes (reference paths are relative to the reference project root):
  * module constants      -> ``triune/model/config.py:1-126``
  * run-config dict       -> ``triune/configs/config.py:15-151`` (``build_config`` / ``validate_config``)
  * canonical presets     -> ``triune/model/base.py:98-297`` (``ModelSpec`` / ``CANONICAL_MODEL_SPECS``)

Differences by design: the reference hard-wires ``top_k`` and the expert hidden
multiplier; here ``top_k``, ``expert_hidden`` and ``dense_hidden`` are explicit so the
same class covers the published ``triune-base`` (E=4, top-1, hidden 6*d) and the
benchmark "90.8M-class" shape (E=8, top-2, hidden 1536).
"""

from __future__ import annotations

import contextlib
import json
import math
import threading
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, Optional, Tuple

# ----------------------------------------------------------------------------
# Behavioural constants (defaults of the reference, triune/model/config.py)
# ----------------------------------------------------------------------------
VOCAB_SIZE = 32000
HIDDEN_DIM = 1536
NUM_LAYERS = 24
NUM_HEADS = 12
GLA_HEAD_DIM = 128
ROUTER_PREFIX_LAYERS = 3
REFLEX_EXIT_LAYER = 6
LIMBIC_EXIT_LAYER = 16
ROPE_MAX_SEQ_LEN = 8192
ROPE_BASE = 10000.0
NUM_EXPERTS = 8
TOP_K_EXPERTS = 1
SHARED_EXPERT = True
SHARED_EXPERT_SCALE = 0.5
EXPERT_HIDDEN_MULTIPLIER = 6
DENSE_HIDDEN_MULTIPLIER = 4
MOE_CAPACITY_MULTIPLIER = 1.5
MOE_BIAS_UPDATE_RATE = 1e-3
MOE_BIAS_CLAMP = 5.0
CENTROID_EMA = 0.98
MOE_TEMPERATURE_STEPS = 5000.0
TARGET_DEPTH_DIST = (0.34, 0.33, 0.33)
DEPTH_BALANCE_COEF = 0.30
DEPTH_USAGE_EMA = 0.98
DEPTH_BIAS_STRENGTH = 4.0
ROUTER_Z_LOSS = 1e-3
EPS = 1e-6

GALORE_RANK = 256
GALORE_UPDATE_GAP = 200
GALORE_LR = 1e-4
GALORE_BETAS = (0.9, 0.999)
GALORE_WEIGHT_DECAY = 0.05
STEER_SCALE = 0.20
STEER_UPDATE_GAP = 10
MUON_LR = 0.02
MUON_MOMENTUM = 0.95
MUON_WEIGHT_DECAY = 0.01
NS_COEFFS = (1.875, -1.25, 0.375)
NS_STEPS = 3
# defaults of the research training script of the reference (``triune/model/config.py``), under its names
USE_GLA, USE_ROPE, ROUTER_NOISE_STD = True, True, 0.0
GALORE, USE_TRIANGULAR_CORE, USE_8BIT_BASE, USE_MUON = True, True, False, True
BATCH_SIZE, GRAD_ACCUM_STEPS, SEQ_LEN, TOTAL_STEPS = 8, 4, 256, 50_000
LR, MIN_LR, WARMUP_STEPS, BETAS, WEIGHT_DECAY, GRAD_CLIP = 1e-4, 1e-6, 500, (0.9, 0.95), 0.05, 1.0
GRAD_CHECKPOINT, SHUFFLE_BUFFER = True, 4096
LOG_EVERY, SAVE_EVERY, EVAL_EVERY, EVAL_BATCHES, CHECKPOINT_DIR = 10, 1000, 200, 5, "checkpoints_full"

_recompute_state = threading.local()


@contextlib.contextmanager
def checkpoint_fwd_ctx():
    """Context of the first pass through an activation-checkpointed region (nothing to mark)."""
    yield


@contextlib.contextmanager
def checkpoint_bwd_ctx():
    """Context of the recomputation pass: ``is_checkpoint_recomputing()`` is true inside, per thread, so that code with
    side effects (running statistics, counters) can skip them the second time. Usable as the second half of
    ``torch.utils.checkpoint.checkpoint(..., context_fn=lambda: (checkpoint_fwd_ctx(), checkpoint_bwd_ctx()))``; the
    blocks of this framework enter it around their own recomputation."""
    old = getattr(_recompute_state, "on", False)
    _recompute_state.on = True
    try:
        yield
    finally:
        _recompute_state.on = old


def is_checkpoint_recomputing() -> bool:
    return getattr(_recompute_state, "on", False)


@dataclass
class ModelConfig:
    """Architecture of a TriuneTransformer (MoE, multi-exit) or a dense UniversalTransformer."""

    family: str = "triune"  # "triune" (multi-exit MoE) or "universal" (dense)
    vocab_size: int = VOCAB_SIZE
    hidden_dim: int = HIDDEN_DIM
    num_layers: int = NUM_LAYERS
    num_heads: int = NUM_HEADS
    head_dim: int = GLA_HEAD_DIM
    num_experts: int = NUM_EXPERTS
    top_k: int = TOP_K_EXPERTS
    shared_expert: bool = SHARED_EXPERT
    shared_scale: float = SHARED_EXPERT_SCALE
    expert_hidden: Optional[int] = None  # None -> EXPERT_HIDDEN_MULTIPLIER * hidden_dim
    dense_hidden: Optional[int] = None  # None -> DENSE_HIDDEN_MULTIPLIER * hidden_dim
    router_prefix_layers: int = ROUTER_PREFIX_LAYERS
    reflex_exit_layer: int = REFLEX_EXIT_LAYER
    limbic_exit_layer: int = LIMBIC_EXIT_LAYER
    target_depth_dist: Tuple[float, float, float] = TARGET_DEPTH_DIST
    balance_coef: float = DEPTH_BALANCE_COEF
    mixer: str = "gla"  # "gla" | "gated_deltanet" | "sdpa"
    ffn: str = "gelu"  # dense FFN activation: "gelu" | "swiglu"
    num_kv_heads: Optional[int] = None  # sdpa mixer only (GQA)
    use_rope: bool = True
    gla_scale: str = "none"  # "fla": GLA outputs times head_dim ** -0.5 (models trained by the reference with flash-linear-attention)
    rope_base: float = ROPE_BASE
    rope_max_seq_len: int = ROPE_MAX_SEQ_LEN
    capacity_multiplier: float = MOE_CAPACITY_MULTIPLIER
    scale_residual_projections: bool = False
    use_fp8: bool = False
    use_fp4: bool = False
    tie_embeddings: bool = True

    def resolved_expert_hidden(self) -> int:
        return int(self.expert_hidden) if self.expert_hidden else EXPERT_HIDDEN_MULTIPLIER * self.hidden_dim

    def resolved_dense_hidden(self) -> int:
        return int(self.dense_hidden) if self.dense_hidden else DENSE_HIDDEN_MULTIPLIER * self.hidden_dim

    def validate(self) -> "ModelConfig":
        if self.hidden_dim != self.num_heads * self.head_dim:
            raise ValueError(
                f"hidden_dim ({self.hidden_dim}) must equal num_heads * head_dim ({self.num_heads * self.head_dim})"
            )
        if self.family == "triune" and not (
            0 < self.router_prefix_layers < self.reflex_exit_layer < self.limbic_exit_layer < self.num_layers
        ):
            raise ValueError(
                "layer hierarchy violation: need 0 < router_prefix_layers < reflex_exit_layer < "
                f"limbic_exit_layer < num_layers, got {self.router_prefix_layers}, {self.reflex_exit_layer}, "
                f"{self.limbic_exit_layer}, {self.num_layers}"
            )
        if self.num_experts < 1 or not (1 <= self.top_k <= self.num_experts):
            raise ValueError(f"need 1 <= top_k <= num_experts, got top_k={self.top_k}, E={self.num_experts}")
        if self.vocab_size < 1:
            raise ValueError("vocab_size must be >= 1")
        if any((not math.isfinite(x)) or x < 0 for x in self.target_depth_dist):
            raise ValueError("target_depth_dist elements must be finite and non-negative")
        if abs(sum(self.target_depth_dist) - 1.0) > 1e-4:
            raise ValueError("target_depth_dist must sum to 1")
        if not math.isfinite(self.balance_coef) or self.balance_coef < 0:
            raise ValueError("balance_coef must be finite and non-negative")
        if self.use_fp4 and self.use_fp8:
            raise ValueError("use_fp4 and use_fp8 are mutually exclusive")
        if self.mixer not in ("gla", "gated_deltanet", "sdpa"):
            raise ValueError(f"unknown mixer {self.mixer!r}")
        return self

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d["target_depth_dist"] = list(self.target_depth_dist)
        return d

    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "ModelConfig":
        names = {f.name for f in fields(cls)}
        kw = {k: v for k, v in data.items() if k in names}
        if "target_depth_dist" in kw:
            kw["target_depth_dist"] = tuple(float(x) for x in kw["target_depth_dist"])
        return cls(**kw)

    def param_count(self) -> Tuple[int, int]:
        """Exact (total, active-per-token) parameter counts of the TriuneTransformer layout."""
        v, d, L = self.vocab_size, self.hidden_dim, self.num_layers
        hd = self.num_heads * self.head_dim
        attn = 4 * d * hd + hd * d
        norms = 2 * d
        if self.family == "universal":
            ff = self.resolved_dense_hidden()
            ffn = (3 if self.ffn == "swiglu" else 2) * d * ff
            extra_attn = 0
            if self.mixer == "gated_deltanet":
                extra_attn = d * self.num_heads  # beta projection
            per = attn + extra_attn + ffn + norms
            total = v * d + L * per + d + (0 if self.tie_embeddings else v * d)
            return total, total
        dh, eh = self.resolved_dense_hidden(), self.resolved_expert_hidden()
        dense_ffn = d * dh + dh + dh * d + d
        one_expert = d * eh + eh + eh * d + d
        s = 1 if self.shared_expert else 0
        moe_total = (self.num_experts + s) * one_expert + d * self.num_experts + self.num_experts
        moe_active = (self.top_k + s) * one_expert + d * self.num_experts + self.num_experts
        n_dense = self.reflex_exit_layer + 1
        n_moe = L - n_dense
        exits = 2 * (d + v * d + v)
        router = d * 256 + 256 + 256 * 3 + 3
        base = v * d + d + exits + router + L * (attn + norms)
        return base + n_dense * dense_ffn + n_moe * moe_total, base + n_dense * dense_ffn + n_moe * moe_active


@dataclass
class ParallelConfig:
    """Process layout: data / tensor / expert / pipeline degrees (one process per GPU)."""

    dp: int = 1
    tp: int = 1
    ep: int = 1
    pp: int = 1
    sequence_parallel: bool = True
    fused_collectives: bool = True  # in-kernel NVLink paths; False selects the NCCL baseline

    @property
    def world_size(self) -> int:
        # experts are sharded over the data-parallel ranks (EP reuses DP ranks)
        return self.dp * self.tp * self.pp

    def describe(self) -> str:
        parts = []
        if self.dp > 1 or (self.tp == 1 and self.pp == 1):
            parts.append(f"dp{self.dp}")
        if self.tp > 1:
            parts.append(f"tp{self.tp}")
        if self.ep > 1:
            parts.append(f"ep{self.ep}")
        if self.pp > 1:
            parts.append(f"pp{self.pp}")
        return "x".join(parts)


@dataclass
class OptimConfig:
    optimizer: str = "centroid_steer"  # "centroid_steer" | "muon" | "adamw"
    lr: float = 1e-4
    min_lr: float = 1e-6
    warmup_steps: int = 500
    total_steps: int = 50_000
    betas: Tuple[float, float] = (0.9, 0.95)
    weight_decay: float = 0.05
    grad_clip: float = 1.0
    use_muon: bool = True
    muon_lr: float = MUON_LR
    muon_momentum: float = MUON_MOMENTUM
    muon_weight_decay: float = MUON_WEIGHT_DECAY
    ns_steps: int = NS_STEPS
    ns_coeffs: Tuple[float, float, float] = NS_COEFFS
    galore: bool = True
    galore_rank: int = GALORE_RANK
    galore_update_gap: int = GALORE_UPDATE_GAP
    galore_lr: float = GALORE_LR
    galore_betas: Tuple[float, float] = GALORE_BETAS
    galore_weight_decay: float = GALORE_WEIGHT_DECAY
    steer_scale: float = STEER_SCALE
    steer_update_gap: int = STEER_UPDATE_GAP
    use_triangular_core: bool = True
    core_mask_mode: str = "full"


@dataclass
class TrainConfig:
    batch_size: int = 8
    seq_len: int = 256
    grad_accum_steps: int = 4
    depth_mode: str = "cortex"  # "cortex" | "joint" | "dynamic"
    log_every: int = 10
    save_every: int = 1000
    eval_every: int = 200
    eval_batches: int = 5
    checkpoint_dir: str = "checkpoints_full"
    grad_checkpoint: bool = True
    precision: str = "bf16"
    exploration: Any = "linear"  # schedule name ("linear", "cosine", "none") or a starting rate
    exploration_steps: int = 5000
    usage_ema_decay: float = DEPTH_USAGE_EMA
    bias_strength: float = DEPTH_BIAS_STRENGTH
    exit_distill_coef: float = 0.2
    z_loss_coef: float = ROUTER_Z_LOSS
    cuda_graph: bool = False
    seed: int = 0


@dataclass
class ServeConfig:
    host: str = "127.0.0.1"
    port: int = 8000
    max_concurrency: int = 16
    lock_timeout_s: float = 30.0
    session_capacity: int = 512
    session_ttl_s: float = 3600.0
    prefill_chunk: int = 1024
    max_new_tokens: int = 8192
    k_draft: int = 3
    quant: str = "bf16"  # "bf16" | "fp8" | "nvfp4"


# ----------------------------------------------------------------------------
# Presets
# ----------------------------------------------------------------------------
def _preset(L, d, h, hd, E, prefix, reflex, limbic, top_k=1, **kw) -> ModelConfig:
    return ModelConfig(
        hidden_dim=d,
        num_layers=L,
        num_heads=h,
        head_dim=hd,
        num_experts=E,
        top_k=top_k,
        router_prefix_layers=prefix,
        reflex_exit_layer=reflex,
        limbic_exit_layer=limbic,
        **kw,
    )


MODEL_PRESETS: Dict[str, ModelConfig] = {
    # canonical family of the reference (triune/model/base.py:98-297)
    "triune-nano": _preset(4, 192, 3, 64, 2, 1, 2, 3),
    "triune-small": _preset(6, 256, 4, 64, 4, 1, 2, 4),
    "triune-base": _preset(8, 384, 6, 64, 4, 1, 2, 5),
    "triune-medium": _preset(12, 512, 8, 64, 8, 2, 4, 8),
    "triune-large": _preset(16, 768, 12, 64, 8, 2, 5, 10),
    "triune-1.5b": _preset(24, 1024, 16, 64, 8, 3, 7, 16),
    "triune-3b": _preset(30, 1280, 20, 64, 8, 3, 7, 19),
    "triune-7b": _preset(32, 1920, 30, 64, 8, 4, 7, 20),
    "triune-14b": _preset(40, 2048, 16, 128, 12, 4, 9, 25),
    "triune-32b": _preset(48, 2560, 20, 128, 16, 5, 11, 30),
    "triune-70b": _preset(64, 3072, 24, 128, 16, 6, 11, 40),
    "triune-default": _preset(24, 1536, 12, 128, 8, 3, 6, 16),
    # benchmark shapes
    # 8 layers, d=384, 6x64 GLA heads, E=8 top-2 + shared, FFN/expert hidden 1536, exits at 2/5/8
    "bench-90m": _preset(8, 384, 6, 64, 8, 1, 2, 5, top_k=2, expert_hidden=1536, dense_hidden=1536),
    # expert-parallel MoE-GLA: d=1536, 24 layers, 24x64 heads, E=64 top-2 + shared, expert hidden 4096
    "bench-ep-moe": _preset(24, 1536, 24, 64, 64, 3, 6, 16, top_k=2, expert_hidden=4096, dense_hidden=4096),
    # dense ~1.5B: d=2048, 24 layers, 16x128 Gated DeltaNet heads, SwiGLU 5632
    "bench-dense-1.5b": ModelConfig(
        family="universal",
        hidden_dim=2048,
        num_layers=24,
        num_heads=16,
        head_dim=128,
        mixer="gated_deltanet",
        ffn="swiglu",
        dense_hidden=5632,
        num_experts=1,
        top_k=1,
    ),
}

_ALIASES = {
    "base": "triune-base",
    "small": "triune-small",
    "nano": "triune-nano",
    "medium": "triune-medium",
    "large": "triune-large",
    "default": "triune-default",
    "90m": "bench-90m",
}


def get_model_config(name: str) -> ModelConfig:
    key = _ALIASES.get(name.lower(), name.lower())
    if key not in MODEL_PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(MODEL_PRESETS)}")
    return ModelConfig.from_dict(MODEL_PRESETS[key].to_dict())


# ----------------------------------------------------------------------------
# Flat run-config dictionary (key names of the reference's build_config)
# ----------------------------------------------------------------------------
_FLAT_DEFAULTS: Dict[str, Any] = {
    "vocab_size": VOCAB_SIZE,
    "hidden_dim": HIDDEN_DIM,
    "num_layers": NUM_LAYERS,
    "num_heads": NUM_HEADS,
    "head_dim": GLA_HEAD_DIM,
    "num_experts": NUM_EXPERTS,
    "top_k": TOP_K_EXPERTS,
    "router_prefix_layers": ROUTER_PREFIX_LAYERS,
    "reflex_exit_layer": REFLEX_EXIT_LAYER,
    "limbic_exit_layer": LIMBIC_EXIT_LAYER,
    "target_depth_dist": TARGET_DEPTH_DIST,
    "balance_coef": DEPTH_BALANCE_COEF,
    "bias_strength": DEPTH_BIAS_STRENGTH,
    "usage_ema_decay": DEPTH_USAGE_EMA,
    "depth_mode": "dynamic",
    "exploration": "linear",  # the reference's schedule name; a number is taken as a starting rate
    "exploration_steps": 5000,
    "exit_distill_coef": 0.2,
    "use_fp4": False,
    "use_fp8": False,
    "batch_size": 8,
    "seq_len": 256,
    "grad_accum_steps": 4,
    "total_steps": 50_000,
    "lr": 1e-4,
    "min_lr": 1e-6,
    "warmup_steps": 500,
    "betas": (0.9, 0.95),
    "weight_decay": 0.05,
    "grad_clip": 1.0,
    "grad_checkpoint": True,
    "galore": True,
    "galore_rank": GALORE_RANK,
    "galore_update_gap": GALORE_UPDATE_GAP,
    "galore_lr": GALORE_LR,
    "galore_betas": GALORE_BETAS,
    "galore_weight_decay": GALORE_WEIGHT_DECAY,
    "steer_scale": STEER_SCALE,
    "steer_update_gap": STEER_UPDATE_GAP,
    "use_triangular_core": True,
    "use_muon": True,
    "muon_lr": MUON_LR,
    "muon_momentum": MUON_MOMENTUM,
    "muon_weight_decay": MUON_WEIGHT_DECAY,
    "log_every": 10,
    "save_every": 1000,
    "eval_every": 200,
    "eval_batches": 5,
    "checkpoint_dir": "checkpoints_full",
    "cuda_graph": False,
    "layer_streaming": False,
    "seed": 0,
    # data source keys of the reference's run config (``triune/configs/config.py:62-65``); with no network the dataset
    # name is only a label unless ``dataset_path`` points at local files
    "shuffle_buffer": 4096,
    "dataset_name": "HuggingFaceFW/fineweb-edu",
    "dataset_config": "sample-10BT",
    "num_workers": 0,
}


def build_config(overrides: Optional[Dict[str, Any]] = None, preset: Optional[str] = None) -> Dict[str, Any]:
    """Return the flat run-config dict: defaults, then preset architecture, then overrides."""
    cfg = dict(_FLAT_DEFAULTS)
    if preset is not None:
        mc = get_model_config(preset)
        for k in (
            "vocab_size hidden_dim num_layers num_heads head_dim num_experts top_k router_prefix_layers "
            "reflex_exit_layer limbic_exit_layer"
        ).split():
            cfg[k] = getattr(mc, k)
        cfg["expert_hidden"] = mc.expert_hidden
        cfg["dense_hidden"] = mc.dense_hidden
        cfg["model_preset"] = preset
    if overrides:
        cfg.update({k: v for k, v in overrides.items() if v is not None})
    validate_config(cfg)
    return cfg


def validate_config(cfg: Dict[str, Any]) -> None:
    """Reject inconsistent or non-finite settings (fp4/fp8 exclusion, seq_len cap, NaN/Inf)."""
    if cfg.get("use_fp4") and cfg.get("use_fp8"):
        raise ValueError("use_fp4 and use_fp8 are mutually exclusive")
    if int(cfg.get("seq_len", 1)) < 1:
        raise ValueError("seq_len must be >= 1")
    if int(cfg.get("seq_len", 1)) > 65536:
        raise ValueError("seq_len above 65536 is not supported for training")
    for k, v in cfg.items():
        vals = v if isinstance(v, (tuple, list)) else (v,)
        for x in vals:
            if isinstance(x, float) and not math.isfinite(x):
                raise ValueError(f"config value {k!r} must be finite, got {x}")
    for k in ("lr", "min_lr", "weight_decay", "grad_clip"):
        if k in cfg and float(cfg[k]) < 0:
            raise ValueError(f"{k} must be non-negative")
    if cfg.get("depth_mode", "cortex") not in ("cortex", "joint", "dynamic"):
        raise ValueError(f"unknown depth_mode {cfg.get('depth_mode')!r}")
    tdd = cfg.get("target_depth_dist")
    if tdd is not None and abs(sum(float(x) for x in tdd) - 1.0) > 1e-4:
        raise ValueError("target_depth_dist must sum to 1")


def model_config_from_flat(cfg: Dict[str, Any]) -> ModelConfig:
    mc = ModelConfig.from_dict(cfg)
    return mc.validate()


def save_json(obj: Any, path: str) -> None:
    with open(path, "w") as f:
        json.dump(obj.to_dict() if hasattr(obj, "to_dict") else asdict(obj), f, indent=2)
