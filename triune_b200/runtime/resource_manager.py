"""Hardware probe, feasibility verdict and resource allotment before a run starts.

Parity (``triune/runtime/resource_manager.py:82-588``): ``probe_hardware`` -> ``HardwareProfile``;
``assess_feasibility`` -> FEASIBLE / TIGHT / HARD_LIMIT_EXCEEDED with suggested micro-batch and accumulation that keep
the effective batch; ``validate_and_allot`` raises ``VRAMBudgetExceededError`` unless ``force`` (and adopts the
suggestion under ``auto_fit`` when the user did not pin the batch size); ``bulk_to_device`` moves the model in stages
under a ceiling; ``LiveVRAMMonitor`` ticks during training and releases cached blocks when fragmentation grows.
The memory model is :class:`MemoryPlanner` (this framework's arena layout), scaled to 180 GB parts.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .memory_planner import GB, MemoryPlanner


class VRAMBudgetExceededError(RuntimeError):
    """The requested configuration does not fit the device and ``force`` was not given."""


@dataclass
class HardwareProfile:
    device_name: str
    total_vram_gb: float
    free_vram_gb: float
    used_vram_gb: float
    compute_capability: Tuple[int, int]
    supports_bf16: bool
    supports_fp8: bool
    has_transformer_engine: bool = False
    sm_count: int = 0
    num_devices: int = 0


@dataclass
class FeasibilityAssessment:
    model_name: str
    num_layers: int
    num_experts: int
    hidden_dim: int
    total_params: int
    precision: str
    param_memory_gb: float
    optimizer_memory_gb: float
    activation_memory_gb: float
    gradient_memory_gb: float
    cuda_overhead_gb: float
    estimated_total_gb: float
    available_vram_gb: float
    free_vram_gb: float
    safe_budget_gb: float
    headroom_gb: float
    status: str
    is_feasible: bool
    is_hard_exceeded: bool
    suggested_batch_size: int
    suggested_grad_accum: int
    recommendations: List[str] = field(default_factory=list)


@dataclass
class AllotmentPlan:
    config: Dict[str, Any]
    total_params: int
    param_memory_gb: float
    optimizer_memory_gb: float
    activation_memory_gb: float
    gradient_memory_gb: float
    estimated_total_gb: float
    available_vram_gb: float
    batch_size: int
    grad_accum_steps: int
    precision: str
    headroom_gb: float
    auto_fitted: bool
    forced_override: bool = False
    adjustment_reason: Optional[str] = None


class LiveVRAMMonitor:
    def __init__(self, device, defrag_threshold: float = 0.70):
        self.device = torch.device(device)
        self.defrag_threshold = defrag_threshold
        self.peak_allocated_gb = 0.0
        self.defrag_count = 0
        self.last: Dict[str, float] = {}

    def tick(self) -> Dict[str, float]:
        if self.device.type != "cuda" or not torch.cuda.is_available():
            self.last = {"allocated_gb": 0.0, "reserved_gb": 0.0, "total_gb": 0.0, "utilization": 0.0, "fragmentation": 0.0}
            return self.last
        alloc, res = torch.cuda.memory_allocated(self.device) / GB, torch.cuda.memory_reserved(self.device) / GB
        total = torch.cuda.get_device_properties(self.device).total_memory / GB
        self.peak_allocated_gb = max(self.peak_allocated_gb, alloc)
        frag = (res - alloc) / max(res, 1e-9)
        if res / total > self.defrag_threshold and frag > 0.25:  # a lot reserved, much of it idle: hand it back
            torch.cuda.empty_cache()
            self.defrag_count += 1
            res = torch.cuda.memory_reserved(self.device) / GB
        self.last = {"allocated_gb": alloc, "reserved_gb": res, "total_gb": total, "utilization": res / total, "fragmentation": frag,
                     "peak_allocated_gb": self.peak_allocated_gb, "defrag_count": float(self.defrag_count)}
        return self.last

    def format_telemetry(self) -> str:
        t = self.last or self.tick()
        return (f"VRAM {t['allocated_gb']:.2f}/{t['total_gb']:.1f} GB allocated, {t['reserved_gb']:.2f} GB reserved "
                f"({100 * t['utilization']:.0f}%), fragmentation {100 * t['fragmentation']:.0f}%")


class DynamicResourceManager:
    @staticmethod
    def probe_hardware(device=None) -> HardwareProfile:
        if not torch.cuda.is_available() or (device is not None and torch.device(device).type != "cuda"):
            import psutil

            vm = psutil.virtual_memory()
            return HardwareProfile("cpu", vm.total / GB, vm.available / GB, (vm.total - vm.available) / GB, (0, 0), False, False)
        dev = torch.device(device or "cuda:0")
        props = torch.cuda.get_device_properties(dev)
        free, total = torch.cuda.mem_get_info(dev)
        cc = (props.major, props.minor)
        try:
            import transformer_engine  # noqa: F401

            te = True
        except Exception:
            te = False
        return HardwareProfile(props.name, total / GB, free / GB, (total - free) / GB, cc, cc >= (8, 0), cc >= (8, 9), te,
                               props.multi_processor_count, torch.cuda.device_count())

    @classmethod
    def calculate_model_size(cls, config: Dict[str, Any], model: Optional[nn.Module] = None) -> Tuple[int, float]:
        if model is not None:
            n = sum(p.numel() for p in model.parameters())
            b = sum(p.numel() * p.element_size() for p in model.parameters())
            return n, b / GB
        est = MemoryPlanner.estimate_vram(config, available_vram_gb=1e9)
        return est.total_params, est.param_memory_gb

    @classmethod
    def assess_feasibility(cls, config: Dict[str, Any], device=None, user_overrides: Optional[Dict[str, Any]] = None,
                           safety_ceiling: float = 0.85, model: Optional[nn.Module] = None,
                           hardware: Optional[HardwareProfile] = None) -> FeasibilityAssessment:
        hw = hardware or cls.probe_hardware(device)
        cfg = {**config, **(user_overrides or {})}
        safe = hw.free_vram_gb * safety_ceiling
        batch, accum = int(cfg.get("batch_size", 16)), int(cfg.get("grad_accum_steps", 1))
        streaming = bool(cfg.get("streaming") or cfg.get("use_layer_streaming"))
        est = MemoryPlanner.estimate_vram(cfg, available_vram_gb=hw.total_vram_gb)
        params, opt, grad, act, over = est.param_memory_gb, est.optimizer_memory_gb, est.gradient_memory_gb, est.activation_memory_gb, est.overhead_gb
        if streaming:  # root + two staged layers on the device, masters and optimizer state on the host
            L = max(1, int(cfg.get("num_layers", 24)))
            params = params * (0.12 + 0.88 * 2.0 / L)
            opt, grad = 0.05, grad * 2.0 / L
            act = act / L * 2.0
        fixed = params + opt + grad + over
        total = fixed + act
        per_sample = act / max(1, batch)
        fit_batch = batch
        if total > safe and per_sample > 0:
            fit_batch = int(max(0.0, safe - fixed) / per_sample)
        hard = fixed > safe or fit_batch < 1
        fit_batch = max(1, min(batch, fit_batch))
        fit_accum = max(1, math.ceil(batch * accum / fit_batch))
        headroom = safe - total
        status = "HARD_LIMIT_EXCEEDED" if hard else ("FEASIBLE" if headroom > 0.1 * safe else ("TIGHT" if headroom >= 0 else "TIGHT"))
        feasible = not hard and total <= safe
        rec: List[str] = []
        if hard:
            rec.append("enable layer streaming (use_layer_streaming=True): only two layers are resident at a time")
            if not cfg.get("use_fp8") and not cfg.get("use_fp4"):
                rec.append("store weights in FP8 or NVFP4 for inference-only runs")
            if hw.num_devices > 1:
                rec.append(f"shard the optimizer state over the {hw.num_devices} GPUs of this node (fused data parallelism)")
        elif not feasible:
            rec.append(f"use micro-batch {fit_batch} with {fit_accum} accumulation steps (same effective batch)")
            if not cfg.get("gradient_checkpointing"):
                rec.append("enable activation checkpointing")
        return FeasibilityAssessment(str(cfg.get("model_name", cfg.get("preset", "custom"))), int(cfg.get("num_layers", 0)),
                                     int(cfg.get("num_experts", 0)), int(cfg.get("hidden_dim", 0)), est.total_params,
                                     est.recommended_precision, params, opt, act, grad, over, total, hw.total_vram_gb,
                                     hw.free_vram_gb, safe, headroom, status, feasible, hard, fit_batch, fit_accum, rec)

    @classmethod
    def format_assessment_report(cls, a: FeasibilityAssessment) -> str:
        lines = [f"Resource assessment for {a.model_name}: {a.status}",
                 f"  parameters      {a.total_params / 1e6:10.1f} M ({a.precision})",
                 f"  weights         {a.param_memory_gb:10.2f} GB", f"  optimizer       {a.optimizer_memory_gb:10.2f} GB",
                 f"  gradients       {a.gradient_memory_gb:10.2f} GB", f"  activations     {a.activation_memory_gb:10.2f} GB",
                 f"  runtime         {a.cuda_overhead_gb:10.2f} GB", f"  total           {a.estimated_total_gb:10.2f} GB",
                 f"  safe budget     {a.safe_budget_gb:10.2f} GB of {a.available_vram_gb:.1f} GB ({a.free_vram_gb:.1f} GB free)",
                 f"  headroom        {a.headroom_gb:10.2f} GB",
                 f"  suggestion      batch {a.suggested_batch_size} x accumulation {a.suggested_grad_accum}"]
        lines += [f"  - {r}" for r in a.recommendations]
        return "\n".join(lines)

    @classmethod
    def validate_and_allot(cls, config: Dict[str, Any], device=None, force: bool = False, auto_fit: bool = False,
                           user_overrides: Optional[Dict[str, Any]] = None, safety_ceiling: float = 0.85,
                           model: Optional[nn.Module] = None, hardware: Optional[HardwareProfile] = None) -> AllotmentPlan:
        over = user_overrides or {}
        a = cls.assess_feasibility(config, device, over, safety_ceiling, model, hardware)
        cfg = {**config, **over}
        reasons, fitted = [], False
        if auto_fit and "batch_size" not in over and not a.is_hard_exceeded and a.suggested_batch_size != cfg.get("batch_size", a.suggested_batch_size):
            reasons.append(f"auto-fit: micro-batch {cfg.get('batch_size')} -> {a.suggested_batch_size}, accumulation -> {a.suggested_grad_accum}")
            cfg["batch_size"], cfg["grad_accum_steps"] = a.suggested_batch_size, a.suggested_grad_accum
            fitted = True
        elif force:
            reasons.append("override 'force': proceeding regardless of the memory budget")
        elif not a.is_feasible:
            raise VRAMBudgetExceededError(cls.format_assessment_report(a) + "\n\nThe requested configuration exceeds the safe "
                                          "memory ceiling. Pass force=True (--force) to run anyway, or auto_fit=True (--auto_fit) "
                                          "to adopt the suggested micro-batch.")
        return AllotmentPlan(cfg, a.total_params, a.param_memory_gb, a.optimizer_memory_gb, a.activation_memory_gb,
                             a.gradient_memory_gb, a.estimated_total_gb, a.available_vram_gb,
                             int(cfg.get("batch_size", a.suggested_batch_size)), int(cfg.get("grad_accum_steps", a.suggested_grad_accum)),
                             a.precision, a.headroom_gb, fitted, force, " | ".join(reasons) or None)

    @staticmethod
    def bulk_to_device(model: nn.Module, device, dtype: torch.dtype = torch.bfloat16, force: bool = False,
                       safety_ceiling_pct: float = 0.92) -> nn.Module:
        """Move the model in stages (root modules, then layer by layer), checking allocated memory against the ceiling
        after each stage so an over-sized model stops with a clear error instead of an out-of-memory fault."""
        from ..utils import place_model

        device = torch.device(device)
        if device.type != "cuda" or not torch.cuda.is_available():
            return place_model(model, device, dtype)
        limit = torch.cuda.get_device_properties(device).total_memory * safety_ceiling_pct
        layers = list(getattr(model, "layers", []))
        layer_ids = {id(l) for l in layers}
        for child in model.children():
            if id(child) not in layer_ids and not isinstance(child, nn.ModuleList):
                place_model(child, device, dtype)
        for i, layer in enumerate(layers):
            place_model(layer, device, dtype)
            used = torch.cuda.memory_allocated(device)
            if not force and used >= limit:
                raise VRAMBudgetExceededError(f"stopped at layer {i + 1}/{len(layers)}: {used / GB:.2f} GB allocated exceeds "
                                              f"{safety_ceiling_pct:.0%} of the device; pass force=True or use layer streaming")
        place_model(model, device, dtype)  # anything not reached above (no-op for tensors already placed)
        return model
