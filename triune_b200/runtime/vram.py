"""Device-memory statistics and a pressure-driven layer offloader (reference: ``triune/runtime/vram.py:11-94``)."""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch


class VRAMProfiler:
    @staticmethod
    def get_vram_stats(device="cuda") -> Dict[str, Any]:
        if not torch.cuda.is_available():
            return {"available": False, "allocated_gb": 0.0, "reserved_gb": 0.0, "free_gb": 0.0, "total_gb": 0.0,
                    "peak_gb": 0.0, "utilization_pct": 0.0}
        dev = torch.device(device)
        free, total = torch.cuda.mem_get_info(dev)
        gb = 2.0**30
        return {"available": True, "device": torch.cuda.get_device_name(dev), "allocated_gb": torch.cuda.memory_allocated(dev) / gb,
                "reserved_gb": torch.cuda.memory_reserved(dev) / gb, "peak_gb": torch.cuda.max_memory_allocated(dev) / gb,
                "free_gb": free / gb, "total_gb": total / gb, "utilization_pct": 100.0 * (total - free) / max(1, total)}

    @staticmethod
    def check_oom_risk(threshold_pct: float = 0.90, device="cuda") -> bool:
        s = VRAMProfiler.get_vram_stats(device)
        return bool(s["available"] and s["utilization_pct"] >= threshold_pct * 100.0)


class AutoOffloader:
    """Moves registered layers to pinned host memory when utilisation crosses ``threshold_pct`` (largest first) and
    brings them back on request."""

    def __init__(self, threshold_pct: float = 0.90, device="cuda"):
        self.threshold_pct, self.device = threshold_pct, device
        self.candidates: List[Tuple[str, torch.nn.Module]] = []
        self.offloaded: Dict[str, torch.nn.Module] = {}

    def register(self, name: str, module: torch.nn.Module) -> None:
        self.candidates.append((name, module))

    def check_and_offload(self) -> bool:
        moved = False
        self.candidates.sort(key=lambda nm: -sum(p.numel() * p.element_size() for p in nm[1].parameters()))
        while self.candidates and VRAMProfiler.check_oom_risk(self.threshold_pct, self.device):
            name, mod = self.candidates.pop(0)
            self.offload_layer(name, mod)
            moved = True
        return moved

    def offload_layer(self, layer_name: str, layer_module: torch.nn.Module) -> None:
        for p in layer_module.parameters():
            host = torch.empty(p.shape, dtype=p.dtype, device="cpu", pin_memory=torch.cuda.is_available())
            host.copy_(p.data, non_blocking=True)
            p.data = host
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
            torch.cuda.empty_cache()
        self.offloaded[layer_name] = layer_module

    def restore_layer(self, layer_name: str, layer_module: Optional[torch.nn.Module] = None, target_device=None) -> None:
        mod = layer_module or self.offloaded.get(layer_name)
        if mod is None:
            return
        dev = torch.device(target_device or self.device)
        for p in mod.parameters():
            p.data = p.data.to(dev, non_blocking=True)
        self.offloaded.pop(layer_name, None)
        self.candidates.append((layer_name, mod))
