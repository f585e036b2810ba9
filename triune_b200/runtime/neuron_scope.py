"""Live activation sampling for the visualiser.

Parity (``triune/runtime/neuron_scope.py:15-108``): forward hooks on every block keep a ``[<=32 tokens, <=64 dims]``
sample of the first sequence, the last 64 routing decisions are recorded, and ``get_snapshot`` returns per-layer
heatmaps, 64-bin magnitude histograms and the active depth tier. Binning runs in the heatmap kernel on the GPU (or the
AVX2 path of the C library on the host), and samples stay on the device until a snapshot is requested: one transfer per
snapshot instead of one per layer per forward.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn

TIER_NAMES = {0: "Reflex", 1: "Limbic", 2: "Cortex"}


class NeuronScope:
    def __init__(self, model: Optional[nn.Module] = None, max_tokens: int = 32, max_dims: int = 64):
        self.model, self.max_tokens, self.max_dims = model, max_tokens, max_dims
        self.is_active = False
        self.activations: Dict[int, torch.Tensor] = {}
        self.router_decisions: List[int] = []
        self._hooks: List[Any] = []

    def attach(self, model: Optional[nn.Module] = None) -> None:
        if model is not None and model is not self.model:
            self.detach()
            self.model = model
        if self._hooks or self.model is None:
            return
        layers = getattr(self.model, "layers", None)
        if layers is None:
            for holder in ("transformer", "model"):
                layers = getattr(getattr(self.model, holder, None), "layers", None)
                if layers is not None:
                    break
        for i, layer in enumerate(layers or ()):
            self._hooks.append(layer.register_forward_hook(self._make_layer_hook(i)))
        self.is_active = True

    def _make_layer_hook(self, idx: int):
        def hook(module, inputs, output):
            if not self.is_active:
                return
            t = output[0] if isinstance(output, tuple) else output
            if not torch.is_tensor(t) or t.ndim < 2:
                return
            act = t.detach()[0] if t.ndim >= 3 else t.detach()
            self.activations[idx] = act[: self.max_tokens, : self.max_dims].float()

        return hook

    def record_routing(self, selected_tier: int) -> None:
        self.router_decisions.append(int(selected_tier))
        del self.router_decisions[:-64]

    def get_snapshot(self, num_bins: int = 64) -> Dict[str, Any]:
        from .. import ops

        heat, bins = {}, {}
        for i, act in sorted(self.activations.items()):
            heat[i] = act.cpu().tolist()
            try:
                hist = ops.neuron_heatmap(act, num_bins)
                bins[i] = (hist[0] if isinstance(hist, (tuple, list)) else hist).float().cpu().tolist()
            except Exception:
                mag = act.abs().flatten()
                bins[i] = torch.histc(mag, bins=num_bins, min=0.0, max=float(mag.max()) + 1e-12).tolist()
        tier = self.router_decisions[-1] if self.router_decisions else 0
        dc = getattr(self.model, "last_depth_choice", None)
        if isinstance(dc, int):
            tier = dc
        elif torch.is_tensor(dc) and dc.numel() > 0:
            tier = int(dc.reshape(-1)[0])
        n_layers = getattr(self.model, "num_layers", None) or getattr(getattr(self.model, "config", None), "num_hidden_layers", None)
        native = None
        try:
            from ..ops._c_bridge import get_native_c_info

            native = get_native_c_info()
        except Exception:
            pass
        return {"layers": heat, "layer_bins": bins, "num_layers": int(n_layers or len(bins) or 8),
                "router_history": self.router_decisions[-16:], "active_tier": tier, "active_tier_name": TIER_NAMES.get(tier, "Reflex"),
                "native_c_engine": native}

    def detach(self, *, clear: bool = True) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()
        self.is_active = False
        if clear:
            self.activations.clear()
        else:  # keep host copies only, so a paused viewer holds no device memory
            self.activations = {k: v.cpu() for k, v in self.activations.items()}
