"""Early-exit retrofits for models that were not trained with exits.

Parity: ``WeightTiedExitProjection``, ``EarlyExitManager``, ``attach_early_exits`` and ``generate_adaptive``
(``triune/model/adapters.py:49-414``). An exit head is a rank-r bottleneck in front of the model's own LM head
(``logits = head(norm(x) + W_up gelu(W_down norm(x)))``, zero-initialised ``W_up`` so it starts as the base head), about
``2*r*d`` parameters per exit instead of ``d*V``. ``attach_early_exits`` finds the layer list and the LM head of a
Hugging Face style model or a TriuneTransformer, hooks two intermediate layers and adds ``generate_adaptive``:
token-level gating by softmax margin / normalised top-16 entropy, or by JEV latent confidence.

Difference: the gate is evaluated on the device and read back with ONE host transfer per token (three booleans)
instead of several ``.item()`` calls per exit.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .jev import JEVExitRouter, JEVLatentPredictor
from .norms import RMSNorm

_LAYER_PATHS = ("layers", "model.layers", "transformer.h", "transformer.layers", "decoder.layers", "gpt_neox.layers")
_HEAD_NAMES = ("final_head", "lm_head", "embed_out", "output")


class WeightTiedExitProjection(nn.Module):
    def __init__(self, hidden_dim: int, base_head: nn.Module, rank: int = 64, eps: float = 1e-6):
        super().__init__()
        self.hidden_dim, self.rank = hidden_dim, rank
        self.norm = RMSNorm(hidden_dim, eps=eps)
        self.down_proj = nn.Linear(hidden_dim, rank, bias=False)
        self.up_proj = nn.Linear(rank, hidden_dim, bias=False)
        nn.init.kaiming_uniform_(self.down_proj.weight, a=math.sqrt(5))
        nn.init.zeros_(self.up_proj.weight)
        object.__setattr__(self, "base_head", base_head)  # shared, deliberately not registered as a sub-module

    def adapter_parameters(self) -> List[nn.Parameter]:
        return [*self.norm.parameters(), *self.down_proj.parameters(), *self.up_proj.parameters()]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xn = self.norm(x)
        return self.base_head(xn + self.up_proj(F.gelu(self.down_proj(xn))))


class EarlyExitManager:
    """Captures the outputs of the two tapped layers during a forward pass."""

    def __init__(self, model, reflex_layer_idx, limbic_layer_idx, reflex_head, limbic_head, layer_list):
        self.model, self.layer_list = model, layer_list
        self.reflex_layer_idx, self.limbic_layer_idx = reflex_layer_idx, limbic_layer_idx
        self.reflex_head, self.limbic_head = reflex_head, limbic_head
        self.intermediate_activations: Dict[int, torch.Tensor] = {}
        self.handles = []

    def capture_hook(self, layer_idx: int):
        def hook(module, inputs, output):
            self.intermediate_activations[layer_idx] = output[0] if isinstance(output, tuple) else output

        return hook

    def remove(self):
        for h in self.handles:
            h.remove()
        self.handles.clear()


def _resolve(model, path):
    cur = model
    for part in path.split("."):
        if not hasattr(cur, part):
            return None
        cur = getattr(cur, part)
    return cur


def attach_early_exits(model: nn.Module, reflex_layer: Optional[int] = None, limbic_layer: Optional[int] = None,
                       rank: int = 64, use_jev: bool = False, jev_threshold: float = 0.85) -> nn.Module:
    layers = next((l for l in (_resolve(model, p) for p in _LAYER_PATHS) if isinstance(l, (nn.ModuleList, list))), None)
    if layers is None:
        raise ValueError("could not find the transformer layer list (tried: %s)" % ", ".join(_LAYER_PATHS))
    head = next((getattr(model, n) for n in _HEAD_NAMES if isinstance(getattr(model, n, None), nn.Linear)), None)
    if head is None:
        raise ValueError("could not find the final linear head (tried: %s)" % ", ".join(_HEAD_NAMES))
    d = getattr(model, "hidden_dim", None) or getattr(getattr(model, "config", None), "hidden_size", None) or head.in_features
    n = len(layers)
    r_idx = reflex_layer if reflex_layer is not None else max(1, int(n * 0.25))
    l_idx = limbic_layer if limbic_layer is not None else max(r_idx + 1, int(n * 0.60))
    p0 = next(model.parameters())
    model.reflex_head = WeightTiedExitProjection(d, head, rank).to(device=p0.device, dtype=p0.dtype)
    model.limbic_head = WeightTiedExitProjection(d, head, rank).to(device=p0.device, dtype=p0.dtype)
    model.reflex_layer_idx, model.limbic_layer_idx = r_idx, l_idx
    mgr = EarlyExitManager(model, r_idx, l_idx, model.reflex_head, model.limbic_head, layers)
    model._exit_manager = mgr
    if use_jev:
        for name, th in (("reflex", jev_threshold), ("limbic", jev_threshold * 0.85)):
            pred = JEVLatentPredictor(d).to(device=p0.device, dtype=p0.dtype)
            setattr(model, f"{name}_jev_predictor", pred)
            setattr(model, f"{name}_jev_router", JEVExitRouter(d, threshold=th, predictor=pred).to(device=p0.device, dtype=p0.dtype))
        model.use_jev = True
    mgr.handles = [layers[r_idx].register_forward_hook(mgr.capture_hook(r_idx)),
                   layers[l_idx].register_forward_hook(mgr.capture_hook(l_idx))]

    def _bound(input_ids, **kw):
        return generate_adaptive(model, input_ids, **kw)

    model.generate_adaptive = _bound
    return model


def _gate(logits: torch.Tensor, temperature: float, threshold: float) -> torch.Tensor:
    """Device-side exit test on [1, V] logits: margin p1-p2 >= threshold, or (p1 >= 0.7*scale and normalised entropy of
    the re-normalised top-16 <= 0.35). ``threshold`` already carries the tier scale."""
    probs = F.softmax(logits.float() / max(temperature, 1e-5), dim=-1)
    k = min(16, probs.size(-1))
    top = torch.topk(probs, k=k, dim=-1).values[0]
    p1, p2 = top[0], (top[1] if k > 1 else top.new_zeros(()))
    tn = top / top.sum().clamp_min(1e-12)
    h = -(tn * tn.clamp_min(1e-12).log()).sum() / max(math.log(k), 1e-12)
    return (p1 - p2 >= threshold[0]) | ((p1 >= 0.70 * threshold[1]) & (h <= 0.35))


@torch.inference_mode()
def generate_adaptive(model: nn.Module, input_ids: torch.Tensor, confidence_threshold: float = 0.85,
                      max_new_tokens: int = 128, temperature: float = 0.7, pad_token_id: Optional[int] = None,
                      eos_token_id: Optional[int] = None, use_jev: Optional[bool] = None) -> Dict[str, Any]:
    if input_ids.size(0) != 1:
        raise ValueError(f"generate_adaptive supports batch_size=1 only; got {input_ids.size(0)}")
    dev = input_ids.device
    ids = input_ids.clone()
    mgr = getattr(model, "_exit_manager", None)
    n_layers = len(mgr.layer_list) if mgr is not None else getattr(model, "num_layers", 24)
    r_idx, l_idx = getattr(model, "reflex_layer_idx", n_layers // 4), getattr(model, "limbic_layer_idx", (3 * n_layers) // 5)
    jev = (getattr(model, "use_jev", False) if use_jev is None else use_jev) and hasattr(model, "reflex_jev_router")
    counts = [0, 0, 0]
    new: List[int] = []
    for _ in range(max_new_tokens):
        if mgr is not None:
            mgr.intermediate_activations.clear()
        if hasattr(model, "forward_all_exits"):
            out = model.forward_all_exits(ids)
            cand = [o[:, -1, :] for o in out[:3]]
            flags = None
        else:
            out = model(ids)
            full = out.logits if hasattr(out, "logits") else (out[0] if isinstance(out, tuple) else out)
            c_logits = full[:, -1, :]
            acts = mgr.intermediate_activations if mgr is not None else {}
            if r_idx in acts and l_idx in acts:
                r_act, l_act = acts[r_idx][:, -1, :], acts[l_idx][:, -1, :]
                cand = [model.reflex_head(r_act), model.limbic_head(l_act), c_logits]
                flags = None
                if jev:
                    er, _ = model.reflex_jev_router.evaluate_latent_exit(r_act, threshold=confidence_threshold)
                    el, _ = model.limbic_jev_router.evaluate_latent_exit(l_act, threshold=confidence_threshold * 0.85)
                    flags = torch.stack((er.reshape(-1)[0], el.reshape(-1)[0]))
            else:
                cand, flags = [c_logits, c_logits, c_logits], None
        if flags is None:
            flags = torch.stack((_gate(cand[0], temperature, (confidence_threshold, 1.0)),
                                 _gate(cand[1], temperature, (confidence_threshold * 0.85, 0.85))))
        fr, fl = flags.tolist()  # the only host read of the gate
        tier = 0 if fr else (1 if fl else 2)
        counts[tier] += 1
        lg = cand[tier][0].float() / max(temperature, 1e-5)
        if pad_token_id is not None:
            lg[pad_token_id] = float("-inf")
        tok = int(lg.argmax()) if temperature <= 0.05 else int(torch.multinomial(F.softmax(lg, -1), 1))
        if eos_token_id is not None and tok == eos_token_id:
            break
        new.append(tok)
        ids = torch.cat((ids, torch.tensor([[tok]], device=dev)), dim=1)
    total = max(1, len(new))
    depth = (counts[0] * r_idx / n_layers + counts[1] * l_idx / n_layers + counts[2]) / total
    names = ("reflex", "limbic", "cortex")
    return {"output_ids": ids, "generated_token_ids": new, "exit_counts": dict(zip(names, counts)),
            "exit_percentages": {k: round(c / total * 100, 1) for k, c in zip(names, counts)},
            "flops_saved_pct": max(0.0, round((1.0 - depth) * 100, 1)),
            "effective_speedup": round(1.0 / max(0.2, depth), 2)}
