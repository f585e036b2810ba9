"""Stand-alone Muon optimizer for 2-D matrices (reference: ``triune/optim/muon.py:84-218``).

Momentum ``M <- lerp(M, G, 1-beta)``, Nesterov blend ``U = lerp(G, M, beta)``, same-shape matrices are
orthogonalised together by the batched Newton-Schulz iteration, update scale ``max(1, d_out/d_in)^0.5``
(times ``rms_target`` when given), decoupled weight decay.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch.optim import Optimizer

from .. import ops
from ..config import MUON_LR, MUON_MOMENTUM, MUON_WEIGHT_DECAY, NS_COEFFS, NS_STEPS


def zeropower_via_newtonschulz5(G: torch.Tensor, steps: int = NS_STEPS, coeffs=NS_COEFFS) -> torch.Tensor:
    """Approximate polar factor U V^T of G (2-D or batched 3-D); the input is left untouched."""
    return ops.muon_ns(G, steps=steps, coeffs=coeffs)


class Muon(Optimizer):
    def __init__(self, params, lr: float = MUON_LR, momentum: float = MUON_MOMENTUM,
                 weight_decay: float = MUON_WEIGHT_DECAY, nesterov: bool = True, ns_steps: int = NS_STEPS,
                 rms_target: Optional[float] = None, ns_coeffs=NS_COEFFS):
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov, ns_steps=ns_steps,
                        rms_target=rms_target, ns_coeffs=tuple(ns_coeffs))
        super().__init__(params, defaults)
        for g in self.param_groups:
            for p in g["params"]:
                if p.ndim != 2:
                    raise ValueError(f"Muon optimizer only supports 2D parameter matrices, got shape {tuple(p.shape)}")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            lr, beta, wd = g["lr"], g["momentum"], g["weight_decay"]
            buckets = {}
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Muon does not support sparse gradients")
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["momentum"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                gr = p.grad.float()
                st["momentum"].lerp_(gr, 1.0 - beta)
                upd = torch.lerp(gr, st["momentum"], beta) if g["nesterov"] else st["momentum"]
                buckets.setdefault((tuple(p.shape), p.device), []).append((p, upd))
            for (shape, _), items in buckets.items():
                U = torch.stack([u for _, u in items])
                O = zeropower_via_newtonschulz5(U, steps=g["ns_steps"], coeffs=g["ns_coeffs"])
                scale = max(1.0, shape[0] / shape[1]) ** 0.5 * (g["rms_target"] or 1.0)
                for (p, _), o in zip(items, O.unbind(0)):
                    if wd != 0.0:
                        p.mul_(1.0 - lr * wd)
                    p.add_(o.to(p.dtype), alpha=-lr * scale)
        return loss
