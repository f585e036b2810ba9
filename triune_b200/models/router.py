"""Depth router: picks Reflex / Limbic / Cortex per sequence after the prefix layers.

Parity: ``GumbelSoftmaxRouter`` (``triune/model/router.py:8-91``): pooled input
``0.75 * mean(last <=12 tokens) + 0.25 * mean(all)`` when T > 8, MLP d -> 256 -> 3, straight-through
Gumbel-softmax in training with a decoupled selection bias (step 0.01, clamp +-2), argmax of the biased
logits in evaluation, unweighted MSE balance loss against ``target_dist``.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class GumbelSoftmaxRouter(nn.Module):
    def __init__(self, hidden_dim: int, target_depth_dist=(0.34, 0.33, 0.33), balance_coef: float | None = None):
        super().__init__()
        self.router_mlp = nn.Sequential(nn.Linear(hidden_dim, 256), nn.ReLU(), nn.Linear(256, 3))
        vals = [float(v) for v in (target_depth_dist.tolist() if torch.is_tensor(target_depth_dist) else target_depth_dist)]
        if len(vals) != 3:
            raise ValueError(f"target_depth_dist must have 3 elements, got {target_depth_dist}")
        if abs(sum(vals) - 1.0) > 1e-4:
            raise ValueError(f"target_depth_dist must sum to 1.0, got {sum(vals):.4f}")
        t = torch.tensor(vals, dtype=torch.float32)  # validated on the host: construction also works on the meta device
        self.balance_coef = balance_coef
        self.register_buffer("target_dist", t)
        self.register_buffer("router_bias", torch.zeros(3, dtype=torch.float32))

    @property
    def target_depth_dist(self) -> torch.Tensor:
        return self.target_dist

    @staticmethod
    def pool(x: torch.Tensor) -> torch.Tensor:
        T = x.shape[1]
        if T > 8:
            return 0.75 * x[:, -min(T, 12):, :].mean(dim=1) + 0.25 * x.mean(dim=1)
        return x.mean(dim=1)

    def forward(self, x: torch.Tensor, temperature: float = 1.0, force_depth: int | None = None):
        if not math.isfinite(temperature) or temperature <= 0:
            raise ValueError(f"Gumbel-Softmax temperature must be a finite positive number, got {temperature}")
        B = x.shape[0]
        logits = self.router_mlp(self.pool(x))
        if force_depth is not None:
            y = F.one_hot(torch.full((B,), force_depth, device=x.device, dtype=torch.long), 3).float()
            return logits, y, torch.zeros((), device=x.device, dtype=x.dtype)
        lf = logits.float()
        sel = lf + self.router_bias
        if self.training:
            u = torch.rand_like(lf)
            gumbel = -torch.log(-torch.log(u + 1e-20) + 1e-20)
            y_soft = F.softmax((lf + gumbel) / temperature, dim=-1)
            hard = torch.zeros_like(lf).scatter_(-1, (sel + gumbel).argmax(-1, keepdim=True), 1.0)
            y = hard + y_soft - y_soft.detach()
            with torch.no_grad():
                self.router_bias.add_(-(y.detach().mean(0) - self.target_dist) * 0.01).clamp_(-2.0, 2.0)
        else:
            y = F.one_hot(sel.argmax(-1), 3).float()
        balance = (y.mean(0) - self.target_dist).pow(2).mean()
        return logits, y, balance
