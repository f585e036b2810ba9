"""RMSNorm module (reference: triune/model/norms.py:1-18)."""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor):
        """Fused (rmsnorm(x + residual), x + residual)."""
        return ops.add_rmsnorm(x, residual, self.weight, self.eps)
