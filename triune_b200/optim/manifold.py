"""Manifold-flavoured optimizers (reference: ``triune/optim/manifold.py:5-95``).

``LowSpaceWeightProjector`` keeps a rank-r left basis per matrix and maps gradients into / out of it
(GaLore style); ``UnitaryManifoldOptimizer`` moves square matrices along the orthogonal group with a Cayley
retraction so they stay orthogonal to round-off.
"""

from __future__ import annotations

import torch
from torch.optim import Optimizer

from .subspace import subspace_projection


class LowSpaceWeightProjector:
    def __init__(self, rank: int = 64, update_gap: int = 200):
        self.rank, self.update_gap = rank, update_gap
        self.basis = None
        self.step = 0

    def project(self, grad: torch.Tensor) -> torch.Tensor:
        if self.basis is None or self.step % self.update_gap == 0:
            self.basis = subspace_projection(grad, min(self.rank, min(grad.shape)))
        self.step += 1
        return self.basis.t() @ grad.float()

    def project_back(self, low: torch.Tensor) -> torch.Tensor:
        return self.basis @ low


class UnitaryManifoldOptimizer(Optimizer):
    """W <- (I + a/2 A)^-1 (I - a/2 A) W with A = G W^T - W G^T (skew), which preserves W^T W = I."""

    def __init__(self, params, lr: float = 1e-2):
        super().__init__(params, dict(lr=lr))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.ndim != 2 or p.shape[0] != p.shape[1]:
                    p.add_(p.grad, alpha=-g["lr"])
                    continue
                W, G = p.float(), p.grad.float()
                A = G @ W.t() - W @ G.t()
                eye = torch.eye(W.shape[0], device=W.device)
                p.copy_(torch.linalg.solve(eye + 0.5 * g["lr"] * A, (eye - 0.5 * g["lr"] * A) @ W).to(p.dtype))
        return loss


QuantumUnitaryOptimizer = UnitaryManifoldOptimizer
