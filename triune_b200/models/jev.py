"""Joint-embedding latent exits (JEV): a latent predictor, its training objective and an exit router that decides
from distances in hidden space instead of from a vocabulary-sized head.

Parity: ``JEVLatentPredictor`` / ``JEVObjective`` / ``JEVExitRouter`` / ``JEVRoutingResult``
(``triune/model/jev.py:14-280``): predictor = RMSNorm -> Linear(d, d/2) -> GELU -> Linear(d/2, d) [-> RMSNorm];
objective = (1 - cos) + lambda_stp * tube(distance^2 - eps^2) + lambda_cov * off-diagonal covariance energy;
router metrics cosine / euclidean / geodesic / stp_tube / learned gate.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from .norms import RMSNorm

_METRICS = ("cosine", "euclidean", "geodesic", "stp_tube", "learned")
_STP_MODES = ("geodesic", "euclidean", "stiefel")


@dataclass
class JEVRoutingResult:
    should_exit: torch.Tensor
    confidence: torch.Tensor
    distance: torch.Tensor


class JEVLatentPredictor(nn.Module):
    def __init__(self, dim: int, d_pred: Optional[int] = None, eps: float = 1e-6, bias: bool = False,
                 normalize_output: bool = True, use_residual: bool = False):
        super().__init__()
        if dim <= 0:
            raise ValueError(f"dim must be positive, got {dim}")
        self.dim, self.d_pred = dim, d_pred if d_pred is not None else max(1, dim // 2)
        self.use_residual = use_residual
        self.norm = RMSNorm(dim, eps=eps)
        self.w1 = nn.Linear(dim, self.d_pred, bias=bias)
        self.w2 = nn.Linear(self.d_pred, dim, bias=bias)
        self.out_norm = RMSNorm(dim, eps=eps) if normalize_output else None
        nn.init.kaiming_uniform_(self.w1.weight, a=math.sqrt(5))
        nn.init.normal_(self.w2.weight, std=0.02)
        for lin in (self.w1, self.w2):
            if lin.bias is not None:
                nn.init.zeros_(lin.bias)

    # the reference exposes the same sub-modules under these names as well
    @property
    def down_proj(self):
        return self.w1

    @property
    def up_proj(self):
        return self.w2

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        zn = self.norm(z)
        out = self.w2(F.gelu(self.w1(zn)))
        if self.use_residual:
            out = zn + out
        if self.out_norm is not None:
            out = self.out_norm(out)
        return out.to(z.dtype)


def _unit(x, eps):
    return F.normalize(x, p=2, dim=-1, eps=eps)


class JEVObjective(nn.Module):
    def __init__(self, lambda_stp: float = 1.0, lambda_cov: float = 0.04, eps_tube: float = 0.1, eps_sim: float = 1e-8,
                 stp_mode: str = "euclidean"):
        super().__init__()
        if stp_mode not in _STP_MODES:
            raise ValueError(f"Unsupported stp_mode: {stp_mode}; expected one of {_STP_MODES}")
        self.lambda_stp, self.lambda_cov = float(lambda_stp), float(lambda_cov)
        self.eps_tube, self.eps_sim, self.stp_mode = float(eps_tube), float(eps_sim), stp_mode
        self.last: Dict[str, torch.Tensor] = {}

    def compute_sim_loss(self, z_pred, z_target):
        return (1.0 - F.cosine_similarity(z_pred.float(), z_target.detach().float(), dim=-1, eps=self.eps_sim)).mean()

    def compute_stp_loss(self, z_pred, z_target):
        p, t = z_pred.float(), z_target.detach().float()
        tube = self.eps_tube**2
        if self.stp_mode == "euclidean":
            d2 = (p - t).pow(2).sum(-1)
        else:
            c = (_unit(p, self.eps_sim) * _unit(t, self.eps_sim)).sum(-1)
            if self.stp_mode == "geodesic":  # squared great-circle distance on the unit sphere
                d2 = torch.acos(c.clamp(-1.0 + 1e-7, 1.0 - 1e-7)).pow(2)
            else:  # "stiefel": projection metric between the two lines
                d2 = 1.0 - c.pow(2)
        return F.relu(d2 - tube).mean()

    def compute_cov_loss(self, z):
        zf = z.float().reshape(-1, z.size(-1))
        n, d = zf.shape
        if n <= 1:
            return zf.sum() * 0.0
        zc = zf - zf.mean(0, keepdim=True)
        cov = zc.t() @ zc / (n - 1)
        return (cov.pow(2).sum() - cov.diagonal().pow(2).sum()) / d

    def forward(self, z_pred, z_target, return_dict: bool = False
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, Dict[str, torch.Tensor]]]:
        l_sim, l_stp, l_cov = (self.compute_sim_loss(z_pred, z_target), self.compute_stp_loss(z_pred, z_target),
                               self.compute_cov_loss(z_pred))
        total = l_sim + self.lambda_stp * l_stp + self.lambda_cov * l_cov
        # device tensors, no host reads: callers that want floats call .item() themselves
        self.last = {"l_sim": l_sim.detach(), "l_stp": l_stp.detach(), "l_cov": l_cov.detach(), "total_loss": total.detach()}
        if return_dict:
            return total, {"l_sim": l_sim, "l_stp": l_stp, "l_cov": l_cov, "total_loss": total}
        return total

    @property
    def last_total_loss(self) -> Optional[float]:
        return float(self.last["total_loss"]) if self.last else None

    # the three terms of the last call as floats (one host read each, made when asked for)
    @property
    def last_sim_loss(self) -> Optional[float]:
        return float(self.last["l_sim"]) if self.last else None

    @property
    def last_stp_loss(self) -> Optional[float]:
        return float(self.last["l_stp"]) if self.last else None

    @property
    def last_cov_loss(self) -> Optional[float]:
        return float(self.last["l_cov"]) if self.last else None


class JEVExitRouter(nn.Module):
    def __init__(self, dim: int, threshold: float = 0.85, distance_metric: str = "cosine",
                 predictor: Optional[JEVLatentPredictor] = None, eps_tube: float = 0.1):
        super().__init__()
        if dim <= 0:
            raise ValueError(f"dim must be positive, got {dim}")
        if distance_metric not in _METRICS:
            raise ValueError(f"Unsupported distance_metric: {distance_metric}")
        self.dim, self.threshold, self.distance_metric, self.eps_tube = dim, float(threshold), distance_metric, float(eps_tube)
        self.predictor = predictor
        self.gate = nn.Linear(dim, 1)
        nn.init.normal_(self.gate.weight, std=0.02)
        nn.init.zeros_(self.gate.bias)

    def _cos(self, z, ref):
        return F.cosine_similarity(z.float(), ref.float(), dim=-1, eps=1e-8)

    def compute_latent_distance(self, z, z_ref=None):
        m = self.distance_metric
        if z_ref is None or m == "learned":
            return F.softplus(self.gate(z)).squeeze(-1)
        if m == "cosine":
            return (1.0 - self._cos(z, z_ref)).clamp(0.0, 2.0)
        if m == "euclidean":
            return (z.float() - z_ref.float()).norm(dim=-1)
        if m == "geodesic":
            return torch.arccos(self._cos(z, z_ref).clamp(-1.0 + 1e-7, 1.0 - 1e-7))
        return F.relu((z.float() - z_ref.float()).pow(2).sum(-1) - self.eps_tube**2)  # stp_tube

    def compute_latent_confidence(self, z, z_ref=None):
        m = self.distance_metric
        if z_ref is None or m == "learned":
            return torch.sigmoid(self.gate(z)).squeeze(-1)
        if m == "cosine":
            return self._cos(z, z_ref).clamp(0.0, 1.0)
        if m == "geodesic":
            return (1.0 - self.compute_latent_distance(z, z_ref) / math.pi).clamp(0.0, 1.0)
        return torch.exp(-self.compute_latent_distance(z, z_ref))

    def evaluate_latent_exit(self, z, z_target=None, threshold: Optional[float] = None):
        r = self.forward(z, z_target, threshold)
        return r.should_exit, r.confidence

    def forward(self, z, z_target=None, threshold: Optional[float] = None) -> JEVRoutingResult:
        th = self.threshold if threshold is None else float(threshold)
        zp = self.predictor(z) if self.predictor is not None else z
        conf = self.compute_latent_confidence(zp, z_target)
        return JEVRoutingResult(conf >= th, conf, self.compute_latent_distance(zp, z_target))


LatentPredictor = TriuneLatentPredictor = JEVLatentPredictor
JointEmbeddingObjective = TriuneLatentObjective = JEVObjective
ContinuousLatentExitRouter = TriuneContinuousExitRouter = JEVExitRouter
