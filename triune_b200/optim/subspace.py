"""Batched subspace algebra for the CentroidSteer tier: shifted CholeskyQR2 with a Householder
fall-back, randomized range finders, polar retraction.

Parity: ``triune/ops/centroid_steer.py:8-317`` of the reference (``batched_qr``, ``cholesky_qr``,
``polar_stiefel_retraction``, ``subspace_projection``, ``batched_subspace_projection``,
``triangular_steer_update``). The fast path is three batched products and two small triangular solves per
pass; slices that fail a health check (degenerate column, non-positive-definite Gram, condition estimate,
orthogonality residual) are re-done with Householder QR, and each failing slice is attributed to exactly one
primary reason.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

REASONS = ("degenerate_columns", "cholesky_non_positive_definite", "condition_ratio_exceeded",
           "orthogonality_tolerance_exceeded")


def new_qr_telemetry() -> Dict:
    return {
        "total_qr_calls": 0,
        "cholesky_fast_path_survivals": 0,
        "householder_fallbacks": 0,
        "primary_fallback_reasons": {k: 0 for k in REASONS},
        "overlapping_triggers": {k: 0 for k in REASONS},
    }


def flush_qr_telemetry(telemetry: Dict) -> Dict:
    """Fold the device-resident counters of :func:`batched_qr` into the dictionary (one device -> host read)."""
    pend = telemetry.pop("_pending", None)
    if pend is not None:
        vals = [int(v) for v in pend.tolist()]
        telemetry["householder_fallbacks"] += vals[0]
        for i, name in enumerate(REASONS):
            telemetry["primary_fallback_reasons"][name] += vals[1 + i]
            telemetry["overlapping_triggers"][name] += vals[5 + i]
    telemetry["cholesky_fast_path_survivals"] = telemetry["total_qr_calls"] - telemetry["householder_fallbacks"]
    return telemetry


def batched_qr(A: torch.Tensor, cond_threshold: float = 1e4, eps_shift: float = 1e-7, orth_tol: float = 1e-4,
               telemetry: Optional[Dict] = None, return_info: bool = False):
    """Orthonormal basis of the columns of each slice of A [K, d, r] (d >= r), fp32.

    sCholQR2: columns are normalised, G = A^T A + shift*I is Cholesky-factored, A <- A L^{-T}; done twice so
    the result is orthonormal to fp32 round-off for cond(A) up to ~1e4 (the shift bias of pass one is removed
    by pass two). Health checks per slice, any of which sends the slice to Householder QR:
      degenerate column (norm < 1e-12), Cholesky failure, diag(L) ratio above ``cond_threshold``,
      ||Q^T Q - I||_F above ``orth_tol``.
    """
    prev_tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False  # the Gram / orthogonality checks need full fp32 products
    try:
        return _batched_qr_impl(A, cond_threshold, eps_shift, orth_tol, telemetry, return_info)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev_tf32


def _batched_qr_impl(A, cond_threshold, eps_shift, orth_tol, telemetry, return_info):
    squeeze = A.dim() == 2
    X = (A.unsqueeze(0) if squeeze else A).float()
    K, d, r = X.shape
    col = X.norm(dim=1, keepdim=True)
    degen = (col < 1e-12).any(dim=-1).squeeze(1)
    Q = X / col.clamp_min(1e-12)
    eye = torch.eye(r, device=X.device, dtype=X.dtype)
    chol_fail = torch.zeros(K, dtype=torch.bool, device=X.device)
    cond_fail = torch.zeros(K, dtype=torch.bool, device=X.device)
    for p in range(2):
        G = Q.transpose(1, 2) @ Q
        if p == 0:
            G = G + eps_shift * eye * G.diagonal(dim1=-2, dim2=-1).mean(-1)[:, None, None].clamp_min(1.0)
        L, info = torch.linalg.cholesky_ex(G)
        bad = info != 0
        chol_fail |= bad
        L = torch.where(bad[:, None, None], eye.expand(K, r, r), L)
        dg = L.diagonal(dim1=-2, dim2=-1).abs()
        if p == 0:
            # a pivot sitting on the shift floor (ratio ~ 1/sqrt(shift)) means the columns were rank deficient
            limit = min(cond_threshold, 0.3 / math.sqrt(eps_shift))
            cond_fail |= (dg.amax(-1) / dg.amin(-1).clamp_min(1e-30)) > limit
        # Q <- Q L^{-T}  <=>  solve L Y = Q^T for Y = (Q_new)^T
        Q = torch.linalg.solve_triangular(L, Q.transpose(1, 2), upper=False).transpose(1, 2)
    orth_err = (Q.transpose(1, 2) @ Q - eye).flatten(1).norm(dim=-1)
    orth_fail = ~(orth_err <= orth_tol)  # also catches NaN
    fallback = degen | chol_fail | cond_fail | orth_fail
    if bool(fallback.any()):
        idx = fallback.nonzero(as_tuple=True)[0]
        Qh, _ = torch.linalg.qr(X[idx], mode="reduced")
        Q = Q.clone()
        Q[idx] = Qh
    if telemetry is not None:
        # Counters accumulate in a device tensor (no host synchronisation on the training path); they are folded into
        # the dictionary by flush_qr_telemetry at the reporting boundary
        # (``triune/optim/centroid.py:1393-1455`` of the reference).
        telemetry["total_qr_calls"] += K
        flags = (degen, chol_fail, cond_fail, orth_fail)
        taken = torch.zeros_like(fallback)
        rows = [fallback]
        prims = []
        for f in flags:
            prim = f & fallback & ~taken
            prims.append(prim)
            taken = taken | prim
        rows += prims + [f & fallback for f in flags]
        counts = torch.stack(rows, dim=0).sum(dim=-1, dtype=torch.long)
        pend = telemetry.get("_pending")
        if pend is None or pend.device != counts.device:
            flush_qr_telemetry(telemetry)
            telemetry["_pending"] = counts
        else:
            pend.add_(counts)
    Q = Q.squeeze(0) if squeeze else Q
    if return_info:
        return Q, {"fallback_mask": fallback, "orth_err": orth_err, "degenerate": degen, "cholesky": chol_fail,
                   "cond": cond_fail, "orth": orth_fail}
    return Q


def cholesky_qr(A: torch.Tensor) -> torch.Tensor:
    """Single-matrix convenience wrapper of :func:`batched_qr`."""
    return batched_qr(A)


def polar_stiefel_retraction(X: torch.Tensor, steps: int = 5) -> torch.Tensor:
    """Nearest matrix with orthonormal columns (polar factor) by Newton-Schulz iteration."""
    from ..ops import reference as ref

    return ref.newton_schulz(X, steps=max(steps, 8))


_SKETCH_GENERATORS: Dict[str, torch.Generator] = {}
_SKETCH_SEED = 0x5EED


def set_sketch_seed(seed: int) -> None:
    """Seed of the Gaussian sketches. Every data-parallel replica must draw the same sketches or the replicas' expert
    weights drift apart, so the sketches come from a dedicated generator and never from the global RNG (which ranks
    seed differently for data order and dropout)."""
    global _SKETCH_SEED
    _SKETCH_SEED = int(seed)
    _SKETCH_GENERATORS.clear()


def _sketch(shape, device) -> torch.Tensor:
    key = str(device)
    g = _SKETCH_GENERATORS.get(key)
    if g is None:
        g = torch.Generator(device=device)
        g.manual_seed(_SKETCH_SEED)
        _SKETCH_GENERATORS[key] = g
    return torch.randn(shape, device=device, dtype=torch.float32, generator=g)


def subspace_projection(G: torch.Tensor, rank: int, oversample: int = 4, power_iters: int = 1) -> torch.Tensor:
    """Randomized range finder: orthonormal basis [m, rank] of the dominant left subspace of G [m, n]."""
    return batched_subspace_projection(G.unsqueeze(0), rank, oversample, power_iters)[0]


def batched_subspace_projection(G: torch.Tensor, rank: int, oversample: int = 4, power_iters: int = 1) -> torch.Tensor:
    K, m, n = G.shape
    r = min(rank + oversample, m, n)
    Gf = G.float()
    Y = Gf @ _sketch((K, n, r), G.device)
    Q = batched_qr(Y)
    for _ in range(power_iters):
        Q = batched_qr(Gf @ batched_qr(Gf.transpose(1, 2) @ Q))
    # rotate to the dominant directions with a small eigen-decomposition
    Bm = Q.transpose(1, 2) @ Gf
    w, V = torch.linalg.eigh(Bm @ Bm.transpose(1, 2))
    V = V.flip(-1)[:, :, : min(rank, r)]
    return Q @ V


def two_sided_bases(G: torch.Tensor, r: int, telemetry: Optional[Dict] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gaussian sketch + three QR passes: (Q_L [K,m,r], Q_R [K,n,r]) capturing the dominant subspaces of G."""
    K, m, n = G.shape
    Gf = G.float()
    Y = Gf @ _sketch((K, n, r), G.device)
    QL = batched_qr(Y, telemetry=telemetry)
    QR = batched_qr(Gf.transpose(1, 2) @ QL, telemetry=telemetry)
    QL = batched_qr(Gf @ QR, telemetry=telemetry)
    return QL, QR


def reorthogonalise(vec: torch.Tensor, Q: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Component of vec [K,d] orthogonal to span(Q [K,d,r]) with two Gram-Schmidt passes (Kahan-Parlett
    "twice is enough"); returns (unit vector or 0, norm of the residual)."""
    v = vec.unsqueeze(-1)
    for _ in range(2):
        v = v - Q @ (Q.transpose(1, 2) @ v)
    v = v.squeeze(-1)
    nrm = v.norm(dim=-1, keepdim=True)
    unit = torch.where(nrm > 1e-8, v / nrm.clamp_min(1e-8), torch.zeros_like(v))
    return unit, nrm.squeeze(-1)
