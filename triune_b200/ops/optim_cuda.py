"""Optimizer math on the sm_100a kernels: batched Newton-Schulz on the tcgen05 GEMM, flat AdamW,
Muon momentum/apply, triangular AdamW core."""

from __future__ import annotations

import math

import torch

from .. import _ext


def ns_supported(G: torch.Tensor) -> bool:
    return (
        _ext.use_kernels(G)
        and G.dim() in (2, 3)
        and G.shape[-1] % 8 == 0
        and G.shape[-2] % 8 == 0
    )


def newton_schulz(G: torch.Tensor, steps: int = 3, coeffs=(1.875, -1.25, 0.375), eps: float = 1e-7) -> torch.Tensor:
    """Batched quintic Newton-Schulz polar iteration; every product runs on the tcgen05 GEMM.

    Per iteration: A = X X^T; T = c A A + b A; X <- T X + a X: three GEMM launches, the two blends in the GEMMs'
    add-rows epilogue. The spectral-norm safeguard of the reference (``triune/kernels/fast_muon.py:15-91``: Frobenius
    norm and a four-step power iteration) and the scaling run as five passes over X (one per power step, X^T (X v) in one
    read, rows split over CTAs) plus one scaling pass.
    """
    from . import gemm, _tick

    a, b, c = coeffs
    squeeze = G.dim() == 2
    X = G.unsqueeze(0) if squeeze else G
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    m, n = X.shape[-2], X.shape[-1]
    e = _ext.ext()
    if n <= 11568 and n % 8 == 0:
        # Frobenius norm, power iteration (one fused pass over X per step, rows split over CTAs) and scaling
        Xb = e.ns_prepare(X.to(torch.bfloat16).contiguous(), float(eps))
        _tick(6)
    else:
        Xf = X.float()
        fro = Xf.flatten(-2).norm(dim=-1).clamp_min(eps)
        vec = torch.full((Xf.shape[0], n, 1), 1.0 / math.sqrt(n), device=G.device, dtype=torch.float32)
        for _ in range(4):
            w = Xf @ vec
            vec = Xf.transpose(-1, -2) @ w
            vec = vec / vec.norm(dim=-2, keepdim=True).clamp_min(eps)
        sigma = (Xf @ vec).norm(dim=-2).squeeze(-1)
        safe = torch.maximum(torch.maximum(1.15 * sigma, fro / math.sqrt(m)), 0.7 * fro)
        Xb = (Xf / safe[:, None, None]).to(torch.bfloat16).contiguous()
    Xn = torch.empty_like(Xb)
    A = torch.empty(Xb.shape[0], m, m, device=G.device, dtype=torch.bfloat16)
    T = torch.empty_like(A)
    for _ in range(steps):
        gemm(Xb, Xb, A)                                   # A = X X^T
        gemm(A, A, T, alpha=c, add_aux=A, beta=b)         # T = c A A + b A   (A symmetric: A A^T = A A)
        gemm(T, Xb, Xn, b_mn=True, add_aux=Xb, beta=a)    # X <- T X + a X
        Xb, Xn = Xn, Xb
    out = Xb.transpose(-1, -2) if transposed else Xb
    out = out.to(G.dtype)
    return out.squeeze(0) if squeeze else out
