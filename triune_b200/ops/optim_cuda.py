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

    Per iteration: A = X X^T; B = b A + c A A; X <- a X + B X (five launches: three GEMMs with the
    blends folded into their accumulate epilogues, two scaled copies). The spectral-norm safeguard
    of the reference (``triune/kernels/fast_muon.py:15-91``) is computed with a short power iteration.
    """
    from . import gemm, _tick

    a, b, c = coeffs
    squeeze = G.dim() == 2
    X = G.unsqueeze(0) if squeeze else G
    transposed = X.shape[-2] > X.shape[-1]
    if transposed:
        X = X.transpose(-1, -2)
    Xf = X.float()
    m, n = Xf.shape[-2], Xf.shape[-1]
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
    e = _ext.ext()
    for _ in range(steps):
        A = gemm(Xb, Xb)  # [B, m, m]
        T = A * b
        gemm(A, A, T, alpha=c, accumulate=True)  # T = b A + c A A   (A symmetric: A A^T = A A)
        torch.mul(Xb, a, out=Xn)
        gemm(T, Xb, Xn, b_mn=True, accumulate=True)  # Xn = a X + T X
        Xb, Xn = Xn, Xb
    out = Xb.transpose(-1, -2) if transposed else Xb
    out = out.to(G.dtype)
    return out.squeeze(0) if squeeze else out
