"""Numerical residuals of the fast orthonormalisation used by the subspace optimizer tier, and how often it holds.

The tier orthonormalises tall matrices with a shifted Cholesky QR done twice (``optim/subspace.batched_qr``) and falls
back to Householder QR for slices whose health checks fail. This evaluation measures, on matrices of controlled
condition number and on gradients of a real training run, (a) the residuals of the fast path against Householder QR
in fp64: orthogonality ``||Q^T Q - I||_F``, projector distance ``||Q Q^T - Q_ref Q_ref^T||_F`` (the basis is only
defined up to rotation, the subspace is what matters), and reconstruction ``||Q Q^T A - A||_F / ||A||_F``; (b) the
share of calls that stay on the fast path and the first reason for each fallback; (c) that rank-deficient and
zero-column inputs are caught by the checks instead of returning a bad basis.

The reference reports the fast-path survival of a training run (83.76 % of 11,832 calls) and verifies the residuals
in ``benchmarks/verify_triangular_qr_residuals.py:1113-1600``; its statistical comparison of whole training runs is
not repeated here.

    python -m triune_b200.evals.qr_residuals
    python -m triune_b200.evals.qr_residuals --train-steps 30      # adds survival on the gradients of a small model
"""

from __future__ import annotations

import argparse
import json
from typing import Dict, List

import torch

from ..optim.subspace import batched_qr, flush_qr_telemetry, new_qr_telemetry


def conditioned(K: int, d: int, r: int, cond: float, gen: torch.Generator, dtype=torch.float32) -> torch.Tensor:
    """K matrices [d, r] whose singular values fall geometrically from 1 to 1 / cond."""
    U, _ = torch.linalg.qr(torch.randn(K, d, r, generator=gen, dtype=torch.float64))
    V, _ = torch.linalg.qr(torch.randn(K, r, r, generator=gen, dtype=torch.float64))
    s = torch.logspace(0, -torch.log10(torch.tensor(float(cond))).item(), r, dtype=torch.float64)
    return (U * s) @ V.transpose(1, 2)


def residuals(A: torch.Tensor, device="cpu") -> Dict:
    """Fast path against fp64 Householder QR on the slices of A [K, d, r] (given in fp64; the fast path sees fp32)."""
    tel = new_qr_telemetry()
    Q, info = batched_qr(A.to(device=device, dtype=torch.float32), telemetry=tel, return_info=True)
    flush_qr_telemetry(tel)
    Q = Q.double().cpu()
    Qr, _ = torch.linalg.qr(A, mode="reduced")
    eye = torch.eye(A.shape[-1], dtype=torch.float64)
    orth = (Q.transpose(1, 2) @ Q - eye).flatten(1).norm(dim=-1)
    proj = (Q @ Q.transpose(1, 2) - Qr @ Qr.transpose(1, 2)).flatten(1).norm(dim=-1)
    recon = (Q @ (Q.transpose(1, 2) @ A) - A).flatten(1).norm(dim=-1) / A.flatten(1).norm(dim=-1).clamp_min(1e-300)
    fb = info["fallback_mask"].cpu()
    fast = ~fb
    pick = lambda v, m: float(v[m].max()) if bool(m.any()) else None
    return {"slices": int(A.shape[0]), "fast_path": int(fast.sum()), "fallbacks": int(fb.sum()),
            "primary_reasons": {k: v for k, v in tel["primary_fallback_reasons"].items() if v},
            "fast_path_max": {"orthogonality": pick(orth, fast), "projector_distance": pick(proj, fast), "reconstruction": pick(recon, fast)},
            "all_max": {"orthogonality": float(orth.max()), "projector_distance": float(proj.max()), "reconstruction": float(recon.max())}}


def sweep(K: int = 64, d: int = 384, r: int = 32, conds=(1e1, 1e2, 1e3, 1e4, 1e5, 1e6), seed: int = 0, device="cpu") -> List[Dict]:
    g = torch.Generator().manual_seed(seed)
    return [{"condition_number": c, "shape": [d, r], **residuals(conditioned(K, d, r, c, g), device)} for c in conds]


def degenerate_cases(d: int = 128, r: int = 16, device="cpu") -> Dict:
    """Inputs the fast path must refuse: a zero column, a repeated column, an all-zero matrix."""
    g = torch.Generator().manual_seed(1)
    base = torch.randn(3, d, r, generator=g, dtype=torch.float64)
    base[0, :, 3] = 0.0
    base[1, :, 5] = base[1, :, 2]
    base[2] = 0.0
    tel = new_qr_telemetry()
    Q, info = batched_qr(base.to(device=device, dtype=torch.float32), telemetry=tel, return_info=True)
    flush_qr_telemetry(tel)
    Q = Q.double().cpu()
    return {"caught": [bool(x) for x in info["fallback_mask"].cpu()], "finite": bool(torch.isfinite(Q).all()),
            "reasons": {k: v for k, v in tel["primary_fallback_reasons"].items() if v}}


def training_survival(steps: int = 30, device="cpu", seed: int = 0) -> Dict:
    """Fast-path survival over the QR calls of a short training run of a small MoE model with the subspace tier."""
    from ..models.zoo import load_model
    from ..optim import CentroidSteerOptimizer
    from ..utils import place_model

    torch.manual_seed(seed)
    dev = torch.device(device)
    model = place_model(load_model("triune-nano", vocab_size=256), dev, torch.bfloat16 if dev.type == "cuda" else torch.float32).train()
    opt = CentroidSteerOptimizer(model, lr=1e-3, rank=8, update_gap=5, grad_clip=1.0)
    g = torch.Generator().manual_seed(seed + 1)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, 256, (4, 65), generator=g).to(dev)
        loss = model.forward_loss(ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), force_depth=2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    qr = opt.get_qr_telemetry()
    total = int(qr.get("total_qr_calls", 0))
    fast = int(qr.get("cholesky_fast_path_survivals", 0))
    return {"steps": steps, "qr_calls": total, "fast_path": fast, "survival": fast / total if total else None,
            "primary_reasons": {k: v for k, v in (qr.get("primary_fallback_reasons") or {}).items() if v},
            "first_loss": losses[0], "last_loss": losses[-1]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="residuals and survival of the fast QR path")
    ap.add_argument("--slices", type=int, default=64)
    ap.add_argument("--rows", type=int, default=384)
    ap.add_argument("--rank", type=int, default=32)
    ap.add_argument("--train-steps", type=int, default=0)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    out = {"eval": "qr residuals", "device": a.device, "sweep": sweep(a.slices, a.rows, a.rank, device=a.device),
           "degenerate_inputs": degenerate_cases(device=a.device)}
    if a.train_steps:
        out["training"] = training_survival(a.train_steps, a.device)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
