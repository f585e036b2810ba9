"""Block-wise 8-bit storage of the Adam moments (the optional 8-bit tier of ``CentroidSteerOptimizer``).

The reference delegates this tier to ``bitsandbytes.optim.AdamW8bit`` when that package is present
(``triune/optim/centroid.py:10-16``); this is a self-contained equivalent. Both moments are kept as one byte per
element plus one fp32 scale per block of 256 elements:

* first moment: signed, ``q = round(127 * sign(x) * sqrt(|x| / absmax))``. The square-root companding spends the
  codes near zero, where most of a momentum vector lives, instead of on the few large entries;
* second moment: unsigned, ``q = round(255 * (x / max)^(1/4))``. The fourth root spreads eight or so decades of a
  non-negative quantity over the 256 codes, and what the update reads is ``sqrt(v)``, whose relative error is half of
  that of ``v``.

Decoded values are exact fp32 for the update arithmetic; only the storage between steps is quantised
(8 bytes per parameter become 2 + 8/256).
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch

BLOCK = 256


class BlockwiseMoments:
    def __init__(self, numel: int, device):
        self.numel = int(numel)
        self.blocks = (self.numel + BLOCK - 1) // BLOCK
        self.m_q = torch.zeros(self.blocks * BLOCK, device=device, dtype=torch.int8)
        self.v_q = torch.zeros(self.blocks * BLOCK, device=device, dtype=torch.uint8)
        self.m_scale = torch.zeros(self.blocks, device=device, dtype=torch.float32)
        self.v_scale = torch.zeros(self.blocks, device=device, dtype=torch.float32)

    def _span(self, b: int, e: int) -> Tuple[int, int]:
        return b // BLOCK, (e + BLOCK - 1) // BLOCK

    def load(self, b: int, e: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """fp32 copies of elements [b, e) of both moments."""
        b0, b1 = self._span(b, e)
        mq = self.m_q[b0 * BLOCK : b1 * BLOCK].view(-1, BLOCK).float() / 127.0
        m = (mq.abs() * mq) * self.m_scale[b0:b1, None]                  # sign(q) q^2 * absmax
        vq = self.v_q[b0 * BLOCK : b1 * BLOCK].view(-1, BLOCK).float() / 255.0
        v = (vq * vq) * (vq * vq) * self.v_scale[b0:b1, None]
        off = b - b0 * BLOCK
        return m.reshape(-1)[off : off + (e - b)].clone(), v.reshape(-1)[off : off + (e - b)].clone()

    def store(self, b: int, e: int, m: torch.Tensor, v: torch.Tensor) -> None:
        """Quantise and keep elements [b, e). Blocks that are only partly covered are re-encoded as a whole (their other
        elements are decoded first), so neighbouring ranges can be updated independently."""
        b0, b1 = self._span(b, e)
        full_m, full_v = self.load(b0 * BLOCK, b1 * BLOCK)
        off = b - b0 * BLOCK
        full_m[off : off + (e - b)] = m
        full_v[off : off + (e - b)] = v
        fm, fv = full_m.view(-1, BLOCK), full_v.view(-1, BLOCK).clamp_min(0.0)
        ms = fm.abs().amax(dim=1)
        vs = fv.amax(dim=1)
        self.m_scale[b0:b1] = ms
        self.v_scale[b0:b1] = vs
        mn = fm / ms.clamp_min(1e-30)[:, None]
        self.m_q[b0 * BLOCK : b1 * BLOCK] = (mn.sign() * mn.abs().sqrt() * 127.0).round().clamp(-127, 127).to(torch.int8).reshape(-1)
        vn = fv / vs.clamp_min(1e-30)[:, None]
        # a non-zero second moment never decodes to zero (that would blow the update up): floor code 1
        code = (vn.sqrt().sqrt() * 255.0).round().clamp(0, 255)
        code = torch.where((fv > 0) & (code < 1), torch.ones_like(code), code)
        self.v_q[b0 * BLOCK : b1 * BLOCK] = code.to(torch.uint8).reshape(-1)

    def nbytes(self) -> int:
        return self.m_q.numel() + self.v_q.numel() + 8 * self.blocks

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {"m_q": self.m_q, "v_q": self.v_q, "m_scale": self.m_scale, "v_scale": self.v_scale, "numel": self.numel}

    def load_state_dict(self, sd) -> None:
        if int(sd["numel"]) != self.numel:
            raise ValueError("8-bit moment state has a different size")
        for k in ("m_q", "v_q", "m_scale", "v_scale"):
            getattr(self, k).copy_(sd[k].to(getattr(self, k).device))


class AdamW8bit(torch.optim.Optimizer):
    """AdamW whose two moments live in :class:`BlockwiseMoments` (2 bytes per parameter plus one scale per 256 elements).

    A stand-alone optimizer with the constructor of ``torch.optim.AdamW`` (the reference re-exports
    ``bitsandbytes.optim.AdamW8bit`` under this name when that package is installed, ``triune/optim/__init__.py``). The
    update arithmetic is fp32 on decoded moments; decoupled weight decay; bias correction per parameter group step."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("invalid AdamW8bit hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["moments"] = BlockwiseMoments(p.numel(), p.device)
                st["step"] += 1
                t = st["step"]
                g = p.grad.detach().float().reshape(-1)
                m, v = st["moments"].load(0, p.numel())
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                st["moments"].store(0, p.numel(), m, v)
                denom = (v / (1 - b2 ** t)).sqrt_().add_(group["eps"])
                upd = (m / (1 - b1 ** t)).div_(denom).view_as(p)
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(upd.to(p.dtype), alpha=-group["lr"])
        return loss

    def state_bytes(self) -> int:
        return sum(s["moments"].m_q.numel() + s["moments"].v_q.numel() + 4 * (s["moments"].m_scale.numel() + s["moments"].v_scale.numel())
                   for s in self.state.values() if "moments" in s)
