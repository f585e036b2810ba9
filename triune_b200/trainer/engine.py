"""Training step engine with the three depth modes of the reference.

Parity: ``TrainingEngine`` (``triune/trainer/engine.py:18-511``). ``step_once``: LR schedule -> tier LRs ->
``grad_accum`` micro-batches in one of
  * ``cortex``  full-depth next-token loss,
  * ``joint``   weighted CE at the three exits ((0.22,0.23,0.55) while Cortex is worse than Limbic, else
                (0.25,0.30,0.45)) + 0.2 * (KL_R + KL_L) toward the detached Cortex distribution + 0.5 * router
                CE + 1e-3 * z-loss + 0.3 * balance,
  * ``dynamic`` router labels from a no-grad all-exits pass (batch-centred exit losses + depth cost + bias
                toward the target usage), exploration schedule, 0.8/0.2 mix with a Cortex anchor, plus
                0.5 * router CE + z-loss + balance on the route logits of the anchor pass (the reference's
                dynamic branch, ``triune/trainer/engine.py:342-411``),
then clip -> optimizer step -> MoE selection-bias update. The duck-typed ``trainer`` protocol is the
reference's (``.model .optimizer .config .device .next_batch() .lr_schedule .set_optimizer_lr ...``).

The per-exit losses go through the fused head-GEMM + cross-entropy op, so no ``[tokens, vocab]`` logits are
materialised in ``cortex`` mode; the KL terms of ``joint`` mode need logits and compute them per row chunk.
"""

from __future__ import annotations

import math
import time
from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F

from ..models.moe import MoE_FFN
from ..profiling import nvtx_range


def _moe_layers(model):
    return [m for m in model.modules() if isinstance(m, MoE_FFN)]


class TrainingEngine:
    def __init__(self, trainer):
        self.trainer = trainer
        self.model = trainer.model
        self.optimizer = trainer.optimizer
        self.config = trainer.config
        self.device = trainer.device
        self.step = 0
        self.best_eval_loss = float("inf")
        tdd = self.config.get("target_depth_dist", (0.34, 0.33, 0.33))
        self.usage_ema = torch.tensor(tdd, dtype=torch.float32)
        self._moe = _moe_layers(self.model)
        self.streaming_engine = getattr(trainer, "streaming_engine", None)

    def sync_streaming_engine(self) -> None:
        """Hand the optimizer and the clip norm to a layer-streaming engine attached to the model."""
        eng = getattr(self.model, "_streaming_engine", None) or self.streaming_engine
        if eng is not None and self.optimizer is not None:
            eng.set_optimizer(self.optimizer)
            eng.cfg.grad_clip = float(self.config.get("grad_clip", 1.0))

    # ------------------------------------------------------------------ helpers
    def _exploration(self) -> float:
        """Probability of a random depth in the dynamic mode. ``exploration`` is either the reference's schedule name
        (``"linear"`` / ``"cosine"`` / ``"none"``: from 1 down to 0 over ``exploration_steps``,
        ``triune/trainer/engine.py:49-58``) or a number: the starting rate of a schedule named by ``exploration_schedule``."""
        mode = self.config.get("exploration", "linear")
        steps = int(self.config.get("exploration_steps", 5000))
        if isinstance(mode, str):
            if mode == "none" or steps <= 0:
                return 0.0
            base, sched = 1.0, mode
        else:
            base, sched = float(mode), str(self.config.get("exploration_schedule", "linear"))
            steps = max(1, steps)
        if self.step >= steps:
            return 0.0
        frac = self.step / steps
        if sched == "cosine":
            return base * 0.5 * (1.0 + math.cos(math.pi * frac))
        return base * (1.0 - frac)

    def _joint_weights(self, losses):
        lr_, ll, lc = (float(x.detach()) for x in losses)
        return (0.22, 0.23, 0.55) if lc > ll else (0.25, 0.30, 0.45)

    @torch.no_grad()
    def _router_labels(self, x, y):
        """argmin over exits of (batch-centred per-sequence loss + depth cost + usage bias)."""
        was = self.model.training
        self.model.eval()
        r, l, c, _ = self.model.forward_all_exits(x, update_stats=False)
        self.model.train(was)
        per = []
        for lg in (r, l, c):
            ce = F.cross_entropy(lg.float().reshape(-1, lg.shape[-1]), y.reshape(-1), reduction="none")
            per.append(ce.view(y.shape).mean(dim=1))
        L = torch.stack(per, dim=1)
        L = L - L.mean(dim=0, keepdim=True)
        cost = torch.tensor([0.0, 0.05, 0.10], device=L.device)
        target = torch.as_tensor(self.config.get("target_depth_dist", (0.34, 0.33, 0.33)), device=L.device)
        bias = float(self.config.get("bias_strength", 4.0)) * (self.usage_ema.to(L.device) - target) * 0.1
        return (L + cost + bias).argmin(dim=1)

    def _micro_loss(self, x, y, n_valid: Optional[int]):
        mode = self.config.get("depth_mode", "cortex")
        model = self.model
        stats: Dict[str, Any] = {}
        if mode == "cortex":
            loss = model.forward_loss(x, y, force_depth=2, n_valid=n_valid)
            stats["lm_loss"] = loss.detach()
            return loss, stats
        if mode == "joint":
            losses, route_logits = model.exit_losses(x, y, n_valid=n_valid)
            w = self._joint_weights(losses)
            loss = sum(wi * li for wi, li in zip(w, losses))
            coef = float(self.config.get("exit_distill_coef", 0.2))
            if coef > 0:
                with torch.no_grad():
                    _, _, xc, _ = model.forward_hidden_all_exits(x, update_stats=False)
                    pc = F.softmax(model._head(xc, 2).float(), dim=-1)
                # KL terms on a row subsample bound the logits memory
                xr, xl, _, _ = model.forward_hidden_all_exits(x, update_stats=False)
                rows = slice(0, min(x.shape[0], 2))
                for d, h in ((0, xr), (1, xl)):
                    lg = model._head(h[rows], d).float()
                    loss = loss + coef * F.kl_div(F.log_softmax(lg, -1).flatten(0, 1), pc[rows].flatten(0, 1),
                                                  reduction="batchmean")
            labels = torch.stack([l.detach() for l in losses]).argmin().expand(x.shape[0])
            rl = route_logits.float()
            loss = loss + 0.5 * F.cross_entropy(rl, labels) + float(self.config.get("z_loss_coef", 1e-3)) * (
                torch.logsumexp(rl, dim=-1) ** 2).mean()
            if model.last_balance_loss is not None:
                loss = loss + float(self.config.get("balance_coef", 0.3)) * model.last_balance_loss
            stats.update(reflex=losses[0].detach(), limbic=losses[1].detach(), lm_loss=losses[2].detach())
            return loss, stats
        # dynamic
        labels = self._router_labels(x, y)
        eps = self._exploration()
        if eps > 0:
            rnd = torch.rand(labels.shape, device=labels.device) < eps
            labels = torch.where(rnd, torch.randint_like(labels, 0, 3), labels)
        total = x.new_zeros((), dtype=torch.float32)
        for d in (0, 1, 2):
            idx = (labels == d).nonzero(as_tuple=True)[0]
            if idx.numel() == 0:
                continue
            ld = model.forward_loss(x[idx], y[idx], force_depth=d)
            total = total + ld * (idx.numel() / x.shape[0])
        # The anchor pass also evaluates the depth router with its graph attached: the router (and the prefix layers
        # under it) learn the exit labels here; at inference it is this router that picks the exit.
        anchor, route_logits, balance = model.forward_loss(x, y, force_depth=2, n_valid=n_valid, return_route=True)
        loss = 0.8 * total + 0.2 * anchor
        rl = route_logits.float()
        if balance is None:
            target = torch.as_tensor(self.config.get("target_depth_dist", (0.34, 0.33, 0.33)), device=rl.device,
                                     dtype=torch.float32)
            balance = (torch.softmax(rl, dim=-1).mean(dim=0) - target).pow(2).mean()
        router_loss = F.cross_entropy(rl, labels)
        z_loss = (torch.logsumexp(rl, dim=-1) ** 2).mean()
        loss = (loss + 0.5 * router_loss + float(self.config.get("z_loss_coef", 1e-3)) * z_loss
                + float(self.config.get("balance_coef", 0.3)) * balance)
        stats.update(router_loss=router_loss.detach(), z_loss=z_loss.detach())
        with torch.no_grad():
            use = torch.bincount(labels, minlength=3).float().cpu() / max(1, labels.numel())
            d = float(self.config.get("usage_ema_decay", 0.98))
            self.usage_ema = self.usage_ema * d + use * (1 - d)
        stats["lm_loss"] = anchor.detach()
        return loss, stats

    # ------------------------------------------------------------------ one optimizer step
    def step_once(self) -> Dict[str, Any]:
        tr = self.trainer
        cfg = self.config
        lr = tr.lr_schedule(cfg, self.step) if hasattr(tr, "lr_schedule") else cfg.get("lr", 1e-4)
        if hasattr(tr, "set_optimizer_lr"):
            tr.set_optimizer_lr(self.optimizer, lr)
        for m in self._moe:
            m._global_step.fill_(self.step)
        accum = int(getattr(tr, "grad_accum", cfg.get("grad_accum_steps", 1)))
        self.model.train()
        tot = None
        stats: Dict[str, Any] = {}
        tokens = 0
        for _ in range(accum):
            batch = tr.next_batch()
            x, y = batch[0], batch[1]
            n_valid = batch[2] if len(batch) > 2 else None
            with nvtx_range("forward"):
                with tr.model_autocast() if hasattr(tr, "model_autocast") else torch.autocast("cpu", enabled=False):
                    loss, st = self._micro_loss(x, y, n_valid)
            with nvtx_range("backward"):
                (loss / accum).backward()
            tot = loss.detach() if tot is None else tot + loss.detach()
            stats.update(st)
            tokens += x.numel()
        if self.streaming_engine is not None:
            self.streaming_engine.step_streaming_optimizer(self.optimizer, float(cfg.get("grad_clip", 1.0)))
        else:
            clip = cfg.get("grad_clip", 1.0)
            if hasattr(self.optimizer, "arena"):
                self.optimizer.grad_clip = clip
            elif clip:
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), clip)
            with nvtx_range("optimizer"):
                self.optimizer.step()
                self.optimizer.zero_grad(set_to_none=True)
        for m in self._moe:
            m.step_bias()
        self.step += 1
        out = {"step": self.step, "loss": tot / accum, "lr": lr, "tokens": tokens}
        out.update(stats)
        return out

    # ------------------------------------------------------------------ loop
    def train(self, total_steps: Optional[int] = None):
        cfg = self.config
        total = int(total_steps if total_steps is not None else cfg.get("total_steps", 1000))
        log_every, eval_every, save_every = (int(cfg.get(k, d)) for k, d in
                                             (("log_every", 10), ("eval_every", 200), ("save_every", 1000)))
        tr = self.trainer
        t0 = time.time()
        last = None
        try:
            while self.step < total:
                last = self.step_once()
                if self.step % log_every == 0:
                    loss = float(last["loss"])
                    tr.logger.log({"step": self.step, "loss": loss, "lr": last["lr"],
                                   "elapsed_s": time.time() - t0}) if getattr(tr, "logger", None) else None
                if eval_every and self.step % eval_every == 0 and hasattr(tr, "run_eval"):
                    ev = tr.run_eval()
                    if ev is not None and ev < self.best_eval_loss:
                        self.best_eval_loss = ev
                        if hasattr(tr, "save_best"):
                            tr.save_best()
                if save_every and self.step % save_every == 0 and hasattr(tr, "save_latest"):
                    tr.save_latest()
        except BaseException:
            if hasattr(tr, "save_latest"):
                try:
                    tr.save_latest()
                except Exception:
                    pass
            raise
        return last
