"""Continuation training that repairs a checkpoint whose deep exit is worse than its shallow ones.

Under dynamic depth routing a run can starve the deepest exit: most tokens leave early, the late layers see little
gradient, and perplexity stops improving (or gets worse) with depth. The repair has three stages, each optional:

1. **deepen**: every token goes to full depth (``force_depth=2``); the whole model trains on the final head alone with a
   warm-up + cosine schedule, so the late layers catch up;
2. **align**: the trunk is frozen and only the two early exit norms + heads train, on half cross entropy and half KL
   towards the (detached) full-depth distribution, with a learning rate per exit;
3. **joint**: a short pass on the weighted sum of the three exit losses at a small learning rate, so that the exits
   stay consistent with a trunk that moved in stage 1.

Before and after, every exit is evaluated on held-out blocks; the report says whether loss is now monotone in depth.
Same purpose as the reference's ``scripts/rescue_checkpoint.py:117-470`` (stages 1 / 1.5 / 2 there), built on this
package's fused head + cross-entropy op so no ``[N, V]`` logits are kept for the full-depth stages.
"""

from __future__ import annotations

import math
import time
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn.functional as F

DEPTH_NAMES = ("reflex", "limbic", "cortex")


def pack_blocks(docs: Iterable[Sequence[int]], seq_len: int, sep_id: Optional[int] = None, max_blocks: Optional[int] = None) -> torch.Tensor:
    """Concatenate tokenised documents (a separator after each when given) and cut ``[n, seq_len + 1]`` blocks; the
    ragged tail is dropped."""
    stride, stream, blocks = seq_len + 1, [], []
    for ids in docs:
        stream.extend(int(t) for t in ids)
        if sep_id is not None:
            stream.append(int(sep_id))
        while len(stream) >= stride:
            blocks.append(stream[:stride])
            stream = stream[stride:]
            if max_blocks is not None and len(blocks) >= max_blocks:
                return torch.tensor(blocks, dtype=torch.long)
    return torch.tensor(blocks, dtype=torch.long).reshape(-1, stride)


def cosine_lr(step: int, total: int, warmup: int, lr_max: float, lr_min: float) -> float:
    if step < warmup:
        return lr_max * (step + 1) / max(1, warmup)
    t = min(1.0, max(0.0, (step - warmup) / max(1, total - warmup)))
    return lr_min + 0.5 * (lr_max - lr_min) * (1.0 + math.cos(math.pi * t))


@torch.no_grad()
def evaluate_all_depths(model, blocks: torch.Tensor, batch_size: int = 8) -> Dict[str, Any]:
    """Mean next-token loss and perplexity at each exit over ``blocks`` ``[n, T + 1]``; ``monotone`` is true when loss
    does not increase with depth."""
    dev = next(model.parameters()).device
    was = model.training
    model.eval()
    tot = [0.0, 0.0, 0.0]
    n = 0
    try:
        for b in blocks.split(batch_size):
            b = b.to(dev)
            losses, _ = model.exit_losses(b[:, :-1], b[:, 1:], update_stats=False)
            for d in range(3):
                tot[d] += float(losses[d]) * b.shape[0]
            n += b.shape[0]
    finally:
        model.train(was)
    out: Dict[str, Any] = {}
    for d, name in enumerate(DEPTH_NAMES):
        loss = tot[d] / max(1, n)
        out[name] = {"loss": loss, "ppl": math.exp(min(loss, 50.0))}
    out["monotone"] = out["reflex"]["loss"] >= out["limbic"]["loss"] >= out["cortex"]["loss"]
    return out


class _Batches:
    """Endless shuffled batches over a block tensor, deterministic for a seed."""

    def __init__(self, blocks: torch.Tensor, batch_size: int, device, seed: int = 0):
        self.blocks, self.bs, self.dev = blocks, batch_size, device
        self.gen = torch.Generator().manual_seed(seed)
        self.perm, self.at = torch.randperm(len(blocks), generator=self.gen), 0

    def next(self):
        if self.at + self.bs > len(self.perm):
            self.perm, self.at = torch.randperm(len(self.blocks), generator=self.gen), 0
        idx = self.perm[self.at : self.at + self.bs]
        self.at += self.bs
        b = self.blocks[idx].to(self.dev)
        return b[:, :-1], b[:, 1:]


def _exit_parameters(model):
    groups = []
    for idx in (model.reflex_exit_layer, model.limbic_exit_layer):
        blk = model.layers[idx]
        groups.append(list(blk.exit_norm.parameters()) + list(blk.exit_head.parameters()))
    return groups


def rescue_checkpoint(model, train_blocks: torch.Tensor, val_blocks: torch.Tensor, deepen_steps: int = 200, align_steps: int = 50,
                      joint_steps: int = 50, lr: float = 1e-4, batch_size: int = 8, accum: int = 1, grad_clip: float = 2.0,
                      align_lrs: Sequence[float] = (3.8e-4, 8.8e-4), joint_weights: Sequence[float] = (0.2, 0.3, 0.5),
                      eval_every: int = 0, seed: int = 0, log: Optional[Callable[[str], None]] = None) -> Dict[str, Any]:
    """Run the three stages on ``model`` in place and return the report (metrics before / after every stage)."""
    from ..optim import build_optimizer

    say = log or (lambda m: None)
    dev = next(model.parameters()).device
    if len(train_blocks) < batch_size:
        raise ValueError(f"need at least {batch_size} training blocks, got {len(train_blocks)}")
    data = _Batches(train_blocks, batch_size, dev, seed)
    report: Dict[str, Any] = {"before": evaluate_all_depths(model, val_blocks, batch_size), "stages": {}}
    say(f"before: {report['before']}")
    t_start, tokens = time.perf_counter(), 0

    def full_model_stage(name: str, steps: int, lr_max: float, loss_fn) -> None:
        nonlocal tokens
        if steps <= 0:
            return
        opt = build_optimizer(model, {"lr": lr_max, "grad_clip": 0.0})
        model.train()
        last = 0.0
        for step in range(steps):
            cur = cosine_lr(step, steps, max(1, steps // 20), lr_max, lr_max * 0.05)
            opt.set_lr(cur) if hasattr(opt, "set_lr") else [g.__setitem__("lr", cur) for g in opt.param_groups]
            opt.zero_grad()
            last = 0.0
            for _ in range(accum):
                x, y = data.next()
                loss = loss_fn(x, y) / accum
                loss.backward()
                last += float(loss.detach())
                tokens += y.numel()
            if grad_clip > 0:
                torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.grad is not None], grad_clip)
            opt.step()
            if eval_every and (step + 1) % eval_every == 0:
                say(f"{name} {step + 1}/{steps}: train {last:.4f} val {evaluate_all_depths(model, val_blocks, batch_size)}")
        report["stages"][name] = {"steps": steps, "final_train_loss": last, "val": evaluate_all_depths(model, val_blocks, batch_size)}
        say(f"{name}: {report['stages'][name]['val']}")

    # stage 1: every token to full depth
    full_model_stage("deepen", deepen_steps, lr, lambda x, y: model.forward_loss(x, y, force_depth=2))

    # stage 2: frozen trunk, the early exit heads learn from the labels and from the full-depth distribution
    if align_steps > 0:
        flags = [(p, p.requires_grad) for p in model.parameters()]
        groups = _exit_parameters(model)
        try:
            for p in model.parameters():
                p.requires_grad_(False)
            for g in groups:
                for p in g:
                    p.requires_grad_(True)
            head_opt = torch.optim.AdamW([{"params": g, "lr": l, "weight_decay": 0.01} for g, l in zip(groups, align_lrs)])
            model.eval()
            last = 0.0
            for step in range(align_steps):
                head_opt.zero_grad()
                last = 0.0
                for _ in range(accum):
                    x, y = data.next()
                    with torch.no_grad():
                        xr, xl, xc, _ = model.forward_hidden_all_exits(x, update_stats=False)
                        pc = F.softmax(model._head(xc, 2).float().flatten(0, 1), dim=-1)
                    loss = 0.0
                    for d, h in ((0, xr), (1, xl)):
                        norm, head = model._head_modules(d)
                        lg = F.linear(norm(h.detach()).float(), head.weight.float(), None if head.bias is None else head.bias.float())
                        lg = lg.flatten(0, 1)
                        loss = loss + 0.5 * F.cross_entropy(lg, y.reshape(-1)) + 0.5 * F.kl_div(F.log_softmax(lg, -1), pc, reduction="batchmean")
                    (loss / accum).backward()
                    last += float(loss.detach()) / accum
                    tokens += y.numel()
                head_opt.step()
        finally:
            for p, f in flags:
                p.requires_grad_(f)
        report["stages"]["align"] = {"steps": align_steps, "final_train_loss": last, "val": evaluate_all_depths(model, val_blocks, batch_size)}
        say(f"align: {report['stages']['align']['val']}")

    # stage 3: all exits together, gently
    def joint_loss(x, y):
        losses, _ = model.exit_losses(x, y, update_stats=False)
        return sum(w * l for w, l in zip(joint_weights, losses))

    full_model_stage("joint", joint_steps, lr * 0.25, joint_loss)

    report["after"] = evaluate_all_depths(model, val_blocks, batch_size)
    report["seconds"] = time.perf_counter() - t_start
    report["tokens_trained"] = tokens
    report["improved"] = {n: report["before"][n]["loss"] - report["after"][n]["loss"] for n in DEPTH_NAMES}
    report["config_update"] = {"depth_mode": "joint", "exit_distill_coef": 0.25,
                               "rescue_stages": {"deepen": deepen_steps, "align": align_steps, "joint": joint_steps}}
    return report


def load_documents(path: str, tokenizer, limit: Optional[int] = None) -> List[List[int]]:
    """Token ids per document from a ``.jsonl`` file (``text`` field) or a plain text file (one document per blank-line
    separated paragraph)."""
    import json

    docs: List[List[int]] = []
    with open(path, encoding="utf-8") as f:
        if path.endswith(".jsonl"):
            for line in f:
                line = line.strip()
                if line:
                    docs.append(tokenizer.encode(str(json.loads(line).get("text", ""))))
                    if limit and len(docs) >= limit:
                        break
        else:
            for para in f.read().split("\n\n"):
                if para.strip():
                    docs.append(tokenizer.encode(para.strip()))
                    if limit and len(docs) >= limit:
                        break
    return docs
