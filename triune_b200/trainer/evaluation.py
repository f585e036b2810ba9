"""Evaluation helpers (reference: ``triune/trainer/evaluation.py:11-84``)."""

from __future__ import annotations

import inspect
from typing import Optional

import torch
import torch.nn.functional as F


def forward_causal_lm(model, input_ids):
    """Logits of any causal LM: Triune models (``force_depth``), HF models (``.logits``) or plain modules."""
    params = inspect.signature(model.forward).parameters
    if "force_depth" in params:
        out = model(input_ids, force_depth=2)
    else:
        out = model(input_ids)
    if hasattr(out, "logits"):
        return out.logits
    return out[0] if isinstance(out, (tuple, list)) else out


@torch.no_grad()
def run_eval(model, loader, device, max_batches: int = 5) -> float:
    was = model.training
    model.eval()
    tot, n = 0.0, 0
    for i, batch in enumerate(loader):
        if i >= max_batches:
            break
        x, y = batch[0].to(device), batch[1].to(device)
        if hasattr(model, "forward_loss"):
            loss = model.forward_loss(x, y, force_depth=2)
        else:
            lg = forward_causal_lm(model, x)
            loss = F.cross_entropy(lg.float().reshape(-1, lg.shape[-1]), y.reshape(-1))
        tot += float(loss)
        n += 1
    model.train(was)
    return tot / max(1, n)


@torch.no_grad()
def run_sample(model, prompt_ids: Optional[torch.Tensor], device, max_new_tokens: int = 16):
    was = model.training
    model.eval()
    ids = prompt_ids.to(device) if prompt_ids is not None else torch.zeros(1, 1, dtype=torch.long, device=device)
    for _ in range(max_new_tokens):
        lg = forward_causal_lm(model, ids)
        ids = torch.cat((ids, lg[:, -1].argmax(-1, keepdim=True)), dim=1)
    model.train(was)
    return ids
