"""Small shared helpers."""

from __future__ import annotations

import torch


def place_model(model: torch.nn.Module, device, dtype=None) -> torch.nn.Module:
    """Move a model to ``device`` and cast its PARAMETERS to ``dtype``; buffers keep their dtype.

    Routing statistics (expert selection bias, depth-router bias, centroids, step counters) are buffers that
    receive increments of 1e-3 and smaller, so they must stay fp32 when the weights run in bf16.
    """
    model.to(device)
    if dtype is not None:
        seen = set()
        for p in model.parameters():
            if id(p) in seen:
                continue
            seen.add(id(p))
            if p.is_floating_point():
                p.data = p.data.to(dtype)
    return model


def count_parameters(model: torch.nn.Module) -> int:
    seen, n = set(), 0
    for p in model.parameters():
        if id(p) not in seen:
            seen.add(id(p))
            n += p.numel()
    return n
