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


def seed_everything(seed: int, *, deterministic: bool = False) -> None:
    """Seed Python's and PyTorch's generators (every CUDA device included); ``deterministic`` also asks PyTorch for
    deterministic algorithms (``triune/utils/seed.py`` of the reference)."""
    import random

    random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if deterministic:
        torch.use_deterministic_algorithms(True)


def device_diagnostic() -> dict:
    """Interpreter, PyTorch version and the visible GPUs (name, memory, compute capability); changes nothing
    (``triune/utils/device.py`` of the reference)."""
    import sys

    out = {"python": sys.executable, "torch": torch.__version__, "cuda_available": torch.cuda.is_available(), "gpus": []}
    if out["cuda_available"]:
        for i in range(torch.cuda.device_count()):
            props = torch.cuda.get_device_properties(i)
            out["gpus"].append({"name": props.name, "memory_gib": props.total_memory / 1024 ** 3,
                                "capability": torch.cuda.get_device_capability(i), "sm_count": props.multi_processor_count})
    return out
