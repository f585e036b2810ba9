"""Bounded profiling of training steps.

Parity: ``profile_model`` (``triune/profiling.py:15-73``) runs warm-up steps, then a fixed number of profiled Cortex
training steps under ``torch.profiler`` and writes the operator table. Here the table is sorted by device time (the
step is GPU-bound once launches are captured), the step goes through the framework's own loss path
(``forward_loss``: fused head + cross entropy), and ``time_steps`` gives the CUDA-event time per step without a profiler
attached, which is the number to quote.
"""

from __future__ import annotations

from pathlib import Path
from typing import Callable, Dict, Optional

import torch


_NVTX = {"on": None}


def nvtx_enabled() -> bool:
    """NVTX ranges are emitted when ``TRIUNE_NVTX=1`` (read once) and CUDA is present."""
    if _NVTX["on"] is None:
        import os

        _NVTX["on"] = os.environ.get("TRIUNE_NVTX", "0") == "1" and torch.cuda.is_available()
    return _NVTX["on"]


class nvtx_range:
    """``with nvtx_range("forward"):`` marks a phase of the step (forward / backward / data-parallel reduction /
    optimizer) for timeline tools. A no-op unless :func:`nvtx_enabled`; safe inside CUDA-graph capture (ranges are
    host-side markers)."""

    __slots__ = ("name", "live")

    def __init__(self, name: str):
        self.name, self.live = name, False

    def __enter__(self):
        if nvtx_enabled():
            torch.cuda.nvtx.range_push(self.name)
            self.live = True
        return self

    def __exit__(self, *exc):
        if self.live:
            torch.cuda.nvtx.range_pop()
        return False


def time_steps(step_fn: Callable[[], object], steps: int = 10, warmup: int = 3) -> Dict[str, float]:
    """CUDA-event timing of ``steps`` calls after ``warmup`` calls; synchronises on both sides."""
    for _ in range(warmup):
        step_fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step_fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"ms_per_step": ms, "steps": steps, "warmup": warmup}


def profile_model(*, model=None, checkpoint_path="checkpoints_full/latest.pt", preset: str = "triune-base",
                  output_path="profiler_output.txt", batch_size: int = 4, seq_len: int = 256, warmup_steps: int = 5,
                  active_steps: int = 10, row_limit: int = 40, vocab_size: Optional[int] = None) -> str:
    if not torch.cuda.is_available():
        raise RuntimeError("GPU profiling requires CUDA")
    from torch.profiler import ProfilerActivity, profile

    from .utils import place_model

    dev = torch.device("cuda")
    if model is None:
        if Path(checkpoint_path).is_file():
            from .inference import load_checkpoint_model

            model = load_checkpoint_model(str(checkpoint_path), dev, torch.bfloat16)[0]
        else:
            from .models.zoo import load_model

            kw = {"vocab_size": vocab_size} if vocab_size else {}
            model = place_model(load_model(preset, **kw), dev, torch.bfloat16)
    model.train()
    V = int(model.vocab_size)

    def step():
        model.zero_grad(set_to_none=True)
        x = torch.randint(0, V, (batch_size, seq_len), device=dev)
        y = torch.randint(0, V, (batch_size, seq_len), device=dev)
        loss = model.forward_loss(x, y, force_depth=2) if hasattr(model, "forward_loss") else \
            torch.nn.functional.cross_entropy(model(x, force_depth=2)[0].reshape(-1, V).float(), y.reshape(-1))
        (loss[0] if isinstance(loss, tuple) else loss).backward()

    timing = time_steps(step, steps=active_steps, warmup=warmup_steps)
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=False) as prof:
        for _ in range(active_steps):
            step()
        torch.cuda.synchronize()
    table = prof.key_averages().table(sort_by="cuda_time_total", row_limit=row_limit)
    text = f"# {timing['ms_per_step']:.3f} ms/step over {active_steps} steps (CUDA events, no profiler attached)\n" + table
    Path(output_path).write_text(text, encoding="utf-8")
    return text
