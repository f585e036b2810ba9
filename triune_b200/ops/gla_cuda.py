"""Dispatch to the sm_100a chunked GLA kernels (forward, backward, decode step)."""

from __future__ import annotations

import torch

from .. import _ext


def supported(q, k, v, g, initial_state) -> bool:
    """True when the CUDA kernels cover this call (bf16, head_dim 64, T a multiple of 64)."""
    if not _ext.use_kernels(q, k, v, g):
        return False
    if not hasattr(_ext.ext(), "gla_fwd"):
        return False
    B, T, H, D = q.shape
    return (
        q.dtype == torch.bfloat16
        and D == 64
        and v.shape[-1] == 64
        and T % 64 == 0
        and T >= 64
    )


def gla_chunk(q, k, v, g, initial_state, scale, gate_logits):
    raise NotImplementedError
