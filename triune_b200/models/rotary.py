"""Rotary position tables with on-demand growth (reference: triune/model/rotary.py:13-63)."""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops


class RotaryEmbedding(nn.Module):
    """Caches cos/sin [max_len, head_dim] (half-split layout); the cache doubles when a longer range is asked."""

    def __init__(self, head_dim: Optional[int] = None, max_seq_len: int = 8192, base: float = 10000.0, dim: Optional[int] = None):
        super().__init__()
        head_dim = head_dim if head_dim is not None else dim  # ``dim`` is the reference's name for this argument
        if head_dim is None:
            raise TypeError("RotaryEmbedding needs the head dimension")
        self.head_dim = head_dim
        self.base = base
        self.max_seq_len = max_seq_len
        self._cos = None
        self._sin = None

    @property
    def cos_cached(self) -> torch.Tensor:
        """The cosine table built so far (built for ``max_seq_len`` on first use); the reference's attribute name."""
        if self._cos is None:
            self._build(self.max_seq_len, "cpu")
        return self._cos

    @property
    def sin_cached(self) -> torch.Tensor:
        if self._sin is None:
            self._build(self.max_seq_len, "cpu")
        return self._sin

    def _build(self, length: int, device):
        cos, sin = ops.rope_tables(length, self.head_dim, self.base, 0, device)
        self._cos, self._sin = cos, sin

    def forward(self, seq_len: int, device, offset=0):
        if torch.is_tensor(offset):
            # position lives on the device (CUDA-graph decoding): gather rows; the caller sized the table beforehand
            if self._cos is None or self._cos.device != torch.device(device):
                self._build(max(self.max_seq_len, 1), device)
            pos = offset.reshape(-1)[:1].long() + torch.arange(seq_len, device=offset.device)
            return self._cos.index_select(0, pos), self._sin.index_select(0, pos)
        need = offset + seq_len
        if self._cos is None or self._cos.device != torch.device(device) or self._cos.shape[0] < need:
            length = max(self.max_seq_len, 1)
            while length < need:
                length *= 2
            self._build(length, device)
        return self._cos[offset:need], self._sin[offset:need]
