"""Batch sources and host->device prefetch.

Parity: ``CyclingDataLoader`` / ``AsyncDevicePrefetcher`` (``triune/data/dataloader.py:10-95``): infinite
iteration over a loader and a side-stream copy of the NEXT batch from pinned host memory while the current
step computes. ``SyntheticTokenSource`` produces uniform-random token ids from a seed (benchmarks, tests).
"""

from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch


class CyclingDataLoader:
    def __init__(self, loader):
        self.loader = loader
        self._it = iter(loader)

    def __iter__(self):
        return self

    def __next__(self):
        try:
            return next(self._it)
        except StopIteration:
            self._it = iter(self.loader)
            return next(self._it)

    next = __next__


class SyntheticTokenSource:
    """Endless (input, next-token label) batches of uniform-random ids; pinned when CUDA is present."""

    def __init__(self, vocab_size: int, batch_size: int, seq_len: int, seed: int = 0, pin: Optional[bool] = None,
                 pool: int = 8):
        g = torch.Generator().manual_seed(seed)
        self.pin = torch.cuda.is_available() if pin is None else pin
        self.pool = []
        for _ in range(pool):
            ids = torch.randint(0, vocab_size, (batch_size, seq_len + 1), generator=g, dtype=torch.int64)
            x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
            if self.pin:
                x, y = x.pin_memory(), y.pin_memory()
            self.pool.append((x, y))
        self.i = 0

    def __iter__(self):
        return self

    def __next__(self) -> Tuple[torch.Tensor, torch.Tensor]:
        b = self.pool[self.i % len(self.pool)]
        self.i += 1
        return b


class AsyncDevicePrefetcher:
    """Copies batch i+1 to the device on a side stream while batch i is being consumed."""

    def __init__(self, source: Iterator, device: torch.device):
        self.source = iter(source)
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.h2d_bytes = 0
        self._next = None
        self._preload()

    def _preload(self):
        try:
            batch = next(self.source)
        except StopIteration:
            self._next = None
            return
        if not self.cuda:
            self._next = tuple(t.to(self.device) for t in batch)
            return
        with torch.cuda.stream(self.stream):
            self._next = tuple(t.to(self.device, non_blocking=True) for t in batch)
        self._last_bytes = sum(t.numel() * t.element_size() for t in batch)

    def __iter__(self):
        return self

    def __next__(self):
        if self._next is None:
            raise StopIteration
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
            for t in self._next:
                t.record_stream(torch.cuda.current_stream(self.device))
            self.h2d_bytes += self._last_bytes
        out = self._next
        self._preload()
        return out

    next_batch = next = __next__
