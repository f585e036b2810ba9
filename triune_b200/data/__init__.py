"""Data pipeline: token-stream datasets, cycling loader, device prefetcher, tokenizers."""

from .dataloader import AsyncDevicePrefetcher, CyclingDataLoader, SyntheticTokenSource

__all__ = ["AsyncDevicePrefetcher", "CyclingDataLoader", "SyntheticTokenSource"]
