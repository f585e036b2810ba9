"""Data pipeline: token-stream datasets, cycling loader, device prefetcher, tokenizers."""

from .dataloader import AsyncDevicePrefetcher, CyclingDataLoader, SyntheticTokenSource
from .dataset import TokenStreamDataset, build_dataloader
from .dynamic_tokenizer import DynamicTokenizer, DynamicTokenizerOutput
from .tokenizer import SPECIAL_TOKENS, PurePythonBPETokenizer, TriuneTokenizer, build_tokenizer, load_tokenizer, train_bpe

__all__ = ["AsyncDevicePrefetcher", "CyclingDataLoader", "SyntheticTokenSource", "TokenStreamDataset", "build_dataloader",
           "DynamicTokenizer", "DynamicTokenizerOutput", "SPECIAL_TOKENS", "PurePythonBPETokenizer", "TriuneTokenizer",
           "build_tokenizer", "load_tokenizer", "train_bpe"]
