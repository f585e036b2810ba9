"""Token-stream dataset: text -> packed ``seq_len + 1`` windows -> ``(input, target)`` pairs.

Parity (``triune/data/dataset.py:14-186``): sources are a Hugging Face streaming dataset (default FineWeb-Edu
sample-10BT) or a local ``.jsonl`` / ``.json`` / ``.parquet`` / text file; documents are joined with the separator id,
cut into windows whose start is moved back (at most 16 tokens) to a word boundary and padded with 0, shuffled in a
buffer, sharded round-robin over DataLoader workers, retried three times with exponential back-off; the hold-out split
is the first ``eval_batches * batch_size * seq_len`` tokens and training skips them.

Differences: local files are read directly (json / pyarrow / plain text) so no ``datasets`` install or network is
needed for them; ranks of a distributed job shard documents the same way workers do (``rank`` / ``world_size``); batches
are collated into pinned memory for asynchronous host-to-device copies.
"""

from __future__ import annotations

import json
import os
import random
import time
from typing import Any, Iterator, List, Optional, Tuple

import torch
from torch.utils.data import DataLoader, IterableDataset

TEXT_KEYS = ("text", "content", "story", "prompt")
_TEXT_EXT = (".txt", ".md", ".py", ".c", ".cpp", ".h", ".rst")


def iter_local_texts(path: str) -> Iterator[str]:
    ext = os.path.splitext(path)[1].lower()
    if ext == ".jsonl":
        with open(path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    elif ext == ".json":
        data = json.load(open(path, encoding="utf-8"))
        yield from (data if isinstance(data, list) else data.get("data", [data]))
    elif ext == ".parquet":
        import pyarrow.parquet as pq

        pf = pq.ParquetFile(path)
        for batch in pf.iter_batches(batch_size=256):
            yield from batch.to_pylist()
    elif ext in _TEXT_EXT:
        with open(path, encoding="utf-8", errors="replace") as f:
            para: List[str] = []
            for line in f:  # one document per blank-line separated paragraph
                if line.strip():
                    para.append(line)
                elif para:
                    yield "".join(para)
                    para = []
            if para:
                yield "".join(para)
    else:
        raise ValueError(f"unsupported local dataset file: {path}")


class TokenStreamDataset(IterableDataset):
    def __init__(self, tokenizer, *, seq_len: int, sep_token_id: int, max_tokens: Optional[int] = None,
                 shuffle_buffer: int = 4096, offset: int = 0, dataset_name: str = "HuggingFaceFW/fineweb-edu",
                 dataset_config: Optional[str] = "sample-10BT", split: str = "train", token: Optional[str] = None,
                 texts: Optional[Any] = None, rank: int = 0, world_size: int = 1, seed: int = 0):
        self.tokenizer, self.seq_len, self.sep_token_id = tokenizer, seq_len, sep_token_id
        self.max_tokens, self.shuffle_buffer, self.offset = max_tokens, shuffle_buffer, offset
        self.dataset_name, self.dataset_config, self.split = dataset_name, dataset_config, split
        self.token = token or os.environ.get("HF_TOKEN") or os.environ.get("HUGGING_FACE_HUB_TOKEN")
        self.texts = texts  # optional in-memory iterable of strings / dicts (tests, synthetic corpora)
        self.rank, self.world_size, self.seed = rank, world_size, seed
        self._boundary_cache: dict = {}

    def _is_word_boundary(self, token_id: int) -> bool:
        hit = self._boundary_cache.get(token_id)
        if hit is not None:
            return hit
        try:
            t = self.tokenizer.id_to_token(token_id)
        except Exception:
            t = None
        if not t:
            r = True
        elif (t[0] == "[" and t[-1] == "]") or (t.startswith("<|") and t.endswith("|>")):
            r = True
        else:
            r = t[0] in ("Ġ", "Ċ", "\n", " ") or not t[0].isalnum()
        self._boundary_cache[token_id] = r
        return r

    def _stream(self):
        if self.texts is not None:
            return iter(self.texts)
        if os.path.exists(self.dataset_name):
            return iter_local_texts(self.dataset_name)
        from datasets import DownloadConfig, load_dataset

        return load_dataset(self.dataset_name, name=self.dataset_config, split=self.split, streaming=True, token=self.token,
                            download_config=DownloadConfig(max_retries=10))

    def _encode(self, text: str) -> List[int]:
        out = self.tokenizer.encode(text)
        return list(getattr(out, "ids", out))

    def _windows(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        info = torch.utils.data.get_worker_info()
        nshard = self.world_size * (info.num_workers if info else 1)
        shard = self.rank * (info.num_workers if info else 1) + (info.id if info else 0)
        rng = random.Random(self.seed + shard)
        skip = self.offset // nshard
        buf: List[int] = []
        pending: List[Tuple[torch.Tensor, torch.Tensor]] = []
        produced, n = 0, self.seq_len + 1

        def flush():
            rng.shuffle(pending)
            yield from pending
            pending.clear()

        for idx, sample in enumerate(self._stream()):
            text = sample if isinstance(sample, str) else next((sample[k] for k in TEXT_KEYS if sample.get(k)), "")
            if not text or not text.strip() or idx % nshard != shard:
                continue
            ids = self._encode(text)
            if skip:
                if skip >= len(ids):
                    skip -= len(ids)
                    continue
                ids, skip = ids[skip:], 0
            buf.extend(ids)
            buf.append(self.sep_token_id)
            while len(buf) >= n:
                cut = n
                if cut < len(buf) and not self._is_word_boundary(buf[cut]):
                    b = cut
                    while b > cut - 16 and b > 0 and not self._is_word_boundary(buf[b]):
                        b -= 1
                    if b > 0:
                        cut = b
                chunk = buf[:cut]
                del buf[:cut]
                chunk += [0] * (n - len(chunk))
                t = torch.tensor(chunk, dtype=torch.long)
                pending.append((t[:-1].clone(), t[1:].clone()))
                produced += self.seq_len
                if len(pending) >= self.shuffle_buffer:
                    yield from flush()
                if self.max_tokens is not None and produced >= self.max_tokens:
                    yield from flush()
                    return
        yield from flush()

    def __iter__(self):
        for attempt in range(3):
            try:
                yield from self._windows()
                return
            except (OSError, ConnectionError, TimeoutError):
                if attempt == 2:
                    raise
                time.sleep(2**attempt)


def _collate_pinned(batch):
    x = torch.stack([b[0] for b in batch])
    y = torch.stack([b[1] for b in batch])
    if torch.cuda.is_available():
        x, y = x.pin_memory(), y.pin_memory()
    return x, y


def build_dataloader(tokenizer, config: dict, sep_token_id: int, *, is_holdout: bool, texts=None, rank: int = 0,
                     world_size: int = 1) -> DataLoader:
    eval_tokens = config.get("eval_batches", 5) * config["batch_size"] * config["seq_len"]
    ds = TokenStreamDataset(tokenizer, seq_len=config["seq_len"], sep_token_id=sep_token_id,
                            max_tokens=eval_tokens if is_holdout else None, offset=0 if is_holdout else eval_tokens,
                            shuffle_buffer=config.get("shuffle_buffer", 4096),
                            dataset_name=config.get("dataset_name", "HuggingFaceFW/fineweb-edu"),
                            dataset_config=config.get("dataset_config", "sample-10BT"), texts=texts, rank=rank,
                            world_size=world_size, seed=int(config.get("seed", 0)))
    workers = 0 if (is_holdout or texts is not None) else int(config.get("num_workers", 2))
    return DataLoader(ds, batch_size=config["batch_size"], num_workers=workers, drop_last=True, collate_fn=_collate_pinned,
                      persistent_workers=workers > 0, prefetch_factor=4 if workers > 0 else None)
