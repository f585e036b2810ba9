"""Lossless sequence compression on top of a base tokenizer.

Parity (``triune/data/dynamic_tokenizer.py:197-807``): frequent adjacent id pairs are replaced by composite ids
allocated from ``dynamic_id_start`` (150 000) upwards; rules nest (a composite can be a child of a later composite)
and expand back to the exact base ids; ``compress_tokens`` first applies the registered rules, then keeps merging the
most frequent pair of the sequence until the length ratio reaches the target (clamped to 2.2x..3.8x); curated n-grams
(common words, indentation runs) are registered up front; ``pack_chunks`` / ``unpack_chunks`` cut compressed streams into
fixed-size chunks with a padding id; telemetry tracks the achieved ratio.

Differences: registered rules are applied in priority order in one pass over a linked list with a pair index instead
of repeated full rescans; ``lookup_vector`` builds one dense table (dynamic id -> first ``max_len`` base ids) that can
live on the GPU so expansion of a batch is a single gather.
"""

from __future__ import annotations

from collections import Counter
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch

from .tokenizer import SPECIAL_TOKENS, load_tokenizer

CURATED_NGRAMS = (" the", " and", " of", " to", " in", " that", " is", " for", "ing", "tion", "    ", "        ", "\n\n",
                  " return", " self", " import", "def ", "class ", "    return ", " = ", "():", "\n    ")
# word beginnings and endings of English and of code identifiers, registered (after the n-grams above, so their ids do
# not move) with and without the space that precedes a prefix or follows a suffix
COMMON_PREFIXES = ("un", "re", "pre", "dis", "anti", "multi", "inter", "over", "under", "sub", "super", "trans", "non", "semi", "auto", "micro")
COMMON_SUFFIXES = ("tion", "tions", "ing", "ment", "ments", "able", "ible", "ness", "less", "ful", "ally", "ized", "izes", "ity", "ous", "ive",
                   "ed", "er", "est", "ly")
CURATED_NGRAM_PATTERNS = list(CURATED_NGRAMS)  # the reference's name of the first table


@dataclass
class DynamicTokenizerOutput:
    input_ids: List[int]
    attention_mask: List[int]
    uncompressed_length: int
    compressed_length: int
    compression_ratio: float
    chunks: List[List[int]] = field(default_factory=list)

    def __getitem__(self, item: str) -> Any:
        return getattr(self, item)

    def to_tensor(self, device=None) -> torch.Tensor:
        return torch.tensor(self.input_ids, dtype=torch.long, device=device)


class _ByteFallback:
    """Stand-in base tokenizer (raw UTF-8 bytes offset past the special tokens) when no vocabulary file is given."""

    def __init__(self):
        self.offset = len(SPECIAL_TOKENS)

    def encode(self, text: str):
        return [b + self.offset for b in text.encode("utf-8")]

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False) -> str:
        return bytes(i - self.offset for i in ids if self.offset <= i < self.offset + 256).decode("utf-8", errors="replace")

    def get_vocab_size(self) -> int:
        return 256 + self.offset


class DynamicTokenizer:
    def __init__(self, base_tokenizer: Any = None, custom_vocab_path: Optional[Union[str, Path]] = None, chunk_size: int = 64,
                 target_compression_ratio: float = 2.6, dynamic_id_start: int = 150_000, enable_compression: bool = True):
        self.chunk_size, self.target_compression_ratio = int(chunk_size), float(target_compression_ratio)
        self.dynamic_id_start = self.next_dynamic_id = int(dynamic_id_start)
        self.enable_compression = enable_compression
        if base_tokenizer is None and custom_vocab_path is not None:
            base_tokenizer = load_tokenizer(custom_vocab_path)
        if base_tokenizer is None and Path("triune_tokenizer.json").is_file():
            base_tokenizer = load_tokenizer("triune_tokenizer.json")
        self.base_tokenizer = base_tokenizer or _ByteFallback()
        self.merge_rules: Dict[Tuple[int, int], int] = {}
        self.decomp_rules: Dict[int, Tuple[int, int]] = {}
        self.expansion_cache: Dict[int, List[int]] = {}
        self.ngram_to_id: Dict[str, int] = {}
        self.id_to_ngram: Dict[int, str] = {}
        self._table: Optional[torch.Tensor] = None
        self.telemetry = {"total_uncompressed_tokens": 0, "total_compressed_tokens": 0, "encodings_processed": 0,
                          "registered_ngrams": 0}
        for g in CURATED_NGRAMS:
            self.register_ngram(g)
        for pre in COMMON_PREFIXES:
            self.register_ngram(" " + pre)
            self.register_ngram(pre)
        for suf in COMMON_SUFFIXES:
            self.register_ngram(suf + " ")
            self.register_ngram(suf)

    # ------------------------------------------------------------------ base tokenizer access
    def _base_ids(self, text: str) -> List[int]:
        out = self.base_tokenizer.encode(text)
        return list(getattr(out, "ids", out))

    def _base_text(self, ids: List[int], skip_special_tokens: bool = False) -> str:
        try:
            return self.base_tokenizer.decode(ids, skip_special_tokens=skip_special_tokens)
        except TypeError:
            return self.base_tokenizer.decode(ids)

    @property
    def vocab_size(self) -> int:
        b = self.base_tokenizer
        base = b.get_vocab_size() if hasattr(b, "get_vocab_size") else len(getattr(b, "vocab", ())) or 32000
        return max(base, self.next_dynamic_id)

    @property
    def compression_ratio(self) -> float:
        c = self.telemetry["total_compressed_tokens"]
        return self.telemetry["total_uncompressed_tokens"] / c if c else 1.0

    # ------------------------------------------------------------------ rules
    def _new_rule(self, pair: Tuple[int, int]) -> int:
        nid = self.merge_rules.get(pair)
        if nid is None:
            nid = self.next_dynamic_id
            self.next_dynamic_id += 1
            self.merge_rules[pair] = nid
            self.decomp_rules[nid] = pair
            self._table = None
        return nid

    def register_ngram(self, ngram: str, token_id: Optional[int] = None) -> int:
        """Register a text n-gram: its base ids are folded left to right into nested pair rules; returns the id that
        stands for the whole n-gram (the base id itself when the n-gram is a single token)."""
        if ngram in self.ngram_to_id:
            return self.ngram_to_id[ngram]
        ids = self._base_ids(ngram)
        if not ids:
            raise ValueError("cannot register an empty n-gram")
        cur = ids[0]
        for nxt in ids[1:]:
            cur = self._new_rule((cur, nxt))
        if token_id is not None and token_id != cur and len(ids) > 1:  # caller-chosen id aliases the top rule
            pair = self.decomp_rules.pop(cur)
            self.merge_rules[pair] = token_id
            self.decomp_rules[token_id] = pair
            self.next_dynamic_id = max(self.next_dynamic_id, token_id + 1)
            cur = token_id
        self.ngram_to_id[ngram], self.id_to_ngram[cur] = cur, ngram
        self.telemetry["registered_ngrams"] += 1
        return cur

    def learn_ngrams(self, texts: Iterable[str], max_new_rules: int = 512, min_count: int = 4) -> int:
        """Greedy pair learning over a corpus (BPE over token ids); returns the number of new rules."""
        seqs = [self.compress_tokens(self._base_ids(t), target_ratio=1.0, min_ratio=1.0) for t in texts]
        added = 0
        while added < max_new_rules:
            pairs: Counter = Counter()
            for s in seqs:
                pairs.update(zip(s, s[1:]))
            if not pairs:
                break
            pair, n = pairs.most_common(1)[0]
            if n < min_count:
                break
            nid = self._new_rule(pair)
            seqs = [self._merge_pair(s, pair, nid) for s in seqs]
            added += 1
        return added

    @staticmethod
    def _merge_pair(seq: List[int], pair: Tuple[int, int], nid: int) -> List[int]:
        out, i, a, b = [], 0, pair[0], pair[1]
        n = len(seq)
        while i < n:
            if i < n - 1 and seq[i] == a and seq[i + 1] == b:
                out.append(nid)
                i += 2
            else:
                out.append(seq[i])
                i += 1
        return out

    # ------------------------------------------------------------------ compression
    def compress_tokens(self, tokens: Sequence[int], target_ratio: Optional[float] = None, max_ratio: float = 3.8,
                        min_ratio: float = 2.2) -> List[int]:
        if len(tokens) <= 2 or not self.enable_compression:
            return list(tokens)
        n0 = len(tokens)
        target = max(min_ratio, min(self.target_compression_ratio if target_ratio is None else target_ratio, max_ratio))
        cur = list(tokens)
        rules = self.merge_rules
        changed = True
        while changed and len(cur) > 1:  # registered rules, nested rules resolve over successive passes
            changed = False
            out, i, n = [], 0, len(cur)
            while i < n:
                nid = rules.get((cur[i], cur[i + 1])) if i < n - 1 else None
                if nid is not None:
                    out.append(nid)
                    i += 2
                    changed = True
                else:
                    out.append(cur[i])
                    i += 1
            cur = out
        steps = 0
        while n0 / max(1, len(cur)) < target and len(cur) > 2 and steps < 250:  # adaptive merges for this sequence
            steps += 1
            pair, _ = Counter(zip(cur, cur[1:])).most_common(1)[0]
            nxt = self._merge_pair(cur, pair, self._new_rule(pair))
            if len(nxt) == len(cur):
                break
            cur = nxt
            if n0 / max(1, len(cur)) >= max_ratio:
                break
        return cur

    def _expand_token(self, tid: int) -> List[int]:
        hit = self.expansion_cache.get(tid)
        if hit is not None:
            return hit
        if tid not in self.decomp_rules:
            return [tid]
        out: List[int] = []
        stack = [tid]
        while stack:  # iterative: rule chains can be hundreds deep
            t = stack.pop()
            pair = self.decomp_rules.get(t)
            if pair is None:
                out.append(t)
            else:
                cached = self.expansion_cache.get(t)
                if cached is not None and t != tid:
                    out.extend(cached)
                else:
                    stack.append(pair[1])
                    stack.append(pair[0])
        self.expansion_cache[tid] = out
        return out

    def decompress_tokens(self, tokens: Iterable[int]) -> List[int]:
        out: List[int] = []
        for t in tokens:
            out.extend(self._expand_token(int(t)) if t >= self.dynamic_id_start or t in self.decomp_rules else [int(t)])
        return out

    # ------------------------------------------------------------------ text API
    def encode(self, text: str, compress: Optional[bool] = None, return_chunks: bool = False, pad_id: int = 0,
               target_ratio: Optional[float] = None) -> DynamicTokenizerOutput:
        base = self._base_ids(text)
        ids = self.compress_tokens(base, target_ratio) if (self.enable_compression if compress is None else compress) else base
        t = self.telemetry
        t["total_uncompressed_tokens"] += len(base)
        t["total_compressed_tokens"] += len(ids)
        t["encodings_processed"] += 1
        chunks = self.pack_chunks(ids, pad_id=pad_id) if return_chunks else []
        return DynamicTokenizerOutput(ids, [1] * len(ids), len(base), len(ids), len(base) / max(1, len(ids)), chunks)

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = False, pad_id: Optional[int] = None) -> str:
        ids = [int(i) for i in (ids.tolist() if torch.is_tensor(ids) else ids)]
        if pad_id is not None:
            ids = [i for i in ids if i != pad_id]
        return self._base_text(self.decompress_tokens(ids), skip_special_tokens)

    def encode_batch(self, texts: Sequence[str], pad_id: int = 0, max_length: Optional[int] = None,
                     return_tensors: bool = True, device=None):
        outs = [self.encode(t) for t in texts]
        L = max_length or max((o.compressed_length for o in outs), default=0)
        ids = [o.input_ids[:L] + [pad_id] * max(0, L - o.compressed_length) for o in outs]
        mask = [[1] * min(L, o.compressed_length) + [0] * max(0, L - o.compressed_length) for o in outs]
        res = {"input_ids": ids, "attention_mask": mask, "compression_ratios": [o.compression_ratio for o in outs]}
        if return_tensors:
            res["input_ids"] = torch.tensor(ids, dtype=torch.long, device=device)
            res["attention_mask"] = torch.tensor(mask, dtype=torch.long, device=device)
        return res

    def decode_batch(self, batch, attention_mask=None, skip_special_tokens: bool = False) -> List[str]:
        rows = batch.tolist() if torch.is_tensor(batch) else batch
        masks = attention_mask.tolist() if torch.is_tensor(attention_mask) else attention_mask
        out = []
        for r, row in enumerate(rows):
            if masks is not None:
                row = [t for t, m in zip(row, masks[r]) if m]
            out.append(self.decode(row, skip_special_tokens))
        return out

    def pack_chunks(self, ids: Sequence[int], chunk_size: Optional[int] = None, pad_id: int = 0) -> List[List[int]]:
        c = chunk_size or self.chunk_size
        chunks = [list(ids[i : i + c]) for i in range(0, len(ids), c)]
        if chunks and len(chunks[-1]) < c:
            chunks[-1] += [pad_id] * (c - len(chunks[-1]))
        return chunks

    def unpack_chunks(self, chunks: Sequence[Sequence[int]], pad_id: int = 0, length: Optional[int] = None) -> List[int]:
        flat = [int(t) for ch in chunks for t in ch]
        if length is not None:
            return flat[:length]
        while flat and flat[-1] == pad_id:
            flat.pop()
        return flat

    def lookup_vector(self, max_len: int = 16, device=None) -> torch.Tensor:
        """[num_dynamic_ids, max_len + 1] table: column 0 = expansion length, then the base ids (truncated to
        ``max_len``), so a batch of composite ids expands with one gather on the device."""
        if self._table is None or self._table.shape[1] != max_len + 1:
            n = self.next_dynamic_id - self.dynamic_id_start
            tab = torch.zeros(max(1, n), max_len + 1, dtype=torch.long)
            for i in range(n):
                ex = self._expand_token(self.dynamic_id_start + i)
                tab[i, 0] = len(ex)
                k = min(len(ex), max_len)
                tab[i, 1 : 1 + k] = torch.tensor(ex[:k])
            self._table = tab
        return self._table.to(device) if device is not None else self._table

    def get_compression_stats(self) -> Dict[str, Any]:
        return dict(self.telemetry, compression_ratio=self.compression_ratio, merge_rules=len(self.merge_rules),
                    dynamic_ids=self.next_dynamic_id - self.dynamic_id_start, vocab_size=self.vocab_size)
