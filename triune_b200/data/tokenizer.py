"""Byte-level BPE tokenizer: loader, pure-Python implementation and trainer.

Parity (``triune/data/tokenizer.py:11-273``): 21 special tokens, ``load_tokenizer`` (Hugging Face ``tokenizers`` when
importable, else the pure-Python class reading the same ``tokenizer.json``), Llama-3 style chat template, streaming
decode that never emits half a UTF-8 sequence, ``build_tokenizer`` trainer.

Differences: the trainer is self-contained (incremental pair counts over a word-frequency table) and takes any
iterable of strings, so a tokenizer can be trained without network access; ``encode`` returns an object with ``.ids``
(like ``tokenizers``) that is also a plain list.
"""

from __future__ import annotations

import json
import re
from collections import Counter, defaultdict
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

SPECIAL_TOKENS = [
    "[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]", "<|endoftext|>", "<|begin_of_text|>", "<|end_of_text|>",
    "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>", "<|thought|>", "<|end_thought|>", "<|tool_call|>",
    "<|tool_return|>", "<|system|>", "<|user|>", "<|assistant|>", "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>",
]

# contractions | optional punctuation + letters (any script) | up to three digits | punctuation run | newlines |
# trailing / inner space | any single character left over, so that no input byte is ever dropped
PRETOKEN_PATTERN = (r"'(?:s|t|re|ve|m|ll|d)|[^\r\n\w\s]?[^\W\d_]+|\d{1,3}| ?(?:[^\s\w]|_)+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+|"
                    r"[\s\S]")
_PRETOKEN = re.compile(PRETOKEN_PATTERN)


def bytes_to_unicode() -> Dict[int, str]:
    """The GPT-2 byte <-> printable-character table: printable Latin-1 bytes map to themselves, the other 68 bytes to
    code points from 256 upwards."""
    keep = [b for b in range(256) if 33 <= b <= 126 or 161 <= b <= 172 or 174 <= b <= 255]
    table, extra = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + extra)
            extra += 1
    return table


class Encoding(list):
    """List of ids that also answers ``.ids`` (the ``tokenizers`` result type)."""

    @property
    def ids(self) -> List[int]:
        return list(self)


class PurePythonBPETokenizer:
    def __init__(self, json_path: Union[str, Path, None] = None, vocab: Optional[Dict[str, int]] = None,
                 merges: Optional[List[Tuple[str, str]]] = None):
        if json_path is not None:
            data = json.loads(Path(json_path).read_text(encoding="utf-8"))
            model = data.get("model", {})
            vocab = dict(model.get("vocab", {}))
            for t in data.get("added_tokens", []):
                vocab.setdefault(t["content"], t["id"])
            merges = [tuple(m) if isinstance(m, list) else tuple(m.split(" ", 1)) for m in model.get("merges", [])]
        self.vocab: Dict[str, int] = vocab or {}
        self.inv_vocab: Dict[int, str] = {v: k for k, v in self.vocab.items()}
        self.ranks: Dict[Tuple[str, str], int] = {tuple(m): i for i, m in enumerate(merges or []) if len(m) == 2}
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {c: b for b, c in self.byte_encoder.items()}
        self.specials = {t for t in SPECIAL_TOKENS if t in self.vocab} | {
            t for t in self.vocab if t.startswith("<|") and t.endswith("|>")}
        self._special_re = re.compile("(" + "|".join(re.escape(t) for t in sorted(self.specials, key=len, reverse=True)) + ")") \
            if self.specials else None
        self._cache: Dict[str, Tuple[str, ...]] = {}
        self.unk_id = self.vocab.get("[UNK]", 1)
        self.pad_token_id = self.vocab.get("[PAD]")
        self.sep_token_id = self.vocab.get("[SEP]")
        self.eos_token_id = self.vocab.get("<|eot_id|>", self.vocab.get("<|endoftext|>", self.sep_token_id))

    # ------------------------------------------------------------------ BPE
    def bpe(self, token: str) -> Tuple[str, ...]:
        hit = self._cache.get(token)
        if hit is not None:
            return hit
        parts = list(token)
        while len(parts) > 1:
            best, best_i = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, best_i = r, i
            if best is None:
                break
            a, b = parts[best_i], parts[best_i + 1]
            merged, i = [], 0
            while i < len(parts):  # merge every occurrence of the winning pair, left to right
                if i < len(parts) - 1 and parts[i] == a and parts[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(parts[i])
                    i += 1
            parts = merged
        out = tuple(parts)
        if len(self._cache) < 262144:
            self._cache[token] = out
        return out

    def _encode_plain(self, text: str, out: List[int]) -> None:
        enc, vocab, unk = self.byte_encoder, self.vocab, self.unk_id
        for m in _PRETOKEN.finditer(text):
            word = "".join(enc[b] for b in m.group(0).encode("utf-8"))
            for piece in self.bpe(word):
                out.append(vocab.get(piece, unk))

    def encode(self, text: str, allowed_special: str = "all") -> Encoding:
        out = Encoding()
        if self._special_re is None or allowed_special == "none":
            self._encode_plain(text, out)
            return out
        for chunk in self._special_re.split(text):
            if not chunk:
                continue
            if chunk in self.specials and allowed_special in ("all", chunk):
                out.append(self.vocab[chunk])
            else:
                self._encode_plain(chunk, out)
        return out

    def encode_batch(self, texts: Iterable[str]) -> List[Encoding]:
        return [self.encode(t) for t in texts]

    # ------------------------------------------------------------------ decoding
    def _is_special(self, tok: str) -> bool:
        return tok in self.specials or tok in SPECIAL_TOKENS or (tok.startswith("<|") and tok.endswith("|>")) or (
            tok.startswith("[") and tok.endswith("]") and tok.isupper())

    def _append_bytes(self, buf: bytearray, tok: str) -> None:
        for ch in tok:
            b = self.byte_decoder.get(ch)
            if b is not None:
                buf.append(b)
            else:
                buf.extend(ch.encode("utf-8"))

    def decode(self, ids: Iterable[int], skip_special_tokens: bool = True) -> str:
        buf = bytearray()
        for i in ids:
            tok = self.inv_vocab.get(int(i))
            if tok is None or (skip_special_tokens and self._is_special(tok)):
                continue
            if self._is_special(tok):
                buf.extend(tok.encode("utf-8"))
            else:
                self._append_bytes(buf, tok)
        return buf.decode("utf-8", errors="replace")

    def decode_stream_step(self, buffer: bytearray, token_id: int) -> Tuple[bytearray, str]:
        """Feed one token; returns (bytes still waiting for the rest of a UTF-8 sequence, text that is now final)."""
        tok = self.inv_vocab.get(int(token_id))
        if tok is None or self._is_special(tok):
            return buffer, ""
        self._append_bytes(buffer, tok)
        for hold in range(0, min(4, len(buffer)) + 1):
            try:
                text = bytes(buffer[: len(buffer) - hold]).decode("utf-8")
            except UnicodeDecodeError:
                continue
            return bytearray(buffer[len(buffer) - hold :]), text
        return buffer, ""

    # ------------------------------------------------------------------ misc API
    def apply_chat_template(self, messages: List[Dict[str, str]], add_generation_prompt: bool = True) -> str:
        parts = ["<|begin_of_text|>"]
        for m in messages:
            parts.append(f"<|start_header_id|>{m.get('role', 'user')}<|end_header_id|>\n\n{m.get('content', '')}<|eot_id|>")
        if add_generation_prompt:
            parts.append("<|start_header_id|>assistant<|end_header_id|>\n\n")
        return "".join(parts)

    def get_vocab_size(self) -> int:
        return len(self.vocab)

    def get_vocab(self) -> Dict[str, int]:
        return dict(self.vocab)

    def token_to_id(self, token: str) -> Optional[int]:
        return self.vocab.get(token)

    def id_to_token(self, tid: int) -> Optional[str]:
        return self.inv_vocab.get(tid)

    def save(self, path: Union[str, Path]) -> None:
        """Write a ``tokenizers``-compatible ``tokenizer.json`` (BPE model, byte-level pre-tokeniser and decoder)."""
        merges = [list(p) for p, _ in sorted(self.ranks.items(), key=lambda kv: kv[1])]
        added = [{"id": self.vocab[t], "content": t, "single_word": False, "lstrip": False, "rstrip": False,
                  "normalized": False, "special": True} for t in SPECIAL_TOKENS if t in self.vocab]
        data = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": added, "normalizer": None,
                "pre_tokenizer": {"type": "Sequence", "pretokenizers": [
                    {"type": "Split", "pattern": {"Regex": PRETOKEN_PATTERN}, "behavior": "Isolated", "invert": False},
                    {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True, "use_regex": False}]},
                "post_processor": None, "decoder": {"type": "ByteLevel", "add_prefix_space": False, "trim_offsets": True,
                                                    "use_regex": True},
                "model": {"type": "BPE", "dropout": None, "unk_token": "[UNK]", "continuing_subword_prefix": None,
                          "end_of_word_suffix": None, "fuse_unk": False, "byte_fallback": False, "vocab": self.vocab,
                          "merges": merges}}
        Path(path).write_text(json.dumps(data, ensure_ascii=False), encoding="utf-8")


TriuneTokenizer = PurePythonBPETokenizer


def load_tokenizer(path: Union[str, Path], prefer_fast: bool = True) -> Any:
    p = Path(path)
    if not p.is_file():
        raise FileNotFoundError(f"Tokenizer file not found: {path}")
    if prefer_fast:
        try:
            from tokenizers import Tokenizer
            from tokenizers.decoders import ByteLevel

            tok = Tokenizer.from_file(str(p))
            if tok.decoder is None:
                tok.decoder = ByteLevel()
            return tok
        except Exception:
            pass
    return PurePythonBPETokenizer(p)


def train_bpe(texts: Iterable[str], vocab_size: int = 32000, min_frequency: int = 2,
              special_tokens: Optional[List[str]] = None) -> PurePythonBPETokenizer:
    """Byte-level BPE training: count pre-tokenised words once, then merge the most frequent adjacent pair until the
    vocabulary is full, updating pair counts only for the words that contain the merged pair."""
    enc = bytes_to_unicode()
    words: Counter = Counter()
    for t in texts:
        for m in _PRETOKEN.finditer(t):
            words["".join(enc[b] for b in m.group(0).encode("utf-8"))] += 1
    specials = list(special_tokens if special_tokens is not None else SPECIAL_TOKENS)
    vocab: Dict[str, int] = {t: i for i, t in enumerate(specials)}
    for b in range(256):
        vocab.setdefault(enc[b], len(vocab))
    seqs = [list(w) for w in words]
    freqs = list(words.values())
    pair_count: Counter = Counter()
    where: Dict[Tuple[str, str], set] = defaultdict(set)
    for wi, s in enumerate(seqs):
        for a, b in zip(s, s[1:]):
            pair_count[(a, b)] += freqs[wi]
            where[(a, b)].add(wi)
    merges: List[Tuple[str, str]] = []
    while len(vocab) < vocab_size and pair_count:
        (a, b), n = max(pair_count.items(), key=lambda kv: (kv[1], kv[0]))
        if n < min_frequency:
            break
        merges.append((a, b))
        vocab.setdefault(a + b, len(vocab))
        for wi in list(where.pop((a, b), ())):
            s, f = seqs[wi], freqs[wi]
            for p in zip(s, s[1:]):
                pair_count[p] -= f
                if pair_count[p] <= 0:
                    del pair_count[p]
            merged, i = [], 0
            while i < len(s):
                if i < len(s) - 1 and s[i] == a and s[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(s[i])
                    i += 1
            seqs[wi] = merged
            for p in zip(merged, merged[1:]):
                pair_count[p] += f
                where[p].add(wi)
        pair_count.pop((a, b), None)
    return PurePythonBPETokenizer(vocab=vocab, merges=merges)


def build_tokenizer(output_path: Union[str, Path], *, texts: Optional[Iterable[str]] = None, vocab_size: int = 131_072,
                    min_frequency: int = 2, target_chars: int = 5_000_000_000, dataset_name: str = "wikitext",
                    dataset_config: Optional[str] = "wikitext-103-raw-v1") -> Any:
    """Train and save a tokenizer. ``texts`` is any iterable of strings; without it the named Hugging Face dataset is
    streamed (needs ``datasets`` and network access)."""
    if texts is None:
        try:
            from datasets import load_dataset
        except ImportError as e:
            raise RuntimeError(f"streaming a training corpus needs the 'datasets' package: {e}")
        ds = load_dataset(dataset_name, dataset_config, split="train", streaming=True)

        def stream():
            seen = 0
            for s in ds:
                t = s.get("text", "")
                if t.strip():
                    seen += len(t)
                    yield t
                    if seen >= target_chars:
                        return

        texts = stream()
    tok = train_bpe(texts, vocab_size=vocab_size, min_frequency=min_frequency)
    tok.save(output_path)
    return tok
