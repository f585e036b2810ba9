"""Files and text scoring shared by the agent stores (memory, skills, workspaces).

Parity: ``triune/agents/_storage.py`` of the reference (atomic JSON files, a loader that never raises on a damaged
file, term extraction with stop words and character trigrams, TF-IDF cosine ranking)."""

from __future__ import annotations

import json
import math
import os
import re
import tempfile
import threading
from collections import Counter
from pathlib import Path
from typing import Any, Dict, List

_LOCK = threading.Lock()
_TERM = re.compile(r"[a-z0-9_]{2,}")
STOPWORDS = frozenset(
    "a an and are as at be but by can do for from has have how if in into is it its not of on or so that the their then there "
    "these this to use was we were what when which who will with you your".split())


def atomic_write_text(path, text: str) -> None:
    """Write ``text`` (UTF-8) so that a reader sees the old file or the new one, never a part of either: the bytes go to
    a temporary file in the same directory, which then replaces the target."""
    target = Path(path).resolve()
    with _LOCK:
        target.parent.mkdir(parents=True, exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=str(target.parent), prefix=f".{target.name}.", suffix=".tmp")
        done = False
        try:
            with os.fdopen(fd, "w", encoding="utf-8", newline="\n") as f:
                f.write(text)
                f.flush()
                try:
                    os.fsync(f.fileno())
                except OSError:
                    pass  # file systems without fsync still get the rename
            os.replace(tmp, target)
            done = True
        finally:
            if not done:
                try:
                    os.unlink(tmp)
                except OSError:
                    pass


def atomic_write_json(path, payload: Any) -> None:
    atomic_write_text(path, json.dumps(payload, indent=2, ensure_ascii=False))


def load_validated_json_dict(path) -> Dict[str, Any]:
    """The JSON object stored at ``path``; ``{}`` when the file is missing, unreadable, not JSON, or not an object."""
    p = Path(path)
    if not p.is_file():
        return {}
    try:
        data = json.loads(p.read_text(encoding="utf-8"))
    except (OSError, ValueError):
        return {}
    return data if isinstance(data, dict) else {}


def tokenize_terms(text: str, *, include_char_ngrams: bool = True) -> List[str]:
    """Lower-case words of two or more characters without stop words; with ``include_char_ngrams`` also ``#abc``
    trigrams of every word of four or more characters, so that inflected forms still overlap."""
    words = [w for w in _TERM.findall((text or "").lower()) if w not in STOPWORDS]
    if not include_char_ngrams:
        return words
    grams = [f"#{w[i:i + 3]}" for w in words if len(w) >= 4 for i in range(len(w) - 2)]
    return words + grams


def compute_tfidf_cosine_scores(query: str, docs: List[str]) -> List[float]:
    """Cosine similarity between ``query`` and each of ``docs`` under sub-linear term frequency (1 + ln tf) and smoothed
    inverse document frequency (ln((1 + N) / (1 + df)) + 1, the query counted as a document)."""
    if not docs:
        return []
    q = Counter(tokenize_terms(query))
    if not q:
        return [0.0] * len(docs)
    counts = [Counter(tokenize_terms(d)) for d in docs]
    df: Counter = Counter()
    for c in counts + [q]:
        df.update(c.keys())
    n = len(docs) + 1
    idf = {t: math.log((1.0 + n) / (1.0 + f)) + 1.0 for t, f in df.items()}

    def vec(c: Counter) -> Dict[str, float]:
        return {t: (1.0 + math.log(k)) * idf.get(t, 1.0) for t, k in c.items()}

    qv = vec(q)
    qn = math.sqrt(sum(v * v for v in qv.values())) or 1.0
    out = []
    for c in counts:
        dv = vec(c)
        dn = math.sqrt(sum(v * v for v in dv.values()))
        dot = sum(w * qv[t] for t, w in dv.items() if t in qv)
        out.append(max(0.0, min(1.0, dot / (qn * dn))) if dn > 0 else 0.0)
    return out
