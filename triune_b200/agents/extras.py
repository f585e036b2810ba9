"""Agent extras: a persistent memory with similarity recall, a library of markdown skills, and provider records.

* :class:`AgentMemoryStore` keeps preferences, per-tool success statistics and free-text lessons in one JSON file
  (written atomically) and recalls the lessons closest to a query by TF-IDF cosine similarity.
* :class:`SkillLibrary` reads ``*.md`` files with a small ``key: value`` header (``name``, ``description``,
  ``triggers``) and returns the skills whose triggers or text match a request, ready to be put in a prompt.
* :class:`ProviderManager` holds bring-your-own-key provider records; it sends nothing by itself: a transport
  callable must be supplied by the embedding application, because this package makes no outbound requests.

Thin counterparts of ``triune/agents/memory.py:77-409``, ``triune/agents/skills.py:103-300`` and
``triune/agents/providers.py:20-342``.
"""

from __future__ import annotations

import json
import math
import os
import re
import tempfile
import time
from collections import Counter
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

_WORD = re.compile(r"[a-z0-9_]+")


def _tokens(text: str) -> List[str]:
    return _WORD.findall(text.lower())


class AgentMemoryStore:
    def __init__(self, path: Optional[str] = None, max_lessons: int = 500):
        self.path, self.max_lessons = (Path(path) if path else None), max_lessons
        self.data: Dict[str, Any] = {"preferences": {}, "tool_stats": {}, "lessons": []}
        if self.path is not None and self.path.is_file():
            try:
                self.data.update(json.loads(self.path.read_text()))
            except ValueError:
                pass  # a corrupt file is replaced at the next save

    # ------------------------------------------------------------------ persistence
    def save(self) -> None:
        if self.path is None:
            return
        self.path.parent.mkdir(parents=True, exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=str(self.path.parent), suffix=".tmp")
        with os.fdopen(fd, "w") as f:
            json.dump(self.data, f)
        os.replace(tmp, self.path)

    # ------------------------------------------------------------------ content
    def set_preference(self, key: str, value: Any) -> None:
        self.data["preferences"][key] = value
        self.save()

    def record_tool(self, tool: str, ok: bool) -> Dict[str, int]:
        s = self.data["tool_stats"].setdefault(tool, {"calls": 0, "failures": 0})
        s["calls"] += 1
        s["failures"] += 0 if ok else 1
        self.save()
        return s

    def add_lesson(self, text: str, tags: Optional[List[str]] = None) -> None:
        self.data["lessons"].append({"text": text, "tags": list(tags or []), "time": time.time()})
        del self.data["lessons"][: max(0, len(self.data["lessons"]) - self.max_lessons)]
        self.save()

    def recall(self, query: str, k: int = 3, min_score: float = 0.05) -> List[Tuple[float, str]]:
        """The ``k`` lessons most similar to ``query`` (TF-IDF cosine), best first."""
        docs = [_tokens(l["text"] + " " + " ".join(l["tags"])) for l in self.data["lessons"]]
        if not docs:
            return []
        df = Counter(t for d in docs for t in set(d))
        n = len(docs)
        idf = {t: math.log((1 + n) / (1 + c)) + 1.0 for t, c in df.items()}

        def vec(toks):
            tf = Counter(toks)
            v = {t: c * idf.get(t, 0.0) for t, c in tf.items()}
            norm = math.sqrt(sum(x * x for x in v.values())) or 1.0
            return {t: x / norm for t, x in v.items()}

        q = vec(_tokens(query))
        scored = []
        for l, d in zip(self.data["lessons"], docs):
            dv = vec(d)
            s = sum(w * dv.get(t, 0.0) for t, w in q.items())
            if s >= min_score:
                scored.append((s, l["text"]))
        return sorted(scored, key=lambda x: -x[0])[:k]


@dataclass
class Skill:
    name: str
    description: str
    triggers: List[str]
    body: str
    path: Optional[str] = None

    uses: int = 0
    successes: int = 0

    @property
    def success_rate(self) -> float:
        return self.successes / self.uses if self.uses else 0.0

    def matches(self, request: str) -> float:
        req = set(_tokens(request))
        hit = sum(1.0 for t in self.triggers if set(_tokens(t)) <= req)
        overlap = len(req & set(_tokens(self.name + " " + self.description))) / (len(req) or 1)
        return hit + overlap


class SkillLibrary:
    def __init__(self, directory: Optional[str] = None):
        self.skills: Dict[str, Skill] = {}
        if directory:
            self.load_directory(directory)

    @staticmethod
    def parse(text: str, path: Optional[str] = None) -> Skill:
        head: Dict[str, str] = {}
        lines = text.splitlines()
        i = 0
        if lines and lines[0].strip() == "---":
            i = 1
            while i < len(lines) and lines[i].strip() != "---":
                k, _, v = lines[i].partition(":")
                head[k.strip().lower()] = v.strip()
                i += 1
            i += 1
        name = head.get("name") or (Path(path).stem if path else "skill")
        trig = [t.strip() for t in head.get("triggers", "").split(",") if t.strip()]
        return Skill(name, head.get("description", ""), trig, "\n".join(lines[i:]).strip(), path)

    def load_directory(self, directory: str) -> int:
        n = 0
        for p in sorted(Path(directory).glob("*.md")):
            s = self.parse(p.read_text(encoding="utf-8"), str(p))
            self.skills[s.name] = s
            n += 1
        return n

    def add(self, skill: Skill) -> None:
        self.skills[skill.name] = skill

    def select(self, request: str, k: int = 2, min_score: float = 0.2) -> List[Skill]:
        scored = sorted(((s.matches(request), s) for s in self.skills.values()), key=lambda x: -x[0])
        return [s for sc, s in scored[:k] if sc >= min_score]

    def prompt_block(self, request: str, k: int = 2) -> str:
        chosen = self.select(request, k)
        return "\n\n".join(f"## Skill: {s.name}\n{s.body}" for s in chosen)


@dataclass
class Provider:
    name: str
    base_url: str
    model: str
    api_key: str = field(default="", repr=False)


class ProviderManager:
    """Provider records plus an injected transport ``(provider, messages, options) -> text``."""

    def __init__(self, transport: Optional[Callable[[Provider, List[Dict[str, str]], Dict[str, Any]], str]] = None):
        self.providers: Dict[str, Provider] = {}
        self.transport = transport

    def save(self, name: str, base_url: str, model: str, api_key: str) -> Provider:
        if not base_url.startswith(("https://", "http://127.0.0.1", "http://localhost")):
            raise ValueError("provider URLs must be https (or loopback http)")
        self.providers[name.lower()] = Provider(name.lower(), base_url.rstrip("/"), model, api_key)
        return self.providers[name.lower()]

    def describe(self) -> List[Dict[str, Any]]:
        return [{"name": p.name, "base_url": p.base_url, "model": p.model, "key_hint": ("..." + p.api_key[-4:]) if p.api_key else ""}
                for p in self.providers.values()]

    # ---- method names of the reference's manager (``triune/agents/providers.py``)
    def register_provider(self, name: str, base_url: str, model: str, api_key: str = "") -> Provider:
        return self.save(name, base_url, model, api_key)

    def get_provider(self, name: str) -> Optional[Provider]:
        return self.providers.get(name.lower())

    def list_active_providers(self) -> List[str]:
        return sorted(n for n, p in self.providers.items() if p.api_key or p.base_url.startswith(("http://127.0.0.1", "http://localhost")))

    def pick_default_model(self) -> Optional[str]:
        act = self.list_active_providers()
        return f"{act[0]}:{self.providers[act[0]].model}" if act else None

    def complete_chat(self, messages: List[Dict[str, str]], model: Optional[str] = None, **options) -> Dict[str, Any]:
        """``model`` is ``provider:model`` (or a provider name); -> ``{"text", "provider", "model"}``."""
        spec = model or self.pick_default_model()
        if spec is None:
            raise RuntimeError("no provider is configured")
        name, _, mdl = spec.partition(":")
        p = self.providers.get(name.lower())
        if p is None:
            raise KeyError(f"unknown provider {name!r}")
        if mdl:
            options = {**options, "model": mdl}
        return {"text": self.chat(name, messages, **options), "provider": p.name, "model": mdl or p.model}

    def chat(self, name: str, messages: List[Dict[str, str]], **options) -> str:
        p = self.providers.get(name.lower())
        if p is None:
            raise KeyError(f"unknown provider {name!r}")
        if self.transport is None:
            raise RuntimeError("no transport configured: this package makes no outbound requests on its own")
        return self.transport(p, messages, options)
