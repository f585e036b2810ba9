"""Search of public model, dataset and plugin repositories (GitHub, Hugging Face) for the module manager.

The only part of the framework that talks to the internet, and only when a caller asks: every method makes one HTTPS
GET with a short timeout and returns ``[]`` when the network, the service or the answer's format fails, so offline
machines see empty result lists rather than errors (``triune/modules/github_client.py:11-188`` of the reference)."""

from __future__ import annotations

import json
import urllib.parse
import urllib.request
from typing import Any, Dict, List, Optional

_KINDS = (("plugin", ("plugin", "node", "dag", "custom-node")), ("adapter", ("lora", "adapter", "peft")), ("dataset", ("dataset", "corpus")))


def classify_repository(name: str, description: str = "") -> str:
    """"plugin", "adapter", "dataset" or "model", from key words in a repository's name and description."""
    text = f"{name} {description}".lower()
    return next((kind for kind, words in _KINDS if any(w in text for w in words)), "model")


class RepoSearchClient:
    GITHUB_API_URL = "https://api.github.com"
    HF_API_URL = "https://huggingface.co/api"
    USER_AGENT = "triune-b200-module-manager/1.0"

    def __init__(self, github_token: Optional[str] = None, hf_token: Optional[str] = None, timeout: float = 5.0) -> None:
        self.github_token, self.hf_token, self.timeout = github_token, hf_token, timeout

    def _get_github_headers(self) -> Dict[str, str]:
        h = {"Accept": "application/vnd.github.v3+json", "User-Agent": self.USER_AGENT}
        if self.github_token:
            h["Authorization"] = f"token {self.github_token}"
        return h

    def _get_hf_headers(self) -> Dict[str, str]:
        h = {"User-Agent": self.USER_AGENT}
        if self.hf_token:
            h["Authorization"] = f"Bearer {self.hf_token}"
        return h

    def _get_json(self, url: str, headers: Dict[str, str]) -> Any:
        try:
            with urllib.request.urlopen(urllib.request.Request(url, headers=headers), timeout=self.timeout) as r:
                return json.loads(r.read().decode("utf-8"))
        except Exception:
            return None

    def search_github_repositories(self, query: str, sort: str = "stars", per_page: int = 12) -> List[Dict[str, Any]]:
        q = urllib.parse.quote(query or "pytorch transformer deep-learning")
        data = self._get_json(f"{self.GITHUB_API_URL}/search/repositories?q={q}&sort={sort}&order=desc&per_page={int(per_page)}",
                              self._get_github_headers())
        out = []
        for it in (data or {}).get("items", []) if isinstance(data, dict) else []:
            try:
                out.append({"id": f"github:{it['full_name']}", "name": it["name"], "full_name": it["full_name"], "source": "github",
                            "type": classify_repository(it["name"], it.get("description") or ""), "description": it.get("description") or "",
                            "stars": int(it.get("stargazers_count", 0)), "url": it.get("html_url"), "clone_url": it.get("clone_url"),
                            "default_branch": it.get("default_branch", "main"), "updated_at": it.get("updated_at"),
                            "license": (it.get("license") or {}).get("spdx_id")})
            except (KeyError, TypeError, ValueError):
                continue
        return out

    def _search_hf(self, kind: str, query: str, limit: int) -> List[Dict[str, Any]]:
        q = urllib.parse.quote(query or "")
        data = self._get_json(f"{self.HF_API_URL}/{kind}?search={q}&limit={int(limit)}&sort=downloads&direction=-1", self._get_hf_headers())
        out = []
        for it in data if isinstance(data, list) else []:
            rid = it.get("id") or it.get("modelId")
            if not rid:
                continue
            out.append({"id": f"hf:{rid}", "name": rid.split("/")[-1], "full_name": rid, "source": "huggingface",
                        "type": "dataset" if kind == "datasets" else classify_repository(rid, " ".join(it.get("tags") or [])),
                        "downloads": int(it.get("downloads") or 0), "likes": int(it.get("likes") or 0), "tags": list(it.get("tags") or [])[:12],
                        "url": f"https://huggingface.co/{'datasets/' if kind == 'datasets' else ''}{rid}"})
        return out

    def search_huggingface_models(self, query: str, limit: int = 12) -> List[Dict[str, Any]]:
        return self._search_hf("models", query, limit)

    def search_huggingface_datasets(self, query: str, limit: int = 12) -> List[Dict[str, Any]]:
        return self._search_hf("datasets", query, limit)


GitHubClient = RepoSearchClient
