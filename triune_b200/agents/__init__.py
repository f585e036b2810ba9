"""Agent harness (thin version of ``triune/agents/*.py``): personas, key/value memory, a tool registry with an
outbound-URL guard, and a loop that lets a locally served model call tools.

The model proposes tool calls as ``<|tool_call|>{"tool": name, "args": {...}}`` lines; results are fed back as
``<|tool_return|>...``. The provider is the in-process engine (no remote keys); the orchestrator runs agents in turn.
"""

from __future__ import annotations

import ipaddress
import json
import re
import socket
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional
from urllib.parse import urlparse


@dataclass
class Tool:
    name: str
    description: str
    fn: Callable[..., Any]
    parameters: Dict[str, str] = field(default_factory=dict)

    def run(self, **args) -> Any:
        return self.fn(**args)


class ToolRegistry:
    def __init__(self):
        self.tools: Dict[str, Tool] = {}
        self.stats: Dict[str, Dict[str, float]] = {}  # per tool: calls, failures, total seconds

    def register(self, tool: Tool) -> None:
        self.tools[tool.name] = tool

    def call(self, name: str, **args) -> Any:
        if name not in self.tools:
            raise KeyError(f"unknown tool {name!r}")
        return self.tools[name].fn(**args)

    def describe(self) -> List[Dict[str, Any]]:
        return [{"name": t.name, "description": t.description, "parameters": t.parameters} for t in self.tools.values()]

    # ---- the same registry under the method names of the reference (``triune/agents/tools.py``)
    def get(self, name: str) -> Optional[Tool]:
        return self.tools.get(name)

    def names(self) -> List[str]:
        return sorted(self.tools)

    def list_tools(self) -> List[Dict[str, Any]]:
        return self.describe()

    def execute(self, name: str, args: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        """Run a tool and report instead of raising: ``{"ok", "result" | "error", "seconds"}``; keeps per-tool statistics."""
        t0 = time.time()
        st = self.stats.setdefault(name, {"calls": 0, "failures": 0, "seconds": 0.0})
        st["calls"] += 1
        try:
            out = {"ok": True, "result": self.call(name, **(args or {}))}
        except Exception as e:
            st["failures"] += 1
            out = {"ok": False, "error": f"{type(e).__name__}: {e}"}
        out["seconds"] = time.time() - t0
        st["seconds"] += out["seconds"]
        return out

    def to_openai_tools(self) -> List[Dict[str, Any]]:
        """The catalogue as ``tools`` of a chat-completions request (JSON-schema parameters)."""
        kinds = {"str": "string", "int": "integer", "float": "number", "bool": "boolean"}
        return [{"type": "function", "function": {"name": t.name, "description": t.description, "parameters": {
            "type": "object", "properties": {k: {"type": kinds.get(v, "string")} for k, v in t.parameters.items()}}}} for t in self.tools.values()]

    def format_prompt_catalog(self) -> str:
        return "\n".join(f"- {t.name}({', '.join(t.parameters)}): {t.description}" for t in self.tools.values())


_GROUP_NETS = (ipaddress.ip_network("224.0.0.0/4"), ipaddress.ip_network("ff00::/8"))  # group-addressed ranges


def is_safe_public_url(url: str, resolve: bool = True) -> bool:
    """Only http(s) URLs whose host resolves exclusively to public addresses: loopback, private, link-local, reserved,
    unspecified and group-addressed targets are refused (server-side request forgery guard)."""
    try:
        u = urlparse(url)
        if u.scheme not in ("http", "https") or not u.hostname:
            return False
        host = u.hostname
        try:
            addrs = [ipaddress.ip_address(host)]
        except ValueError:
            if not resolve:
                return not host.endswith((".local", ".internal", ".localhost")) and host != "localhost"
            addrs = [ipaddress.ip_address(ai[4][0]) for ai in socket.getaddrinfo(host, None)]
        return bool(addrs) and all(a.is_global and not a.is_loopback and not a.is_private and not a.is_link_local
                                   and not a.is_reserved and not a.is_unspecified and not any(a in n for n in _GROUP_NETS if n.version == a.version)
                                   for a in addrs)
    except (OSError, ValueError):
        return False


LOCAL_SERVICE_PORTS = frozenset({11434, *range(8000, 8021)})  # a local Ollama daemon and this framework's own servers


def validate_http_url(url: str, *, allow_local_services: bool = False) -> str:
    """The raising form of ``is_safe_public_url`` (``triune/agents/tools.py:23-62`` of the reference): returns the cleaned
    URL, raises ``ValueError`` for anything that is not a plain http(s) URL with a resolvable host and ``PermissionError``
    when an address it resolves to is not public. ``allow_local_services`` admits loopback on the ports of
    ``LOCAL_SERVICE_PORTS`` only."""
    clean = str(url or "").strip()
    u = urlparse(clean)
    if u.scheme.lower() not in ("http", "https"):
        raise ValueError("Only http:// and https:// URLs are permitted.")
    if u.username or u.password:
        raise ValueError("URLs that carry user credentials are not permitted.")
    if not u.hostname:
        raise ValueError("URL is missing a valid hostname.")
    port = u.port or (443 if u.scheme.lower() == "https" else 80)
    try:
        infos = socket.getaddrinfo(u.hostname, port, type=socket.SOCK_STREAM)
    except socket.gaierror as e:
        raise ValueError(f"Unable to resolve hostname '{u.hostname}': {e}") from e
    if not infos:
        raise ValueError(f"Hostname '{u.hostname}' resolved to no addresses.")
    for info in infos:
        a = ipaddress.ip_address(str(info[4][0]).split("%")[0])
        if a.is_loopback:
            if allow_local_services and port in LOCAL_SERVICE_PORTS:
                continue
            raise PermissionError(f"SSRF guard blocked loopback access to {u.hostname}:{port}.")
        if (not a.is_global or a.is_private or a.is_link_local or a.is_reserved or a.is_unspecified or a.is_multicast
                or any(a in n for n in _GROUP_NETS if n.version == a.version)):
            raise PermissionError(f"SSRF guard blocked non-public IP {a} for host '{u.hostname}'.")
    return clean


def build_integrated_toolbelt() -> ToolRegistry:
    from ..runtime.sandbox import PythonSandbox

    reg = ToolRegistry()
    reg.register(Tool("python", "run Python in the restricted sandbox; set `result`", lambda code: PythonSandbox(5).execute_code(code), {"code": "str"}))
    reg.register(Tool("clock", "current UTC time", lambda: time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())))
    reg.register(Tool("check_url", "whether a URL is a safe public target", lambda url: is_safe_public_url(url, resolve=False), {"url": "str"}))
    return reg


@dataclass
class Persona:
    name: str = "assistant"
    system_prompt: str = "You are a helpful assistant."
    temperature: float = 0.7


class AgentMemory:
    def __init__(self, max_items: int = 256):
        self.items: Dict[str, Any] = {}
        self.max_items = max_items

    def set(self, key: str, value: Any) -> None:
        self.items[key] = value
        while len(self.items) > self.max_items:
            self.items.pop(next(iter(self.items)))

    def get(self, key: str, default=None):
        return self.items.get(key, default)

    def delete(self, key: str) -> bool:
        return self.items.pop(key, None) is not None

    def clear(self) -> None:
        self.items.clear()


_CALL = re.compile(r"<\|tool_call\|>\s*(\{.*?\})\s*(?:$|\n)", re.S)


class Agent:
    def __init__(self, generate: Callable[[str], str], persona: Optional[Persona] = None, tools: Optional[ToolRegistry] = None,
                 memory: Optional[AgentMemory] = None, max_tool_rounds: int = 3):
        self.generate, self.persona = generate, persona or Persona()
        self.tools, self.memory, self.max_tool_rounds = tools or ToolRegistry(), memory or AgentMemory(), max_tool_rounds
        self.transcript: List[Dict[str, str]] = []

    def _prompt(self, user: str) -> str:
        tools = "\n".join(f"- {t['name']}: {t['description']}" for t in self.tools.describe())
        hist = "".join(f"{m['role'].capitalize()}: {m['content']}\n" for m in self.transcript[-8:])
        return f"System: {self.persona.system_prompt}\nTools:\n{tools}\n{hist}User: {user}\nAssistant:"

    def run_task(self, task: str) -> Dict[str, Any]:
        return self.run(task)

    def run(self, user: str) -> Dict[str, Any]:
        calls = []
        prompt = self._prompt(user)
        text = ""
        for _ in range(self.max_tool_rounds + 1):
            text = self.generate(prompt)
            m = _CALL.search(text)
            if not m:
                break
            try:
                req = json.loads(m.group(1))
                result = self.tools.call(req["tool"], **req.get("args", {}))
            except Exception as e:
                result = f"error: {type(e).__name__}: {e}"
            calls.append({"request": m.group(1), "result": result})
            prompt += f"{text}\n<|tool_return|>{json.dumps(result, default=str)}\nAssistant:"
        self.transcript += [{"role": "user", "content": user}, {"role": "assistant", "content": text}]
        return {"text": text, "tool_calls": calls, "persona": self.persona.name}


class MultiAgentOrchestrator:
    def __init__(self, agents: Dict[str, Agent]):
        self.agents = agents

    def run(self, task: str, order: Optional[List[str]] = None) -> List[Dict[str, Any]]:
        out, msg = [], task
        for name in order or list(self.agents):
            r = self.agents[name].run(msg)
            out.append({"agent": name, **r})
            msg = f"{task}\n\nPrevious agent ({name}) said: {r['text']}"
        return out


from .extras import AgentMemoryStore, Provider, ProviderManager, Skill, SkillLibrary  # noqa: E402

__all__ = ["Tool", "ToolRegistry", "build_integrated_toolbelt", "is_safe_public_url", "Persona", "AgentMemory", "Agent", "MultiAgentOrchestrator",
           "AgentMemoryStore", "SkillLibrary", "Skill", "ProviderManager", "Provider"]
