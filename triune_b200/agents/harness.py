"""The agent harness: personas, workspace tools, memory, skills and the loop that ties them to a text generator.

``AgentHarness.run(goal)`` picks a persona (a named one, or by the words of the goal), adds the skills and the
lessons of earlier runs that match the goal to the prompt, lets the agent call tools for a bounded number of rounds,
records which tools worked, keeps a one-line lesson, and, when the run used tools successfully, writes the sequence
down as a markdown skill so that the next similar goal starts with it. The tools work inside one workspace directory
(paths that resolve outside it are refused), writing tools can be left out (``read_only``), a shell tool exists only
when asked for, and the one network tool refuses anything but public http(s) targets.

Counterpart in the reference: ``triune/agents/engine.py:81-540`` (harness and orchestrator), ``personas.py:14-314``,
``tools.py:23-766``, ``skills.py:103-300``, ``memory.py:77-409``. This is a compact version of the same parts; the text
generator is whatever callable the caller provides (the local model, a provider transport, a test double).
"""

from __future__ import annotations

import json
import re
import subprocess
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

from . import Agent, MultiAgentOrchestrator, Persona, Tool, ToolRegistry, build_integrated_toolbelt, is_safe_public_url
from .extras import AgentMemoryStore, Skill, SkillLibrary

MAX_READ_BYTES = 64 * 1024


@dataclass(frozen=True)
class PersonaSpec:
    name: str
    prompt: str
    temperature: float
    keywords: tuple  # words of a goal that point to this persona

    def to_dict(self) -> Dict[str, Any]:
        return {"name": self.name, "system_prompt": self.prompt, "temperature": self.temperature, "keywords": list(self.keywords)}


PERSONAS: Dict[str, PersonaSpec] = {p.name: p for p in (
    PersonaSpec("architect", "You design systems. State the components, their interfaces and the trade-offs before any detail.", 0.5,
                ("design", "architecture", "structure", "plan", "interface", "module", "layout", "refactor")),
    PersonaSpec("engineer", "You write and change code. Make the smallest change that does the job, then say how to check it.", 0.3,
                ("implement", "write", "code", "function", "add", "fix", "build", "script", "file")),
    PersonaSpec("researcher", "You find out and compare. Separate what is measured from what is assumed and cite where each fact comes from.", 0.6,
                ("why", "compare", "survey", "paper", "explain", "evidence", "literature", "study")),
    PersonaSpec("debugger", "You find causes. Reproduce, narrow down, state the cause in one sentence, then the fix.", 0.2,
                ("bug", "error", "crash", "fails", "traceback", "exception", "wrong", "debug", "hang")),
    PersonaSpec("optimizer", "You make things faster or smaller. Measure first, name the bound (compute, memory, latency), change one thing at a time.", 0.3,
                ("fast", "faster", "slow", "speed", "latency", "throughput", "memory", "profile", "optimise", "optimize", "kernel")),
    PersonaSpec("tutor", "You teach. Start from what the learner knows, one idea at a time, with a small worked example.", 0.7,
                ("teach", "learn", "understand", "beginner", "tutorial", "example", "how does")),
    PersonaSpec("sentinel", "You review for safety and correctness. List what can go wrong, how likely, and what guards against it.", 0.2,
                ("security", "safe", "risk", "review", "audit", "vulnerab", "permission", "secret", "leak")),
)}
DEFAULT_PERSONA = PersonaSpec("assistant", "You are a helpful assistant. Be brief and concrete.", 0.7, ())


def choose_persona(goal: str) -> PersonaSpec:
    """The persona whose keywords occur most often in the goal; the general assistant when none occurs."""
    low = goal.lower()
    best, score = DEFAULT_PERSONA, 0
    for p in PERSONAS.values():
        s = sum(len(re.findall(r"\b" + re.escape(k), low)) for k in p.keywords)  # a keyword counts where a word starts with it
        if s > score:
            best, score = p, s
    return best


def resolve_persona(spec: str, goal: str = "") -> Persona:
    """``auto`` (by the goal), a built-in name, or ``name=system prompt`` for one defined on the spot."""
    name, sep, prompt = spec.partition("=")
    name = name.strip()
    if sep:
        return Persona(name or "custom", prompt.strip(), 0.7)
    p = choose_persona(goal) if name in ("", "auto") else PERSONAS.get(name.lower())
    if p is None:
        return Persona(name, f"You are the {name} of the team. Be brief and concrete.", 0.7)
    return Persona(p.name, p.prompt, p.temperature)


# ---------------------------------------------------------------------------------------------------- workspace tools
def _confined(root: Path, rel: str) -> Path:
    p = (root / rel).resolve()
    if p != root and root not in p.parents:
        raise PermissionError(f"{rel!r} is outside the workspace")
    return p


def workspace_tools(workspace: str, read_only: bool = False, allow_shell: bool = False, registry: Optional[ToolRegistry] = None,
                    fetch: Optional[Callable[[str], str]] = None) -> ToolRegistry:
    """File tools confined to ``workspace`` (plus the sandbox, clock and URL check of the basic toolbelt)."""
    root = Path(workspace).resolve()
    root.mkdir(parents=True, exist_ok=True)
    reg = registry if registry is not None else build_integrated_toolbelt()

    def list_dir(path: str = ".") -> List[str]:
        d = _confined(root, path)
        return sorted(f"{c.name}/" if c.is_dir() else c.name for c in d.iterdir())[:500]

    def read_file(path: str, start: int = 0, length: int = MAX_READ_BYTES) -> str:
        f = _confined(root, path)
        with open(f, "rb") as h:
            h.seek(max(0, int(start)))
            return h.read(min(int(length), MAX_READ_BYTES)).decode("utf-8", "replace")

    def search(pattern: str, path: str = ".", max_hits: int = 50) -> List[Dict[str, Any]]:
        rx = re.compile(pattern)
        hits: List[Dict[str, Any]] = []
        base = _confined(root, path)
        files = [base] if base.is_file() else sorted(f for f in base.rglob("*") if f.is_file() and f.stat().st_size <= 2 * 1024 * 1024)
        for f in files:
            try:
                for n, line in enumerate(f.read_text(encoding="utf-8", errors="replace").splitlines(), 1):
                    if rx.search(line):
                        hits.append({"file": str(f.relative_to(root)), "line": n, "text": line[:200]})
                        if len(hits) >= max_hits:
                            return hits
            except OSError:
                continue
        return hits

    def write_file(path: str, content: str) -> str:
        f = _confined(root, path)
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(content, encoding="utf-8")
        return f"wrote {len(content)} characters to {f.relative_to(root)}"

    def append_file(path: str, content: str) -> str:
        f = _confined(root, path)
        f.parent.mkdir(parents=True, exist_ok=True)
        with open(f, "a", encoding="utf-8") as h:
            h.write(content)
        return f"appended {len(content)} characters to {f.relative_to(root)}"

    def edit_file(path: str, old: str, new: str) -> str:
        f = _confined(root, path)
        text = f.read_text(encoding="utf-8")
        if text.count(old) != 1:
            raise ValueError(f"the text to replace occurs {text.count(old)} times; it must occur exactly once")
        f.write_text(text.replace(old, new), encoding="utf-8")
        return f"edited {f.relative_to(root)}"

    def http_get(url: str) -> str:
        if not is_safe_public_url(url):
            raise PermissionError("only public http(s) targets may be fetched")
        if fetch is not None:
            return fetch(url)[:MAX_READ_BYTES]
        import urllib.request

        with urllib.request.urlopen(url, timeout=10) as r:  # noqa: S310 - the URL passed the public-target check above
            return r.read(MAX_READ_BYTES).decode("utf-8", "replace")

    def shell(command: str) -> Dict[str, Any]:
        r = subprocess.run(command, shell=True, cwd=str(root), capture_output=True, text=True, timeout=30)
        return {"exit_code": r.returncode, "stdout": r.stdout[-4000:], "stderr": r.stderr[-2000:]}

    reg.register(Tool("list_dir", "names in a workspace directory", list_dir, {"path": "str"}))
    reg.register(Tool("read_file", "text of a workspace file (at most 64 KB per call)", read_file, {"path": "str", "start": "int", "length": "int"}))
    reg.register(Tool("search", "lines of workspace files that match a regular expression", search, {"pattern": "str", "path": "str"}))
    reg.register(Tool("http_get", "fetch a public http(s) URL", http_get, {"url": "str"}))
    if not read_only:
        reg.register(Tool("write_file", "create or replace a workspace file", write_file, {"path": "str", "content": "str"}))
        reg.register(Tool("append_file", "append to a workspace file", append_file, {"path": "str", "content": "str"}))
        reg.register(Tool("edit_file", "replace one exact occurrence of a text in a workspace file", edit_file, {"path": "str", "old": "str", "new": "str"}))
    if allow_shell and not read_only:
        reg.register(Tool("shell", "run a shell command in the workspace (30 s)", shell, {"command": "str"}))
    return reg


# ---------------------------------------------------------------------------------------------------- harness
class AgentHarness:
    def __init__(self, generate: Callable[[str], str], store_dir: str, workspace: str = ".", persona: str = "auto", read_only: bool = False,
                 allow_shell: bool = False, auto_skill: bool = True, max_steps: int = 3, fetch: Optional[Callable[[str], str]] = None):
        self.generate, self.persona_spec, self.max_steps, self.auto_skill = generate, persona, int(max_steps), auto_skill
        self.store_dir = Path(store_dir)
        self.store_dir.mkdir(parents=True, exist_ok=True)
        self.memory = AgentMemoryStore(str(self.store_dir / "memory.json"))
        self.skill_dir = self.store_dir / "skills"
        self.skill_dir.mkdir(exist_ok=True)
        self.skills = SkillLibrary(str(self.skill_dir))
        self.tools = workspace_tools(workspace, read_only, allow_shell, fetch=fetch)

    def _context(self, goal: str) -> str:
        parts = []
        block = self.skills.prompt_block(goal)
        if block:
            parts.append(block)
        lessons = self.memory.recall(goal, k=3)
        if lessons:
            parts.append("Notes from earlier runs:\n" + "\n".join(f"- {t}" for _, t in lessons))
        prefs = self.memory.data.get("preferences") or {}
        if prefs:
            parts.append("User preferences: " + "; ".join(f"{k} = {v}" for k, v in sorted(prefs.items())))
        return ("\n\n" + "\n\n".join(parts)) if parts else ""

    def run(self, goal: str, persona: Optional[str] = None) -> Dict[str, Any]:
        pers = resolve_persona(persona or self.persona_spec, goal)
        agent = Agent(self.generate, pers, self.tools, max_tool_rounds=self.max_steps)
        t0 = time.time()
        out = agent.run(goal + self._context(goal))
        ok_calls = []
        for c in out["tool_calls"]:
            failed = isinstance(c["result"], str) and c["result"].startswith("error:")
            try:
                name = json.loads(c["request"]).get("tool", "?")
            except ValueError:
                name = "?"
            self.memory.record_tool(name, not failed)
            if not failed:
                ok_calls.append(name)
        self.memory.add_lesson(f"goal: {goal[:160]} -> {str(out['text'])[:300]}", tags=[pers.name])
        skill = self._synthesise_skill(goal, ok_calls) if self.auto_skill and ok_calls else None
        self.memory.save()
        return {**out, "seconds": time.time() - t0, "new_skill": skill, "tools_offered": sorted(self.tools.tools)}

    def run_goal(self, goal: str, persona: Optional[str] = None) -> Dict[str, Any]:
        return self.run(goal, persona)

    def _synthesise_skill(self, goal: str, calls: List[str]) -> Optional[str]:
        """Write the tool sequence that served this goal down as a skill (one file per distinct sequence)."""
        words = [w for w in re.findall(r"[a-z0-9]+", goal.lower()) if len(w) > 3][:4]
        if not words:
            return None
        name = "-".join(["use"] + list(dict.fromkeys(calls))[:3] + ["for"] + words[:2])
        path = self.skill_dir / f"{name}.md"
        if path.exists():
            return None
        steps = "\n".join(f"{i}. call `{c}`" for i, c in enumerate(calls, 1))
        text = (f"---\nname: {name}\ndescription: tool sequence that served the goal \"{goal[:100]}\"\ntriggers: {', '.join(words)}\n---\n"
                f"For goals like this one the following worked:\n{steps}\n")
        path.write_text(text, encoding="utf-8")
        self.skills.add(SkillLibrary.parse(text, str(path)))
        return name

    def run_team(self, goal: str, personas: List[str]) -> List[Dict[str, Any]]:
        """The goal passes through the personas in turn, each seeing the previous answer; they share tools and context."""
        agents = {n: Agent(self.generate, resolve_persona(n, goal), self.tools, max_tool_rounds=self.max_steps) for n in personas}
        out = MultiAgentOrchestrator(agents).run(goal + self._context(goal), personas)
        self.memory.add_lesson(f"goal: {goal[:160]} -> {str(out[-1]['text'])[:300]}", tags=["team"] + personas)
        self.memory.save()
        return out


__all__ = ["PERSONAS", "PersonaSpec", "choose_persona", "resolve_persona", "workspace_tools", "AgentHarness", "Skill"]
