"""Restricted execution of user-supplied Python (DAG "code" nodes, agent tools).

Parity (``triune/runtime/sandbox.py:23-212``): the code is checked against an AST allow-list (no imports outside a
small set, no dunder attribute access, no ``exec`` / ``eval`` / ``open`` / ``__import__``), then run in a child
process with a wall-clock timeout and an address-space limit; results come back as JSON.
"""

from __future__ import annotations

import ast
import json
import os
import subprocess
import sys
import tempfile
import textwrap
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Optional

ALLOWED_IMPORTS = {"math", "json", "re", "random", "statistics", "itertools", "functools", "collections", "datetime", "string",
                   "fractions", "decimal", "heapq", "bisect", "operator", "typing", "dataclasses", "textwrap"}
FORBIDDEN_NAMES = {"exec", "eval", "compile", "open", "__import__", "input", "breakpoint", "globals", "locals", "vars", "getattr",
                   "setattr", "delattr", "memoryview", "exit", "quit", "help"}


class SandboxError(Exception):
    """The code was rejected by validation, timed out or failed."""


@dataclass
class SandboxResult:
    success: bool
    stdout: str = ""
    stderr: str = ""
    result: Any = None
    locals: Dict[str, Any] = field(default_factory=dict)
    error: Optional[str] = None
    timed_out: bool = False

    def to_dict(self) -> Dict[str, Any]:
        return {"success": self.success, "stdout": self.stdout, "stderr": self.stderr, "result": self.result,
                "locals": self.locals, "error": self.error, "timed_out": self.timed_out}


def validate_sandbox_ast(code: str) -> None:
    try:
        tree = ast.parse(code)
    except SyntaxError as e:
        raise SandboxError(f"syntax error: {e}") from e
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name.split(".")[0] not in ALLOWED_IMPORTS:
                    raise SandboxError(f"import of '{a.name}' is not allowed")
        elif isinstance(node, ast.ImportFrom):
            if (node.module or "").split(".")[0] not in ALLOWED_IMPORTS or node.level:
                raise SandboxError(f"import from '{node.module}' is not allowed")
        elif isinstance(node, ast.Attribute) and node.attr.startswith("__"):
            raise SandboxError(f"access to '{node.attr}' is not allowed")
        elif isinstance(node, ast.Name) and (node.id in FORBIDDEN_NAMES or node.id.startswith("__")):
            raise SandboxError(f"use of '{node.id}' is not allowed")
        elif isinstance(node, (ast.Global, ast.Nonlocal)):
            raise SandboxError("global / nonlocal statements are not allowed")


_RUNNER = textwrap.dedent('''
    import json, sys, io, contextlib
    try:
        import resource
        lim = int(sys.argv[2]) * 1024 * 1024
        resource.setrlimit(resource.RLIMIT_AS, (lim, lim))
        resource.setrlimit(resource.RLIMIT_CPU, (int(sys.argv[3]) + 1, int(sys.argv[3]) + 2))
    except Exception:
        pass
    payload = json.load(open(sys.argv[1]))
    env = dict(payload.get("locals") or {})
    out = io.StringIO()
    res = {"success": True, "error": None}
    try:
        with contextlib.redirect_stdout(out):
            exec(compile(payload["code"], "<sandbox>", "exec"), {"__builtins__": __builtins__}, env)
    except BaseException as e:
        res = {"success": False, "error": f"{type(e).__name__}: {e}"}
    def ok(v):
        try:
            json.dumps(v); return True
        except Exception:
            return False
    res["stdout"] = out.getvalue()
    res["locals"] = {k: v for k, v in env.items() if not k.startswith("_") and ok(v)}
    res["result"] = res["locals"].get("result")
    sys.stdout.write("\\n__SANDBOX_JSON__" + json.dumps(res))
''')


class PythonSandbox:
    def __init__(self, timeout: int = 10, max_memory_mb: int = 256):
        self.timeout, self.max_memory_mb = int(timeout), int(max_memory_mb)

    def execute_code(self, code_str: str, locals_dict: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        try:
            validate_sandbox_ast(code_str)
        except SandboxError as e:
            return SandboxResult(False, error=str(e)).to_dict()
        with tempfile.TemporaryDirectory() as d:
            payload, runner = os.path.join(d, "payload.json"), os.path.join(d, "runner.py")
            safe_locals = {}
            for k, v in (locals_dict or {}).items():
                try:
                    json.dumps(v)
                    safe_locals[k] = v
                except (TypeError, ValueError):
                    pass
            json.dump({"code": code_str, "locals": safe_locals}, open(payload, "w"))
            open(runner, "w").write(_RUNNER)
            env = {"PATH": os.environ.get("PATH", ""), "PYTHONIOENCODING": "utf-8"}
            try:
                p = subprocess.run([sys.executable, "-I", "-S", runner, payload, str(self.max_memory_mb), str(self.timeout)],
                                   capture_output=True, text=True, timeout=self.timeout, cwd=d, env=env)
            except subprocess.TimeoutExpired:
                return SandboxResult(False, error=f"timed out after {self.timeout}s", timed_out=True).to_dict()
        marker = "\n__SANDBOX_JSON__"
        if marker not in p.stdout:
            return SandboxResult(False, stdout=p.stdout, stderr=p.stderr[-2000:], error=f"sandbox process failed (exit {p.returncode})").to_dict()
        data = json.loads(p.stdout.rsplit(marker, 1)[1])
        return SandboxResult(bool(data["success"]), data.get("stdout", ""), p.stderr[-2000:], data.get("result"),
                             data.get("locals", {}), data.get("error")).to_dict()

    def execute_function(self, fn: Callable, *args: Any, **kwargs: Any) -> Any:
        """Run a Python function defined in source form: its source goes through the same validation and child process."""
        import inspect

        src = textwrap.dedent(inspect.getsource(fn))
        call = f"\nresult = {fn.__name__}(*_args, **_kwargs)\n"
        code = src + call.replace("_args", "args_").replace("_kwargs", "kwargs_")
        out = self.execute_code(code, {"args_": list(args), "kwargs_": kwargs})
        if not out["success"]:
            raise SandboxError(out["error"] or "sandboxed function failed")
        return out["result"]
