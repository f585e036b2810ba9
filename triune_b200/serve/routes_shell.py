"""Product-shell routes: thin HTTP fronts for components that live elsewhere in the package.

Model discovery (``runtime/model_scanner.py``), the DAG executor and its node catalogue (``execution/dag.py``), plugins
(``plugins/registry.py``), agents (``agents``), checkpoint housekeeping, dataset registration, kernel benchmarks and the
in-process tuning knobs. None of these does GPU work of its own. Counterparts in the reference: the route decorators of
``triune/api/routes.py:3239-8346`` outside the chat / training core (``/v1/models/scan``, ``/v1/system/*``, ``/v1/dag/*``,
``/v1/nodes/catalog``, ``/v1/plugins*``, ``/v1/modules/*``, ``/v1/agents/*``, ``/v1/checkpoints/{delete,export,projects,assign_project,prune_project}``,
``/v1/datasets*``, ``/v1/engine/{benchmarks,turbo_mode}``, ``/v1/hardware/{tune,autotune}``, ``/v1/training/{optimizer,export}``,
``/v1/byok/*``, ``/v1/finetune/export``, ``/v1/models/{upgrade_to_triune,distill}``). Endpoints whose job is to reach the internet (module search / clone, provider proxying) answer with
what can be known locally and say so.
"""

from __future__ import annotations

import asyncio
import os
import time
from pathlib import Path
from typing import Any, Dict, List, Optional

from fastapi import APIRouter, HTTPException

from .engine_state import get_state

shell_router = APIRouter()

# Process-wide shell state: small, in memory, reset with the process.
_SHELL: Dict[str, Any] = {
    "config": {"default_checkpoint_dir": "checkpoints_full", "plugin_dir": "plugins", "turbo_mode": False},
    "datasets": {}, "selected_dataset": None, "byok": {}, "registry": None, "agents": None,
}

# Environment switches that change which kernel variant a launch picks (read at launch time by the extension).
TUNING_KNOBS = ("TRIUNE_GEMM_BN", "TRIUNE_GEMM_PAIR", "TRIUNE_GEMM_PAIR_MIN_K", "TRIUNE_GEMM_MAX_SPLITS")


def _bad(e: Exception, code: int = 400):
    return HTTPException(code, f"{type(e).__name__}: {e}")


def _registry():
    if _SHELL["registry"] is None:
        from ..plugins.registry import PluginRegistry

        _SHELL["registry"] = PluginRegistry()
    return _SHELL["registry"]


def _inside(directory: str, name: str) -> Path:
    """``directory/name`` resolved, refused unless it stays inside ``directory``."""
    root = Path(directory).resolve()
    p = (root / name).resolve()
    if root != p.parent and root not in p.parents:
        raise ValueError("path escapes the directory")
    return p


# ---------------------------------------------------------------------------------------------------- discovery, config
@shell_router.get("/v1/models/scan")
@shell_router.get("/v1/system/scan")
async def models_scan(roots: Optional[str] = None, max_depth: int = 4):
    from ..runtime.model_scanner import scan_models

    return await asyncio.to_thread(scan_models, roots.split(os.pathsep) if roots else None, max_depth)


@shell_router.get("/v1/system/config")
async def system_config_get():
    return {"config": dict(_SHELL["config"]), "tuning": {k: os.environ.get(k) for k in TUNING_KNOBS}}


@shell_router.post("/v1/system/config")
async def system_config_set(body: Dict[str, Any]):
    unknown = sorted(set(body) - set(_SHELL["config"]))
    if unknown:
        raise HTTPException(400, f"unknown configuration keys: {unknown}")
    _SHELL["config"].update(body)
    return {"config": dict(_SHELL["config"])}


# ---------------------------------------------------------------------------------------------------- DAG, nodes, plugins
@shell_router.get("/v1/nodes/catalog")
async def nodes_catalog():
    """``nodes``: this executor's own node types; ``studio_nodes``: the canvas catalogue (typed ports, default parameters)."""
    from ..execution.dag import node_catalog
    from ..execution.studio import studio_catalog

    return {"nodes": node_catalog(), "studio_nodes": studio_catalog()}


# One graph runs at a time against the shared model / training state; the others wait (``/v1/dag/queue`` shows both).
_DAG_QUEUE: Dict[str, Any] = {"active_run_id": None, "waiting": 0, "lock": None}


def _dag_lock() -> asyncio.Lock:
    if _DAG_QUEUE["lock"] is None:
        _DAG_QUEUE["lock"] = asyncio.Lock()
    return _DAG_QUEUE["lock"]


@shell_router.get("/v1/dag/queue")
async def dag_queue():
    return {"active_run_id": _DAG_QUEUE["active_run_id"], "waiting": _DAG_QUEUE["waiting"], "capacity": 1}


@shell_router.post("/v1/dag/execute")
async def dag_execute(body: Dict[str, Any]):
    """Both graph formats: the canvas' (``nodes`` / ``edges`` with ``source`` and ``target``, optional ``run_id``; node
    events go to the telemetry listeners as ``dag_event`` records) and this executor's own (``{"dag": ...}``)."""
    import uuid

    from ..execution.dag import DAGValidationError, execute_dag
    from ..execution.studio import StudioGraphError, is_studio_graph, run_studio_graph

    spec = body.get("dag", body)
    state = get_state()
    run_id = str(body.get("run_id") or uuid.uuid4().hex)[:80]
    _DAG_QUEUE["waiting"] += 1
    t_queue = time.perf_counter()
    acquired = False
    try:
        async with _dag_lock():
            acquired = True
            _DAG_QUEUE["waiting"] -= 1
            _DAG_QUEUE["active_run_id"] = run_id
            waited_ms = round((time.perf_counter() - t_queue) * 1000, 1)
            try:
                if is_studio_graph(spec):
                    def emit(ev):
                        state._broadcast({"type": "dag_event", "data": {**ev, "run_id": run_id}})

                    ctx = {"state": state, "provider_keys": _SHELL["byok"]}
                    out = await asyncio.to_thread(run_studio_graph, {"nodes": spec.get("nodes", []), "edges": spec.get("edges", [])}, ctx, emit)
                    out.update(run_id=run_id, queue_wait_ms=waited_ms)
                    return _jsonable(out)
                out = await asyncio.to_thread(execute_dag, spec, {"state": state})
            finally:
                _DAG_QUEUE["active_run_id"] = None
    except (DAGValidationError, StudioGraphError) as e:
        raise _bad(e, 422)
    except HTTPException:
        raise
    except Exception as e:
        raise _bad(e)
    finally:
        if not acquired:  # cancelled while waiting for its turn
            _DAG_QUEUE["waiting"] = max(0, _DAG_QUEUE["waiting"] - 1)
    return _jsonable(out)


@shell_router.post("/v1/dag/compile_to_training")
@shell_router.post("/v1/model/compile_dag")
async def dag_compile_to_training(body: Dict[str, Any]):
    """Read a canvas graph as a training recipe and apply it: a model node rebuilds the active model when it names an
    architecture (``apply_model`` false keeps the loaded one), the rest becomes the configuration of the next training run."""
    from ..execution.studio import StudioGraphError, compile_to_training

    try:
        rec = compile_to_training({"nodes": body.get("nodes", []), "edges": body.get("edges", [])})
    except StudioGraphError as e:
        raise _bad(e, 422)
    state = get_state()
    applied: Dict[str, Any] = {}
    arch = {k: v for k, v in rec["model"].items() if k != "preset"}
    if (arch or rec["model"].get("preset")) and body.get("apply_model", True):
        if state.train_status.get("running"):
            raise HTTPException(409, "pause background training before changing the architecture")
        if arch.get("hidden_dim") and arch.get("num_heads") and "head_dim" not in arch:
            arch["head_dim"] = arch["hidden_dim"] // arch["num_heads"]
        try:
            if arch.get("num_layers"):
                from ..execution.studio import shallow_exit_layout

                arch = {**shallow_exit_layout(arch["num_layers"]), **arch}
            applied["model_architecture"] = await asyncio.to_thread(state.load_model, rec["model"].get("preset", "default"),
                                                                    None, rec["run"].get("precision"), **arch)
        except Exception as e:
            raise _bad(e)
    run = {k: v for k, v in rec["run"].items() if k != "precision"}
    if run:
        _SHELL["config"].setdefault("training", {}).update(run)
        state.pending_training_config = {**getattr(state, "pending_training_config", {}), **run}
        state.trainer = None  # the next step or run builds its trainer from the new settings
        applied["training"] = run
    if rec["data"]:
        _SHELL["selected_dataset"] = rec["data"].get("path") or rec["data"].get("source")
        applied["data"] = rec["data"]
    return {"status": "compiled", "applied": applied, "sections": rec["applied"]}


@shell_router.post("/v1/dag/execute_node")
async def dag_execute_node(body: Dict[str, Any]):
    """One node on its own. Canvas form: the node object itself (``type`` / ``title`` / ``params`` ...), optional
    ``inputs``. Own form: ``{"type": ..., "params": {...}, "inputs": {port: value}}``; inputs become constant nodes."""
    from ..execution.dag import NODE_TYPES, execute_dag
    from ..execution.studio import resolve_kind, run_studio_node

    node = body.get("node") if isinstance(body.get("node"), dict) else body
    if node.get("type") not in NODE_TYPES and resolve_kind(node) is not None:
        state = get_state()
        try:
            out = await asyncio.to_thread(run_studio_node, {k: v for k, v in node.items() if k != "inputs"}, body.get("inputs") or node.get("inputs"),
                                          {"state": state, "provider_keys": _SHELL["byok"]})
        except Exception as e:
            raise _bad(e)
        return _jsonable(out)
    try:
        nodes = [{"id": "n", "type": body["type"], "params": body.get("params", {})}]
        edges = []
        for i, (port, value) in enumerate(sorted((body.get("inputs") or {}).items())):
            nodes.append({"id": f"in{i}", "type": "constant", "params": {"value": value}})
            edges.append({"from": f"in{i}.out", "to": f"n.{port}"})
        out = await asyncio.to_thread(execute_dag, {"nodes": nodes, "edges": edges}, {"state": get_state()})
    except Exception as e:
        raise _bad(e)
    mine = {k.split(".", 1)[1]: v for k, v in out["outputs"].items() if k.startswith("n.")}
    return {"outputs": _jsonable(mine), "seconds": out["timings"].get("n")}


@shell_router.get("/v1/plugins")
@shell_router.get("/v1/modules/installed")
async def plugins_list():
    return {"plugins": _registry().list()}


@shell_router.get("/v1/plugins/nodes")
async def plugins_nodes():
    return {"nodes": sorted(n for p in _registry().list() for n in p["nodes"])}


@shell_router.post("/v1/modules/scan_local")
async def modules_scan_local(body: Dict[str, Any]):
    d = str(body.get("directory") or _SHELL["config"]["plugin_dir"])
    if not Path(d).is_dir():
        raise HTTPException(404, f"no such directory: {d}")
    return {"found": [p.name for p in _registry().discover(d)], "plugins": _registry().list()}


@shell_router.post("/v1/modules/activate")
async def modules_activate(body: Dict[str, Any]):
    from ..plugins.registry import PluginError

    try:
        info = _registry().load(str(body["name"]))
    except (PluginError, KeyError) as e:
        raise _bad(e, 403 if isinstance(e, PluginError) else 400)
    return {"name": info.name, "loaded": info.loaded, "nodes": info.nodes}


@shell_router.post("/v1/modules/create_plugin")
async def modules_create_plugin(body: Dict[str, Any]):
    from ..plugins.registry import PluginError, create_plugin

    d = str(body.get("directory") or _SHELL["config"]["plugin_dir"])
    try:
        path = create_plugin(d, str(body.get("name", "")))
    except PluginError as e:
        raise _bad(e)
    _registry().discover(d)
    return {"created": str(path), "plugins": _registry().list()}


def _local_source(src: str) -> Optional[Path]:
    """A module source this server can reach: a local directory or a ``file://`` URL. Remote URLs return None."""
    if src.startswith("builtin://"):  # a module that ships with the framework
        from ..plugins.curated import curated_path

        try:
            return curated_path(src[len("builtin://"):])
        except KeyError:
            return None
    if src.startswith("file://"):
        src = src[len("file://"):]
    if "://" in src or src.startswith("git@"):
        return None
    p = Path(src).expanduser()
    return p if p.is_dir() else None


_NO_NETWORK = "remote repositories need network access, which this server does not use; give a local directory or a file:// URL"


@shell_router.post("/v1/modules/install")
@shell_router.post("/v1/modules/clone")
async def modules_install(body: Dict[str, Any]):
    """Copy a module (a plugin directory with its signed manifest, or a local git repository, cloned with ``git``) into
    the plugin directory and register what it holds. Nothing is loaded until ``/v1/modules/activate``."""
    import shutil
    import subprocess

    src = str(body.get("download_url") or body.get("url") or body.get("repo_url") or body.get("path") or body.get("source") or "")
    root = _local_source(src)
    if root is None:
        raise HTTPException(400 if not src else 501, "a module source is required" if not src else _NO_NETWORK)
    name = str(body.get("name") or root.name)
    try:
        dst = _inside(str(_SHELL["config"]["plugin_dir"]), name)
    except ValueError as e:
        raise _bad(e, 403)
    if dst.exists():
        raise HTTPException(409, f"module {name!r} is already installed")
    dst.parent.mkdir(parents=True, exist_ok=True)
    if (root / ".git").exists():
        cmd = ["git", "clone", "--quiet", "--depth", "1"] + (["--branch", str(body["branch"])] if body.get("branch") else []) + [str(root), str(dst)]
        r = await asyncio.to_thread(subprocess.run, cmd, capture_output=True, text=True, timeout=120)
        if r.returncode != 0:
            raise HTTPException(400, f"git clone failed: {r.stderr.strip()[:300]}")
    else:
        await asyncio.to_thread(shutil.copytree, root, dst)
    found = _registry().discover(str(dst.parent))
    return {"status": "installed", "id": name, "path": str(dst), "is_git": (dst / ".git").exists(),
            "plugins_found": [p.name for p in found if Path(p.path).resolve().is_relative_to(dst.resolve())]}


@shell_router.post("/v1/modules/pull")
async def modules_pull(body: Dict[str, Any]):
    """``git pull`` in an installed module that is a clone of a local repository."""
    import subprocess

    name = str(body.get("id") or body.get("module_id") or body.get("name") or "")
    try:
        dst = _inside(str(_SHELL["config"]["plugin_dir"]), name)
    except ValueError as e:
        raise _bad(e, 403)
    if not name or not (dst / ".git").exists():
        raise HTTPException(404, f"no git module {name!r} is installed")
    url = await asyncio.to_thread(subprocess.run, ["git", "-C", str(dst), "config", "--get", "remote.origin.url"], capture_output=True, text=True)
    if _local_source(url.stdout.strip()) is None:
        raise HTTPException(501, _NO_NETWORK)
    r = await asyncio.to_thread(subprocess.run, ["git", "-C", str(dst), "pull", "--quiet", "--ff-only"], capture_output=True, text=True, timeout=120)
    if r.returncode != 0:
        raise HTTPException(400, f"git pull failed: {r.stderr.strip()[:300]}")
    head = await asyncio.to_thread(subprocess.run, ["git", "-C", str(dst), "rev-parse", "--short", "HEAD"], capture_output=True, text=True)
    return {"status": "updated", "id": name, "head": head.stdout.strip()}


@shell_router.post("/v1/modules/uninstall")
async def modules_uninstall(body: Dict[str, Any]):
    import shutil

    name = str(body.get("id") or body.get("name") or "")
    try:
        dst = _inside(str(_SHELL["config"]["plugin_dir"]), name)
    except ValueError as e:
        raise _bad(e, 403)
    if not name or not dst.is_dir():
        raise HTTPException(404, f"module {name!r} is not installed")
    await asyncio.to_thread(shutil.rmtree, dst)
    _SHELL["registry"] = None  # forget what was discovered there; the next listing rescans
    return {"status": "uninstalled", "id": name}


@shell_router.get("/v1/modules/search")
async def modules_search(q: str = "", source: str = "all"):
    """The modules that ship with the framework (installable from ``builtin://<id>``) that match ``q``."""
    from ..plugins.curated import CURATED

    ql = q.lower()
    hits = [dict(c, source="curated") for c in CURATED if not ql or ql in (c["id"] + " " + c["name"] + " " + c["description"]).lower()]
    return {"results": hits, "curated": hits, "github": [], "huggingface": [],
            "note": "remote module catalogues need network access, which this server does not use"}


@shell_router.get("/v1/modules/updates")
async def modules_remote():
    return {"results": [], "note": "remote module catalogues need network access, which this server does not use"}


def _jsonable(x: Any, depth: int = 0) -> Any:
    """Tensors and other rich values become short descriptions so that any DAG output can be returned as JSON."""
    if depth > 6:
        return repr(x)[:200]
    if isinstance(x, (str, int, float, bool)) or x is None:
        return x
    if isinstance(x, dict):
        return {str(k): _jsonable(v, depth + 1) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v, depth + 1) for v in x]
    shape = getattr(x, "shape", None)
    if shape is not None and hasattr(x, "dtype"):
        return {"tensor": list(shape), "dtype": str(x.dtype)}
    return repr(x)[:200]


# ---------------------------------------------------------------------------------------------------- agents
def _agents() -> Dict[str, Any]:
    if _SHELL["agents"] is None:
        from ..agents import AgentMemory, Persona, build_integrated_toolbelt

        _SHELL["agents"] = {"memory": AgentMemory(), "persona": Persona(), "tools": build_integrated_toolbelt(), "runs": 0}
    return _SHELL["agents"]


def _agent(persona=None, max_tokens: int = 256):
    from ..agents import Agent

    a, st = _agents(), get_state()
    pers = persona or a["persona"]

    def generate(prompt: str) -> str:
        return st.generate(prompt, max_new_tokens=max_tokens, temperature=pers.temperature, template=False)["text"]

    return Agent(generate, pers, a["tools"], a["memory"])


@shell_router.get("/v1/agents/state")
async def agents_state():
    a = _agents()
    return {"persona": vars(a["persona"]), "tools": a["tools"].describe(), "memory_items": len(a["memory"].items), "runs": a["runs"]}


@shell_router.get("/v1/agents/memory")
async def agents_memory_get():
    return {"items": _jsonable(_agents()["memory"].items)}


@shell_router.post("/v1/agents/memory")
async def agents_memory_set(body: Dict[str, Any]):
    mem = _agents()["memory"]
    if body.get("clear"):
        mem.clear()
    for k in body.get("delete", []):
        mem.delete(str(k))
    for k, v in (body.get("set") or {}).items():
        mem.set(str(k), v)
    return {"items": _jsonable(mem.items)}


@shell_router.post("/v1/agents/persona")
async def agents_persona(body: Dict[str, Any]):
    from ..agents import Persona

    cur = _agents()["persona"]
    _agents()["persona"] = Persona(str(body.get("name", cur.name)), str(body.get("system_prompt", cur.system_prompt)),
                                   float(body.get("temperature", cur.temperature)))
    return {"persona": vars(_agents()["persona"])}


@shell_router.post("/v1/agents/run")
async def agents_run(body: Dict[str, Any]):
    """``{"message": ...}`` runs the session agent (its persona and in-memory notes). With ``"harness": true`` (or a
    ``persona`` / ``team`` / ``workspace`` key) the goal goes through the agent harness instead: persona by name or by the
    goal's words, file tools confined to ``workspace`` (read-only unless ``allow_write``), skills and lessons kept under
    ``store_dir`` between runs. The shell tool is never offered over HTTP."""
    goal = str(body.get("message") or body.get("goal") or "")
    try:
        st = get_state()
        st.require_model()
        if body.get("harness") or any(k in body for k in ("persona", "team", "workspace")):
            from ..agents.harness import AgentHarness

            max_tokens = int(body.get("max_tokens", 256))

            def generate(prompt: str) -> str:
                return st.generate(prompt, max_new_tokens=max_tokens, temperature=float(body.get("temperature", 0.7)), template=False)["text"]

            h = AgentHarness(generate, str(body.get("store_dir") or "checkpoints/agent_harness"), workspace=str(body.get("workspace") or "."),
                             persona=str(body.get("persona") or "auto"), read_only=not bool(body.get("allow_write", False)), allow_shell=False,
                             auto_skill=bool(body.get("auto_skill", True)), max_steps=int(body.get("max_steps", 3)))
            team = body.get("team")
            out = await asyncio.to_thread(h.run_team, goal, [str(t) for t in team]) if team else await asyncio.to_thread(h.run, goal)
            out = {"steps": out} if team else out
        else:
            out = await asyncio.to_thread(_agent(max_tokens=int(body.get("max_tokens", 256))).run, goal)
    except RuntimeError as e:
        raise _bad(e, 409)
    _agents()["runs"] += 1
    return _jsonable(out)


@shell_router.post("/v1/agents/orchestrate")
async def agents_orchestrate(body: Dict[str, Any]):
    """``{"task": ..., "agents": [{"name", "system_prompt"}...]}``: the agents answer in turn, each seeing the previous one."""
    from ..agents import MultiAgentOrchestrator, Persona

    specs = body.get("agents") or [{"name": "planner", "system_prompt": "Break the task into steps."},
                                   {"name": "worker", "system_prompt": "Carry out the steps and answer."}]
    try:
        get_state().require_model()
        team = {str(s["name"]): _agent(Persona(str(s["name"]), str(s.get("system_prompt", "")), float(s.get("temperature", 0.7))),
                                       int(body.get("max_tokens", 256))) for s in specs}
        out = await asyncio.to_thread(MultiAgentOrchestrator(team).run, str(body.get("task", "")))
    except RuntimeError as e:
        raise _bad(e, 409)
    return {"steps": _jsonable(out)}


# ---------------------------------------------------------------------------------------------------- checkpoints, export
@shell_router.post("/v1/checkpoints/delete")
async def checkpoints_delete(body: Dict[str, Any]):
    d = str(body.get("directory") or _SHELL["config"]["default_checkpoint_dir"])
    try:
        p = _inside(d, str(body["name"]))
    except (KeyError, ValueError) as e:
        raise _bad(e)
    if p.suffix != ".pt" or not p.is_file():
        raise HTTPException(404, f"no checkpoint {p.name!r} in {d}")
    p.unlink()
    return {"deleted": str(p), "checkpoints": get_state().list_checkpoints(d)}


def _projects(d: str) -> Dict[str, List[str]]:
    import json as _json

    f = Path(d) / "projects.json"
    try:
        return dict(_json.loads(f.read_text()).get("projects", {})) if f.is_file() else {}
    except ValueError:
        return {}


def _save_projects(d: str, projects: Dict[str, List[str]]) -> None:
    import json as _json

    Path(d).mkdir(parents=True, exist_ok=True)
    tmp = Path(d) / "projects.json.tmp"
    tmp.write_text(_json.dumps({"projects": projects}, indent=2))
    os.replace(tmp, Path(d) / "projects.json")


@shell_router.get("/v1/checkpoints/projects")
async def checkpoints_projects(directory: Optional[str] = None):
    """Checkpoints grouped by project (a JSON side file in the checkpoint directory); unassigned ones come last."""
    d = directory or _SHELL["config"]["default_checkpoint_dir"]
    have = {c["name"]: c for c in get_state().list_checkpoints(d)}
    projects = {p: [have[n] for n in names if n in have] for p, names in _projects(d).items()}
    taken = {n for names in _projects(d).values() for n in names}
    return {"projects": projects, "unassigned": [c for n, c in have.items() if n not in taken]}


@shell_router.post("/v1/checkpoints/assign_project")
async def checkpoints_assign(body: Dict[str, Any]):
    d = str(body.get("directory") or _SHELL["config"]["default_checkpoint_dir"])
    try:
        name, project = _inside(d, str(body["name"])).name, str(body["project"]).strip()
    except (KeyError, ValueError) as e:
        raise _bad(e)
    if not project or not (Path(d) / name).is_file():
        raise HTTPException(404, f"no checkpoint {name!r} in {d}, or empty project name")
    projects = {p: [n for n in names if n != name] for p, names in _projects(d).items()}
    projects.setdefault(project, []).append(name)
    _save_projects(d, {p: v for p, v in projects.items() if v})
    return {"project": project, "checkpoints": projects[project]}


@shell_router.post("/v1/checkpoints/prune_project")
async def checkpoints_prune(body: Dict[str, Any]):
    """Keep the ``keep`` newest checkpoints of a project and delete the rest of that project's files."""
    d = str(body.get("directory") or _SHELL["config"]["default_checkpoint_dir"])
    project, keep = str(body.get("project", "")), max(1, int(body.get("keep", 3)))
    projects = _projects(d)
    if project not in projects:
        raise HTTPException(404, f"unknown project {project!r}")
    files = sorted((p for p in (_inside(d, n) for n in projects[project]) if p.is_file() and p.suffix == ".pt"),
                   key=lambda p: -p.stat().st_mtime)
    for p in files[keep:]:
        p.unlink()
    projects[project] = [p.name for p in files[:keep]]
    _save_projects(d, projects)
    return {"project": project, "kept": projects[project], "deleted": [p.name for p in files[keep:]]}


@shell_router.post("/v1/checkpoints/export")
@shell_router.post("/v1/training/export")
async def checkpoints_export(body: Dict[str, Any]):
    """Write the loaded model as ``format`` (safetensors, hf or pt) to ``path``."""
    from ..export.exporter import export_model

    try:
        model = get_state().require_model()
        out = await asyncio.to_thread(export_model, model, str(body["path"]), str(body.get("format", "safetensors")))
    except RuntimeError as e:
        raise _bad(e, 409)
    except Exception as e:
        raise _bad(e)
    return {"path": str(out), "format": body.get("format", "safetensors")}


@shell_router.post("/v1/finetune/export")
async def finetune_export(body: Dict[str, Any]):
    """Re-write a saved adapter as one ``safetensors`` (or ``pt``) file."""
    from ..trainer.finetune import export_adapter

    try:
        out = await asyncio.to_thread(export_adapter, str(body["adapter_path"]), body.get("output_path"), str(body.get("format", "safetensors")))
    except (KeyError, FileNotFoundError) as e:
        raise _bad(e, 404 if isinstance(e, FileNotFoundError) else 400)
    return {"path": str(out)}


@shell_router.post("/v1/models/upgrade_to_triune")
@shell_router.post("/v1/models/distill")
async def models_upgrade(body: Dict[str, Any]):
    """Turn a local Hugging Face causal LM into a Triune model: ``mode="exits"`` attaches early exits to it,
    ``mode="native"`` transfers its weights into a native multi-exit MoE student. Local files only."""
    from ..models.transmuter import transfer_weights_to_native_triune, transmute_hf_to_triune

    src = str(body.get("source", ""))
    if not src or not Path(src).exists():
        raise HTTPException(404, f"no local model at {src!r} (this server downloads nothing)")

    def work():
        import torch

        if str(body.get("mode", "exits")) == "exits":
            model, meta = transmute_hf_to_triune(src, reflex_ratio=float(body.get("reflex_ratio", 0.25)), rank=int(body.get("rank", 64)),
                                                 use_jev=bool(body.get("use_jev", True)), device=get_state().device, local_files_only=True)
        else:
            from transformers import AutoModelForCausalLM

            teacher = AutoModelForCausalLM.from_pretrained(src, local_files_only=True)
            model, meta = transfer_weights_to_native_triune(teacher, num_experts=int(body.get("experts", 8)), top_k=int(body.get("top_k", 2)),
                                                            target_layers=body.get("layers"), target_dim=body.get("dim"),
                                                            reflex_ratio=float(body.get("reflex_ratio", 0.25)))
        if body.get("output"):
            Path(str(body["output"])).parent.mkdir(parents=True, exist_ok=True)
            torch.save({"model_state": model.state_dict(), "config": {}, "transmute": meta}, str(body["output"]))
            meta["saved_to"] = str(body["output"])
        return meta

    try:
        return _jsonable(await asyncio.to_thread(work))
    except Exception as e:
        raise _bad(e)


@shell_router.post("/v1/training/optimizer")
async def training_optimizer(body: Dict[str, Any]):
    """Change hyper-parameters of the live optimizer (``lr``, ``weight_decay``) without rebuilding it."""
    tr = get_state().trainer
    if tr is None:
        raise HTTPException(409, "no training run exists; POST /v1/training/start or /v1/training/step first")
    changed = {}
    for group in tr.optimizer.param_groups:
        for key in ("lr", "weight_decay"):
            if key in body and key in group:
                group[key] = float(body[key])
                changed[key] = float(body[key])
    return {"changed": changed, "groups": len(tr.optimizer.param_groups)}


# ---------------------------------------------------------------------------------------------------- datasets
@shell_router.get("/v1/datasets")
async def datasets_list():
    return {"datasets": list(_SHELL["datasets"].values()), "selected": _SHELL["selected_dataset"]}


@shell_router.post("/v1/datasets/local/register")
async def datasets_register(body: Dict[str, Any]):
    p = Path(str(body.get("path", "")))
    if not p.exists():
        raise HTTPException(404, f"no such file or directory: {p}")
    files = [p] if p.is_file() else sorted(f for f in p.rglob("*") if f.suffix in (".jsonl", ".txt", ".parquet"))
    if not files:
        raise HTTPException(400, "no .jsonl, .txt or .parquet files there")
    name = str(body.get("name") or p.stem)
    _SHELL["datasets"][name] = {"name": name, "path": str(p), "files": len(files), "bytes": sum(f.stat().st_size for f in files),
                                "registered": time.time()}
    return _SHELL["datasets"][name]


@shell_router.post("/v1/datasets/select")
async def datasets_select(body: Dict[str, Any]):
    name = str(body.get("name", ""))
    if name not in _SHELL["datasets"]:
        raise HTTPException(404, f"unknown dataset {name!r}")
    _SHELL["selected_dataset"] = name
    return {"selected": name, "train_config": {"dataset_path": _SHELL["datasets"][name]["path"]}}


@shell_router.post("/v1/datasets/stream/connect")
async def datasets_stream_connect(body: Dict[str, Any]):
    """Make a dataset the active training stream. A local file or directory (or a ``file://`` URL, or a hub name that
    exists as a local path) is read and registered; anything that needs the network answers ``status: error``."""
    from ..execution.studio import _read_local_texts

    name = str(body.get("dataset_name") or body.get("url") or "").strip()
    if not name:
        return {"status": "error", "message": "Dataset identifier or URL cannot be empty."}
    local = name[len("file://"):] if name.startswith("file://") else (str(body.get("local_path") or "") or name)
    if "://" in local or not os.path.exists(local):
        return {"status": "error", "message": f"Could not stream from '{name}': remote hubs and URLs need network access, which this "
                                              f"server does not use (give a local path, a file:// URL or 'local_path')"}
    docs = await asyncio.to_thread(_read_local_texts, local, 20)
    if not docs:
        return {"status": "error", "message": f"'{local}' holds no text"}
    _SHELL["stream"] = {"is_streaming": True, "dataset_name": name, "dataset_type": "local", "path": local, "split": body.get("split", "train"),
                        "text_column": body.get("text_column", "text"), "buffered_chunks": len(docs), "connected": time.time()}
    _SHELL["selected_dataset"] = local
    return {"status": "connected", "dataset_name": name, "buffered_chunks": len(docs), "sample_preview": docs[0][:200],
            "train_config": {"dataset_path": local}}


@shell_router.get("/v1/datasets/stream/status")
async def datasets_stream_status():
    st = _SHELL.get("stream")
    if st:
        return dict(st)
    return {"is_streaming": False, "connected": False,
            "note": "no stream is connected; remote hubs need network access, which this server does not use"}


# ---------------------------------------------------------------------------------------------------- engine, hardware
@shell_router.post("/v1/engine/turbo_mode")
async def engine_turbo(body: Dict[str, Any]):
    """Turbo mode: greedy requests (temperature 0, repetition penalty 1, no session, no streaming) decode through the
    graph-replayed decoder (pure arg-max: no repetition or count penalty); every other request keeps the sampling path."""
    st = get_state()
    st.turbo_mode = bool(body.get("enabled", True))
    _SHELL["config"]["turbo_mode"] = st.turbo_mode
    return {"turbo_mode": st.turbo_mode}


@shell_router.get("/v1/engine/benchmarks")
async def engine_benchmarks():
    """What can be measured from here, and the peaks measurements are compared against."""
    from .. import bench_kernels

    return {"cases": sorted(bench_kernels.CASES), "peaks": bench_kernels.peaks(),
            "how": "POST /v1/engine/benchmarks {\"case\": name, ...sizes} runs one case on the server's GPU"}


_BENCH_SIZES = ("m", "n", "k", "batch", "seq", "heads", "head_dim", "iters", "warmup")


def _kernel_bench(case: str, sizes: Dict[str, Any], knobs: Optional[Dict[str, Any]] = None, timeout: float = 600.0) -> List[Dict[str, Any]]:
    """One case of the kernel benchmark in a CHILD process (the kernel-selection switches are read once per process,
    so a new setting needs a new process); returns the JSON records it printed."""
    import json as _json
    import subprocess
    import sys

    cmd = [sys.executable, "-m", "triune_b200.bench_kernels", "--case", case]
    for k in _BENCH_SIZES:
        if k in sizes:
            cmd += ["--" + k.replace("_", "-"), str(int(sizes[k]))]
    env = dict(os.environ)
    root = str(Path(__file__).resolve().parents[2])
    env["PYTHONPATH"] = root + (os.pathsep + env["PYTHONPATH"] if env.get("PYTHONPATH") else "")
    for k, v in (knobs or {}).items():
        if v is None:
            env.pop(k, None)
        else:
            env[k] = str(int(v))
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    recs = []
    for line in r.stdout.splitlines():
        if line.startswith("{"):
            try:
                recs.append(_json.loads(line))
            except ValueError:
                pass
    if r.returncode != 0 and not recs:
        raise RuntimeError(f"benchmark exited with {r.returncode}: {r.stderr[-400:]}")
    return recs


def _need_cuda() -> None:
    import torch

    if not torch.cuda.is_available():
        raise HTTPException(409, "kernel benchmarks need a CUDA device")


@shell_router.post("/v1/engine/benchmarks")
async def engine_benchmark_run(body: Dict[str, Any]):
    from .. import bench_kernels

    case = str(body.get("case", ""))
    if case not in bench_kernels.CASES:
        raise HTTPException(404, f"unknown case {case!r}; one of {sorted(bench_kernels.CASES)}")
    _need_cuda()
    try:
        return {"results": await asyncio.to_thread(_kernel_bench, case, body, body.get("knobs"))}
    except Exception as e:
        raise _bad(e, 500)


def _check_knobs(knobs: Dict[str, Any]) -> None:
    for k in knobs:
        if k not in TUNING_KNOBS:
            raise HTTPException(400, f"unknown knob {k!r}; one of {list(TUNING_KNOBS)}")


@shell_router.post("/v1/hardware/tune")
async def hardware_tune(body: Dict[str, Any]):
    """Set kernel-selection switches in this server's environment. They are read once per process by the extension,
    so they apply to processes started from now on (the benchmarks this server runs are such processes) and to this
    process only if it has not launched a GEMM yet. This never touches clocks, power limits or any other device
    setting: those belong to the machine's operator."""
    knobs = body.get("knobs") or {}
    _check_knobs(knobs)
    changed = {}
    for k, v in knobs.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = str(int(v))
        changed[k] = os.environ.get(k)
    return {"changed": changed, "tuning": {k: os.environ.get(k) for k in TUNING_KNOBS}}


@shell_router.post("/v1/hardware/autotune")
async def hardware_autotune(body: Dict[str, Any]):
    """Time one GEMM shape under each candidate setting (one child process each) and report the fastest.
    ``{"m", "n", "k", "candidates": [{knob: value}, ...], "apply": false}``; the default candidates toggle CTA pairs
    and move their shortest reduction. ``apply`` stores the winner in this server's environment."""
    _need_cuda()
    cands = body.get("candidates") or [{}, {"TRIUNE_GEMM_PAIR": 0}, {"TRIUNE_GEMM_PAIR_MIN_K": 384}, {"TRIUNE_GEMM_PAIR_MIN_K": 1536}]
    for c in cands:
        _check_knobs(c)
    sizes = {k: body[k] for k in ("m", "n", "k", "iters", "warmup") if k in body}
    table = []
    for c in cands:
        try:
            recs = await asyncio.to_thread(_kernel_bench, "gemm", sizes, c)
            table.append({"knobs": c, "ms": min(r["ms"] for r in recs if "ms" in r), "tflops": max(r.get("tflops", 0.0) for r in recs)})
        except Exception as e:
            table.append({"knobs": c, "error": f"{type(e).__name__}: {e}"[:300]})
    ok = [t for t in table if "ms" in t]
    best = min(ok, key=lambda t: t["ms"]) if ok else None
    if best and body.get("apply"):
        for k, v in best["knobs"].items():
            os.environ[k] = str(int(v))
    return {"results": table, "best": best, "applied": bool(best and body.get("apply"))}


# ---------------------------------------------------------------------------------------------------- provider keys
@shell_router.post("/v1/byok/save")
async def byok_save(body: Dict[str, Any]):
    """Keep a provider key in this process's memory (never written to disk, never echoed back)."""
    provider, key = str(body.get("provider", "")).strip().lower(), str(body.get("api_key", ""))
    if not provider or len(key) < 8:
        raise HTTPException(400, "provider and an api_key of at least 8 characters are required")
    _SHELL["byok"][provider] = key
    return {"provider": provider, "stored": True, "hint": f"...{key[-4:]}"}


@shell_router.post("/v1/byok/test")
async def byok_test(body: Dict[str, Any]):
    provider = str(body.get("provider", "")).strip().lower()
    return {"provider": provider, "configured": provider in _SHELL["byok"], "reachable": None,
            "note": "this server makes no outbound requests; only the presence of a key is reported"}
