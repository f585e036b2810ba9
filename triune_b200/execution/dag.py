"""Typed-port DAG execution (thin version of ``triune/execution/dag.py``).

A graph is ``{"nodes": [{"id", "type", "params"}], "edges": [{"from": "a.out", "to": "b.in"}]}``. Every node type
declares typed input / output ports; validation checks unknown types, dangling or doubly driven inputs, port type
mismatches and cycles before anything runs; execution is a topological sweep that passes port values and emits
``on_node_start`` events. The handlers registered here wrap framework calls (model loading, tokenisation, generation,
training steps, fine-tuning, export, memory planning, sandboxed code); plugins add more through ``register_node``.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..callbacks import global_emitter

ANY = "any"


@dataclass
class NodeType:
    name: str
    inputs: Dict[str, str]
    outputs: Dict[str, str]
    handler: Callable[[Dict[str, Any], Dict[str, Any], Dict[str, Any]], Dict[str, Any]]  # (inputs, params, context) -> outputs
    description: str = ""
    optional_inputs: Tuple[str, ...] = ()


NODE_TYPES: Dict[str, NodeType] = {}


def register_node(name: str, inputs: Dict[str, str], outputs: Dict[str, str], description: str = "", optional: Tuple[str, ...] = ()):
    def deco(fn):
        NODE_TYPES[name] = NodeType(name, dict(inputs), dict(outputs), fn, description, tuple(optional))
        return fn

    return deco


class DAGValidationError(ValueError):
    pass


@dataclass
class DAG:
    nodes: Dict[str, Dict[str, Any]]
    edges: List[Tuple[str, str, str, str]]  # (src node, src port, dst node, dst port)
    order: List[str] = field(default_factory=list)


def parse_dag(spec: Dict[str, Any]) -> DAG:
    nodes = {}
    for n in spec.get("nodes", []):
        if n["id"] in nodes:
            raise DAGValidationError(f"duplicate node id {n['id']!r}")
        nodes[n["id"]] = {"type": n["type"], "params": dict(n.get("params", {}))}
    edges = []
    for e in spec.get("edges", []):
        s, d = e["from"], e["to"]
        sn, _, sp = s.partition(".")
        dn, _, dp = d.partition(".")
        edges.append((sn, sp or "out", dn, dp or "in"))
    return validate_dag(DAG(nodes, edges))


def validate_dag(dag: DAG) -> DAG:
    for nid, n in dag.nodes.items():
        if n["type"] not in NODE_TYPES:
            raise DAGValidationError(f"node {nid!r}: unknown type {n['type']!r}")
    driven = set()
    indeg = {n: 0 for n in dag.nodes}
    succ: Dict[str, List[str]] = {n: [] for n in dag.nodes}
    for sn, sp, dn, dp in dag.edges:
        if sn not in dag.nodes or dn not in dag.nodes:
            raise DAGValidationError(f"edge {sn}.{sp} -> {dn}.{dp} references a missing node")
        st, dt = NODE_TYPES[dag.nodes[sn]["type"]], NODE_TYPES[dag.nodes[dn]["type"]]
        if sp not in st.outputs:
            raise DAGValidationError(f"{sn} ({st.name}) has no output port {sp!r}")
        if dp not in dt.inputs:
            raise DAGValidationError(f"{dn} ({dt.name}) has no input port {dp!r}")
        a, b = st.outputs[sp], dt.inputs[dp]
        if ANY not in (a, b) and a != b:
            raise DAGValidationError(f"type mismatch on {sn}.{sp} ({a}) -> {dn}.{dp} ({b})")
        if (dn, dp) in driven:
            raise DAGValidationError(f"input {dn}.{dp} is driven twice")
        driven.add((dn, dp))
        indeg[dn] += 1
        succ[sn].append(dn)
    for nid, n in dag.nodes.items():
        t = NODE_TYPES[n["type"]]
        for port in t.inputs:
            if (nid, port) not in driven and port not in t.optional_inputs and port not in n["params"]:
                raise DAGValidationError(f"input {nid}.{port} is not connected and has no parameter value")
    ready = [n for n, d in indeg.items() if d == 0]
    order = []
    while ready:
        n = ready.pop(0)
        order.append(n)
        for m in succ[n]:
            indeg[m] -= 1
            if indeg[m] == 0:
                ready.append(m)
    if len(order) != len(dag.nodes):
        raise DAGValidationError("the graph has a cycle")
    dag.order = order
    return dag


def execute_dag(spec_or_dag, context: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """Run a graph. Graphs saved by the Studio canvas (edges with ``source`` / ``target``, the canvas' node names) are
    handed to ``execution/studio.py`` and answer in that format; everything else is this module's own format."""
    if not isinstance(spec_or_dag, DAG):
        from .studio import is_studio_graph, run_studio_graph

        if is_studio_graph(spec_or_dag):
            return run_studio_graph(spec_or_dag, context)
    dag = spec_or_dag if isinstance(spec_or_dag, DAG) else parse_dag(spec_or_dag)
    ctx = context if context is not None else {}
    values: Dict[Tuple[str, str], Any] = {}
    timings: Dict[str, float] = {}
    for nid in dag.order:
        n = dag.nodes[nid]
        t = NODE_TYPES[n["type"]]
        inputs = {p: n["params"][p] for p in t.inputs if p in n["params"]}
        for sn, sp, dn, dp in dag.edges:
            if dn == nid:
                inputs[dp] = values[(sn, sp)]
        global_emitter.emit_node_start(nid, t.name, n["params"])
        t0 = time.perf_counter()
        out = t.handler(inputs, n["params"], ctx) or {}
        timings[nid] = time.perf_counter() - t0
        for p in t.outputs:
            values[(nid, p)] = out.get(p)
    return {"outputs": {f"{n}.{p}": v for (n, p), v in values.items()}, "timings": timings, "order": dag.order}


def node_catalog() -> List[Dict[str, Any]]:
    return [{"type": t.name, "inputs": t.inputs, "outputs": t.outputs, "optional_inputs": list(t.optional_inputs),
             "description": t.description} for t in NODE_TYPES.values()]


# ---------------------------------------------------------------------------------------------------- built-in nodes
@register_node("constant", {}, {"out": ANY}, "emits params['value']")
def _constant(i, p, c):
    return {"out": p.get("value")}


@register_node("text", {}, {"out": "text"}, "emits params['text']")
def _text(i, p, c):
    return {"out": str(p.get("text", ""))}


@register_node("concat_text", {"a": "text", "b": "text"}, {"out": "text"}, "a + separator + b")
def _concat(i, p, c):
    return {"out": f"{i['a']}{p.get('separator', '')}{i['b']}"}


@register_node("load_model", {}, {"model": "model"}, "preset / checkpoint / config -> model")
def _load_model(i, p, c):
    from ..models.zoo import load_model

    return {"model": load_model(p.get("model", "triune-nano"), **p.get("overrides", {}))}


@register_node("model_info", {"model": "model"}, {"out": "json"}, "parameter count and shape facts")
def _model_info(i, p, c):
    m = i["model"]
    return {"out": {"parameters": sum(x.numel() for x in m.parameters()), "layers": getattr(m, "num_layers", None),
                    "hidden_dim": getattr(m, "hidden_dim", None), "vocab_size": getattr(m, "vocab_size", None)}}


@register_node("tokenize", {"text": "text"}, {"ids": "tokens"}, "UTF-8 bytes or params['tokenizer_path']")
def _tokenize(i, p, c):
    if p.get("tokenizer_path"):
        from ..data.tokenizer import load_tokenizer

        out = load_tokenizer(p["tokenizer_path"]).encode(i["text"])
        return {"ids": list(getattr(out, "ids", out))}
    return {"ids": list(i["text"].encode("utf-8"))}


@register_node("generate", {"model": "model", "prompt": "text"}, {"text": "text", "telemetry": "json"}, "greedy / sampled generation")
def _generate(i, p, c):
    from ..inference import generate_response
    from ..serve.engine_state import ByteTokenizer

    tok = c.get("tokenizer") or ByteTokenizer(min(256, int(getattr(i["model"], "vocab_size", 256))))
    out = generate_response(i["model"], tok, i["prompt"], max_new_tokens=int(p.get("max_new_tokens", 32)),
                            temperature=float(p.get("temperature", 0.0)), template=bool(p.get("template", False)))
    return {"text": out["text"], "telemetry": out["telemetry"]}


@register_node("train_steps", {"model": "model"}, {"model": "model", "losses": "json"}, "synthetic-data training steps")
def _train(i, p, c):
    import torch

    from ..data import SyntheticTokenSource
    from ..optim import CentroidSteerOptimizer
    from ..trainer import Trainer

    m = i["model"]
    dev = next(m.parameters()).device
    run = {"lr": float(p.get("lr", 1e-3)), "warmup_steps": 2, "total_steps": 1000, "depth_mode": p.get("depth_mode", "cortex"),
           "grad_accum_steps": 1, "grad_clip": 1.0, "vocab_size": int(m.vocab_size)}
    tr = Trainer(m, run, optimizer=CentroidSteerOptimizer(m, lr=run["lr"], grad_clip=1.0),
                 train_loader=SyntheticTokenSource(int(m.vocab_size), int(p.get("batch_size", 2)), int(p.get("seq_len", 32)), seed=0, pool=1),
                 device=dev)
    return {"model": m, "losses": [float(tr.engine.step_once()["loss"]) for _ in range(int(p.get("steps", 2)))]}


@register_node("estimate_memory", {}, {"out": "json"}, "memory plan of a preset")
def _estimate(i, p, c):
    from ..config import get_model_config
    from ..runtime.memory_planner import MemoryPlanner

    cfg = {**get_model_config(p.get("model", "triune-base")).to_dict(), "batch_size": int(p.get("batch_size", 16)), "seq_len": int(p.get("seq_len", 2048))}
    return {"out": MemoryPlanner.estimate_vram(cfg, available_vram_gb=p.get("vram_gb", 180.0)).to_dict()}


@register_node("export_model", {"model": "model"}, {"path": "text"}, "safetensors / hf / pt export")
def _export(i, p, c):
    from ..export import export_model

    return {"path": str(export_model(i["model"], p["output"], p.get("format", "safetensors")))}


@register_node("python", {"value": ANY}, {"out": ANY}, "sandboxed code; reads `value`, sets `result`", optional=("value",))
def _python(i, p, c):
    from ..runtime.sandbox import PythonSandbox

    r = PythonSandbox(int(p.get("timeout", 5))).execute_code(str(p.get("code", "")), {"value": i.get("value")})
    if not r["success"]:
        raise RuntimeError(r["error"])
    return {"out": r["result"]}


from . import nodes  # noqa: E402,F401  (registers the component nodes)
