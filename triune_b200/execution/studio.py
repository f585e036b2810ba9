"""Graphs in the Studio canvas format, run on this framework.

The canvas of the reference project saves a graph as ``{"nodes": [{"id", "type", "title", "details" | "params" |
"config", ...}], "edges": [{"source", "target", "source_port", "target_port"}]}`` and names 49 node kinds
(``triune/execution/dag.py:474-541``) with the ports of its catalogue (``triune/plugins/registry.py:178-803``). This
module accepts those graphs unchanged: the same node names, port names and parameter names, resolved the same way
(a node's title before its broad category, ``details`` lines ``key=value`` under explicit ``params`` under ``config``
values), typed edges checked before anything runs, edges without ports passing every output of their source on, one
driver per input, cycles refused, subgraphs with declared sockets nested at most eight deep, execution stopping at
the first node that fails. The response has the reference's shape (``status``, ``results[node]`` with ``status`` /
``elapsed_sec`` / ``output``, ``failed_node``, ``error``).

What differs is underneath: every node here calls this framework (models, CUDA operators, optimizers, exporters);
values travel between nodes as live tensors and modules and are summarised only for the response; nodes that would
need the internet (hub and URL streams, provider chat) work on local files and say so instead of pretending.
``execution/dag.py`` is this framework's own, smaller graph format; ``parse_dag`` hands Studio graphs over to here.
"""

from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

from ..callbacks import global_emitter

MAX_SUBGRAPH_DEPTH = 8

# port types of the catalogue (``triune/plugins/node_schema.py:14-26``)
TENSOR, TEXT, STREAM, MODEL, OPT, LOSS, TUPLE, METRICS, FILE, ANY = (
    "tensor", "text", "dataset_stream", "model_handle", "optimizer_handle", "loss", "tensor_tuple", "metrics", "file", "any")
CONFIG = "config"
# (source type, target type) pairs that may be wired although the types differ: a dataset stream yields text samples, a
# loss is a scalar tensor and a metric, tensors feed losses and metrics, a tuple of tensors stands in for its first member
_COMPATIBLE = {(STREAM, TEXT), (LOSS, TENSOR), (LOSS, METRICS), (TENSOR, LOSS), (TENSOR, METRICS), (TUPLE, TENSOR)}


class StudioGraphError(ValueError):
    pass


class NodeFailure(RuntimeError):
    """Raised by a node to fail the run with a message for the user (not a bug in the runner)."""


@dataclass
class StudioNode:
    name: str
    category: str
    inputs: Dict[str, str]
    outputs: Dict[str, str]
    parameters: Dict[str, Any]
    fn: Callable[[Dict[str, Any], Dict[str, Any], Dict[str, Any]], Dict[str, Any]]
    description: str = ""
    dynamic_ports: bool = False  # sockets declared per instance (subgraphs)


STUDIO_NODES: Dict[str, StudioNode] = {}


def studio_node(name: str, category: str, inputs: Dict[str, str], outputs: Dict[str, str], parameters: Optional[Dict[str, Any]] = None,
                description: str = "", aliases: Tuple[str, ...] = (), dynamic_ports: bool = False):
    def deco(fn):
        for n in (name,) + tuple(aliases):
            STUDIO_NODES[n] = StudioNode(n, category, dict(inputs), dict(outputs), dict(parameters or {}), fn, description, dynamic_ports)
        return fn

    return deco


def ports_compatible(a: str, b: str) -> bool:
    return a == b or ANY in (a, b) or (a, b) in _COMPATIBLE


class PortType(str, Enum):
    """Port types under the reference's enumeration names (``triune/plugins/node_schema.py``)."""

    TEXT = TEXT
    TENSOR = TENSOR
    TENSOR_TUPLE = TUPLE
    DATASET_STREAM = STREAM
    MODEL_HANDLE = MODEL
    OPTIMIZER_HANDLE = OPT
    LOSS = LOSS
    METRICS = METRICS
    CONFIG = CONFIG
    FILE = FILE
    ANY = ANY


class NodeExecutionType(str, Enum):
    EXECUTION = "execution"  # runs tensor work
    SPECIFICATION = "specification"  # only describes (hyper-parameters, blueprints, provider settings)


def is_port_compatible(source_type: Any, target_type: Any) -> bool:
    """``ports_compatible`` for enumeration members or strings in any case."""
    a = str(getattr(source_type, "value", source_type)).lower()
    b = str(getattr(target_type, "value", target_type)).lower()
    return ports_compatible(a, b)


@dataclass
class Port:
    name: str
    type: str = ANY
    description: str = ""
    required: bool = True

    def to_dict(self) -> Dict[str, Any]:
        return {"name": self.name, "type": str(getattr(self.type, "value", self.type)), "description": self.description,
                "required": self.required}


@dataclass
class NodeSchema:
    """Declarative description of a node kind, as the canvas and validators exchange it."""

    id: str
    name: str
    category: str
    execution_type: str = NodeExecutionType.EXECUTION.value
    inputs: List[Port] = field(default_factory=list)
    outputs: List[Port] = field(default_factory=list)
    config_params: Dict[str, Any] = field(default_factory=dict)
    description: str = ""
    requires_cuda: bool = False

    def to_dict(self) -> Dict[str, Any]:
        return {"id": self.id, "name": self.name, "category": self.category,
                "execution_type": str(getattr(self.execution_type, "value", self.execution_type)),
                "inputs": [p.to_dict() for p in self.inputs], "outputs": [p.to_dict() for p in self.outputs],
                "config_params": dict(self.config_params), "description": self.description, "requires_cuda": self.requires_cuda}


def node_schema(kind: str) -> NodeSchema:
    """The ``NodeSchema`` of a catalogue entry."""
    n = STUDIO_NODES[kind]
    return NodeSchema(id=n.name, name=n.name, category=n.category,
                      inputs=[Port(k, t) for k, t in n.inputs.items()], outputs=[Port(k, t, required=False) for k, t in n.outputs.items()],
                      config_params=dict(n.parameters), description=n.description)


def is_studio_graph(spec: Any) -> bool:
    """True for the canvas format (edges carry ``source`` / ``target``), false for ``{"from": "a.out", "to": "b.in"}``."""
    if not isinstance(spec, dict):
        return False
    edges = spec.get("edges") or []
    if any(isinstance(e, dict) and ("source" in e or "target" in e) for e in edges):
        return True
    nodes = spec.get("nodes") or []
    return not edges and any(isinstance(n, dict) and resolve_kind(n) in STUDIO_NODES and n.get("type") not in _native_types()
                             for n in nodes)


def _native_types():
    from .dag import NODE_TYPES

    return NODE_TYPES


# keyword fall-back for nodes whose type and title name no known kind (first match wins)
_KEYWORDS: Tuple[Tuple[Tuple[str, ...], str], ...] = (
    (("hugging", "hf", "stream"), "HuggingFaceStreamer"), (("token", "bpe"), "BPETokenizer"),
    (("centroid", "galore"), "CentroidSteerOptimizer"), (("muon",), "MuonOptimizer"), (("optim", "adam"), "Optimizer"),
    (("schedul", "lr"), "CosineLRScheduler"), (("joint", "exitloss"), "JointExitLoss"),
    (("accumul", "microbatch"), "GradientAccumulator"), (("checkpoint", "ckpt"), "CheckpointManager"),
    (("resource", "feasib"), "DynamicResourceManager"), (("generat", "autoregress", "decode"), "AutoregressiveGenerator"),
    (("rope", "rotary"), "FastRoPE"), (("byok", "frontier", "llm"), "BYOKChatRouter"), (("loss", "entropy"), "Loss"),
    (("router", "exit"), "DepthRouter"), (("gla", "attention"), "VectorisedGLA"), (("moe", "expert"), "MoE_FFN"),
    (("lora", "peft", "adapt"), "LoRAAdapter"), (("vram", "profil"), "VRAMProfiler"), (("eval", "perplex"), "Evaluation"),
    (("gguf",), "GGUFExport"), (("onnx",), "ONNXExport"), (("export", "safetensor"), "Export"),
    (("model", "transformer"), "Model"), (("data", "dataset"), "Data"),
)
_CATEGORIES = ("Data", "Model", "Optimizer", "Loss", "Runtime", "Evaluation", "Export")


# display titles of the canvas' palette (lower case, letters and digits only) -> node kind; the canvas stores the title a
# node was created with and the broad category in ``type``, so this table is what identifies most nodes of a saved graph
_TITLES = {
    "huggingfacestreamer": "HuggingFaceStreamer", "urldatasetstreamer": "URLDatasetStreamer", "localfilereader": "LocalFileReader",
    "bpetokenizer": "BPETokenizer", "cyclingdataloader": "CyclingDataLoader", "autogradtrainingstep": "TrainingStep",
    "triunemoetransformer": "TriuneTransformer", "triunemoettransformer": "TriuneTransformer", "vectorisedglaattention": "VectorisedGLA",
    "hybridglaropeattention": "HybridAttention", "sparsemoeffnlayer": "MoE_FFN", "hierarchicaldepthrouter": "DepthRouter",
    "fp8scaledlinear": "FP8Linear", "nvfp4microscalinglinear": "FP4Linear", "tensorinspector": "TensorInspector",
    "tokenbatchinspector": "TokenBatchInspector", "fastrmsnorm": "RMSNorm", "loraadapterlayer": "LoRAAdapter",
    "centroidsteeroptimizer": "CentroidSteerOptimizer", "muonmatrixoptimizer": "MuonOptimizer", "adamwoptimizer": "AdamWOptimizer",
    "cosinelrscheduler": "CosineLRScheduler", "fastcrossentropyloss": "FastCrossEntropy", "jointexitloss": "JointExitLoss",
    "routerstabilityzloss": "RouterZLoss", "fastropekernel": "FastRoPE", "fastrmsnormkernel": "FastRMSNorm",
    "autoregressivegenerator": "AutoregressiveGenerator", "byokchatrouter": "BYOKChatRouter", "gradientaccumulator": "GradientAccumulator",
    "checkpointmanager": "CheckpointManager", "dynamicresourcemanager": "DynamicResourceManager", "layerstreamingengine": "LayerStreamingEngine",
    "vramprofiler": "VRAMProfiler", "restrictedpythonrunner": "PythonSandbox", "wandbtelemetrylogger": "WandbLogger",
    "perplexityevaluator": "PerplexityEvaluator", "lorafinetunerengine": "LoRAFineTuner", "safetensorsexporter": "SafeTensorsExport",
    "ggufexportconfigurationonly": "GGUFExport", "onnxgraphexporter": "ONNXExport", "reroutenode": "RerouteNode", "reroute": "RerouteNode",
}


def _squash(text: str) -> str:
    return "".join(ch for ch in text.lower() if ch.isalnum())


def resolve_kind(node: Dict[str, Any]) -> Optional[str]:
    """The node kind: a title that names one (its kind, or its display title in the palette) wins over the broad category
    in ``type``; then ``type``; then keywords."""
    title, typ = str(node.get("title") or node.get("name") or ""), str(node.get("type") or "")
    if title in STUDIO_NODES and title not in _CATEGORIES:
        return title
    by_title = _TITLES.get(_squash(title)) or next((k for k in STUDIO_NODES if k not in _CATEGORIES and _squash(k) == _squash(title)), None)
    if by_title in STUDIO_NODES:
        return by_title
    if typ in STUDIO_NODES:
        return typ
    if title in STUDIO_NODES:
        return title
    low = f"{typ} {title}".lower()
    if not low.strip():
        return None
    for words, kind in _KEYWORDS:
        if any(w in low for w in words):
            return kind
    return None


def node_params(node: Dict[str, Any]) -> Dict[str, Any]:
    """``details`` lines ``key=value`` (JSON where it parses), overridden by ``params``, overridden by ``config``
    entries (``{"value": v}`` or plain values)."""
    out: Dict[str, Any] = {}
    details = node.get("details")
    if isinstance(details, str):
        for line in details.splitlines():
            key, sep, raw = line.partition("=")
            if not sep or not key.strip():
                continue
            raw = raw.strip()
            try:
                out[key.strip()] = json.loads(raw)
            except (ValueError, TypeError):
                out[key.strip()] = raw
    if isinstance(node.get("params"), dict):
        out.update(node["params"])
    if isinstance(node.get("config"), dict):
        for k, v in node["config"].items():
            out[k] = v.get("value", v) if isinstance(v, dict) else v
    return out


def _ports_of(node: Dict[str, Any], kind: Optional[str]) -> Tuple[Optional[Dict[str, str]], Optional[Dict[str, str]]]:
    """(inputs, outputs) as name -> type, or (None, None) when the node publishes no schema."""
    if kind is None or kind not in STUDIO_NODES:
        return None, None
    spec = STUDIO_NODES[kind]
    if not spec.dynamic_ports:
        return spec.inputs, spec.outputs
    if kind == "SubgraphInput":
        return {}, {"value": str(node_params(node).get("port_type", ANY))}
    d = node.get("subgraph") if isinstance(node.get("subgraph"), dict) else {}
    ins = {str(i.get("name")): str(i.get("type", ANY)) for i in d.get("inputs", []) if isinstance(i, dict) and i.get("name")}
    outs = {str(o.get("name")): str(o.get("type", ANY)) for o in d.get("outputs", []) if isinstance(o, dict) and o.get("name")}
    return ins, outs


@dataclass
class ParsedGraph:
    nodes: Dict[str, Dict[str, Any]]
    edges: List[Dict[str, Any]]
    order: List[str] = field(default_factory=list)
    kinds: Dict[str, Optional[str]] = field(default_factory=dict)


def parse_studio_graph(graph: Dict[str, Any]) -> ParsedGraph:
    if not isinstance(graph, dict):
        raise StudioGraphError("a graph is an object with nodes and edges")
    nodes, edges = graph.get("nodes", []), graph.get("edges", [])
    if not isinstance(nodes, list) or not isinstance(edges, list):
        raise StudioGraphError("nodes and edges must both be arrays")
    node_map: Dict[str, Dict[str, Any]] = {}
    for k, n in enumerate(nodes):
        if not isinstance(n, dict):
            raise StudioGraphError(f"node {k + 1} must be an object")
        nid = n.get("id")
        if not isinstance(nid, str) or not nid.strip():
            raise StudioGraphError(f"node {k + 1} needs a non-empty string id")
        if nid in node_map:
            raise StudioGraphError(f"duplicate node id: {nid}")
        node_map[nid] = n
    kinds = {nid: resolve_kind(n) for nid, n in node_map.items()}
    seen, driven = set(), set()
    indeg = {nid: 0 for nid in node_map}
    succ: Dict[str, List[str]] = {nid: [] for nid in node_map}
    for k, e in enumerate(edges):
        if not isinstance(e, dict):
            raise StudioGraphError(f"edge {k + 1} must be an object")
        s, t = e.get("source"), e.get("target")
        if s not in node_map or t not in node_map:
            raise StudioGraphError(f"edge {k + 1} references a missing node ({s!r} -> {t!r})")
        sp, tp = e.get("source_port"), e.get("target_port")
        if (sp is None) != (tp is None):
            raise StudioGraphError(f"edge {k + 1} must name both ports or neither")
        if sp is not None and not (isinstance(sp, str) and sp and isinstance(tp, str) and tp):
            raise StudioGraphError(f"edge {k + 1}: port names must be non-empty strings")
        sig = (s, sp, t, tp)
        if sig in seen:
            raise StudioGraphError(f"duplicate edge {s}:{sp or '*'} -> {t}:{tp or '*'}")
        seen.add(sig)
        if tp is not None:
            if (t, tp) in driven:
                raise StudioGraphError(f"input {t}:{tp} has more than one incoming edge")
            driven.add((t, tp))
            _, outs = _ports_of(node_map[s], kinds[s])
            ins, _ = _ports_of(node_map[t], kinds[t])
            if outs is not None and ins is not None:
                if sp not in outs:
                    raise StudioGraphError(f"node '{node_map[s].get('title', s)}' has no output port '{sp}'")
                if tp not in ins:
                    raise StudioGraphError(f"node '{node_map[t].get('title', t)}' has no input port '{tp}'")
                if not ports_compatible(outs[sp], ins[tp]):
                    raise StudioGraphError(f"type mismatch: '{sp}' ({outs[sp]}) on '{node_map[s].get('title', s)}' cannot feed "
                                           f"'{tp}' ({ins[tp]}) on '{node_map[t].get('title', t)}'")
        indeg[t] += 1
        succ[s].append(t)
    ready = [nid for nid in node_map if indeg[nid] == 0]
    order: List[str] = []
    while ready:
        nid = ready.pop(0)
        order.append(nid)
        for m in succ[nid]:
            indeg[m] -= 1
            if indeg[m] == 0:
                ready.append(m)
    if len(order) != len(node_map):
        raise StudioGraphError("the graph has a cycle")
    return ParsedGraph(node_map, edges, order, kinds)


# ---------------------------------------------------------------------------------------------------- summaries
def summarise(v: Any, depth: int = 0) -> Any:
    """A JSON-safe description of a value that travelled between nodes (tensors and modules are described, not dumped)."""
    try:
        import torch
    except Exception:  # pragma: no cover
        torch = None
    if v is None or isinstance(v, (bool, int, str)):
        return v
    if isinstance(v, float):
        return v if math.isfinite(v) else str(v)
    if torch is not None and isinstance(v, torch.Tensor):
        d: Dict[str, Any] = {"tensor": list(v.shape), "dtype": str(v.dtype).replace("torch.", ""), "device": str(v.device)}
        if v.numel() == 1:
            d["value"] = summarise(float(v.detach().float().item()))
        elif v.numel() and v.is_floating_point():
            f = v.detach().float()
            d.update(mean=summarise(float(f.mean())), std=summarise(float(f.std())) if f.numel() > 1 else 0.0,
                     finite=bool(torch.isfinite(f).all()))
        return d
    if torch is not None and isinstance(v, torch.nn.Module):
        return {"module": type(v).__name__, "parameters": sum(p.numel() for p in v.parameters())}
    if torch is not None and isinstance(v, torch.optim.Optimizer):
        return {"optimizer": type(v).__name__, "param_groups": len(v.param_groups)}
    if depth > 4:
        return str(type(v).__name__)
    if isinstance(v, dict):
        return {str(k): summarise(x, depth + 1) for k, x in list(v.items())[:64] if not str(k).startswith("_")}
    if isinstance(v, (list, tuple)):
        return [summarise(x, depth + 1) for x in list(v)[:64]]
    if isinstance(v, Path):
        return str(v)
    return f"<{type(v).__name__}>"


# ---------------------------------------------------------------------------------------------------- runner
class StudioGraphRunner:
    def __init__(self, emit: Optional[Callable[[Dict[str, Any]], None]] = None):
        self.emit = emit

    def _event(self, payload: Dict[str, Any]) -> None:
        if self.emit is not None:
            try:
                self.emit(payload)
            except Exception:
                pass
        if payload.get("event") == "node_started":
            global_emitter.emit_node_start(payload["node_id"], payload.get("node_type", ""), {})

    def run(self, graph: Dict[str, Any], context: Optional[Dict[str, Any]] = None, *, _keep_values: bool = False) -> Dict[str, Any]:
        g = parse_studio_graph(graph)
        ctx: Dict[str, Any] = context if context is not None else {}
        ctx.setdefault("shared", {})
        values: Dict[str, Dict[str, Any]] = {}
        results: Dict[str, Dict[str, Any]] = {}
        incoming: Dict[str, List[Dict[str, Any]]] = {}
        for e in g.edges:
            incoming.setdefault(e["target"], []).append(e)
        failed: Optional[str] = None
        for nid in g.order:
            node, kind = g.nodes[nid], g.kinds[nid]
            title = node.get("title", node.get("name", nid))
            inputs: Dict[str, Any] = {}
            for e in incoming.get(nid, []):
                src = values.get(e["source"], {})
                sp, tp = e.get("source_port"), e.get("target_port")
                if sp is None:
                    inputs.update(src)  # an edge without ports passes every output of its source on
                elif sp in src:
                    inputs[tp] = src[sp]
            t0 = time.time()
            self._event({"event": "node_started", "node_id": nid, "node_name": title, "node_type": node.get("type", ""), "timestamp": t0})
            try:
                if kind is None or kind not in STUDIO_NODES:
                    raise NodeFailure(f"no handler is registered for node '{title}' ({node.get('type')})")
                spec = STUDIO_NODES[kind]
                params = {**spec.parameters, **node_params(node)}
                call_ctx = dict(ctx, _node=node, _node_id=nid, _runner=self)
                out = spec.fn(inputs, params, call_ctx) or {}
                ctx["shared"] = call_ctx.get("shared", ctx["shared"])
                values[nid] = {k: v for k, v in out.items() if not k.startswith("_")}
                info = {"kind": kind, "ports": summarise(values[nid])}
                if isinstance(out.get("_info"), dict):
                    info.update(summarise(out["_info"]))
                status = "specification" if out.get("_specification") else "completed"
                results[nid] = {"status": status, "elapsed_sec": round(time.time() - t0, 4), "output": info}
                self._event({"event": "node_finished", "node_id": nid, "node_name": title, "node_type": node.get("type", ""),
                             "elapsed_sec": results[nid]["elapsed_sec"], "output": info, "timestamp": time.time()})
            except Exception as err:  # a failing node ends the run; the response says where and why
                msg = str(err) if isinstance(err, NodeFailure) else f"{type(err).__name__}: {err}"
                results[nid] = {"status": "failed", "error": msg, "elapsed_sec": round(time.time() - t0, 4)}
                self._event({"event": "node_failed", "node_id": nid, "node_name": title, "node_type": node.get("type", ""),
                             "elapsed_sec": results[nid]["elapsed_sec"], "error": msg, "timestamp": time.time()})
                failed = nid
                break
        spec_nodes = [n for n, r in results.items() if r["status"] == "specification"]
        resp: Dict[str, Any] = {"results": results, "specification_nodes": spec_nodes, "order": g.order}
        if failed is not None:
            resp.update(status="failed", failed_node=failed, error=results[failed]["error"])
        else:
            resp["status"] = "partial" if spec_nodes else "success"
        if _keep_values:
            resp["_values"] = values
        return resp


def run_studio_graph(graph: Dict[str, Any], context: Optional[Dict[str, Any]] = None, emit=None) -> Dict[str, Any]:
    return StudioGraphRunner(emit).run(graph, context)


def run_studio_node(node: Dict[str, Any], inputs: Optional[Dict[str, Any]] = None, context: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """One node on its own; ``inputs`` (port -> value) reach it as if connected."""
    node = dict(node)
    node.setdefault("id", "single_node")
    feeder = {"id": "__inputs__", "type": "__Inputs__", "params": {"values": dict(inputs or {})}}
    g = {"nodes": [feeder, node], "edges": [{"source": "__inputs__", "target": node["id"]}]} if inputs else {"nodes": [node], "edges": []}
    out = run_studio_graph(g, context)
    res = out["results"].get(node["id"], {"status": "failed", "error": out.get("error", "node did not run")})
    return {**res, "node_status": res.get("status"), "status": out["status"]}


def studio_catalog() -> List[Dict[str, Any]]:
    """The node catalogue in the canvas' shape: typed inputs / outputs, default parameters, category."""
    cat = []
    for n in STUDIO_NODES.values():
        if n.name.startswith("__"):
            continue
        cat.append({"name": n.name, "category": n.category, "description": n.description, "parameters": dict(n.parameters),
                    "typed_inputs": [{"name": k, "type": t} for k, t in n.inputs.items()],
                    "typed_outputs": [{"name": k, "type": t} for k, t in n.outputs.items()],
                    "inputs": list(n.inputs), "outputs": list(n.outputs), "dynamic_ports": n.dynamic_ports})
    return cat


# ---------------------------------------------------------------------------------------------------- helpers for nodes
def _torch():
    import torch

    return torch


def _shared(c) -> Dict[str, Any]:
    return c.setdefault("shared", {})


def _pick(i, c, *names):
    """The first of these that is connected, else the last value a node published under that name."""
    for n in names:
        if i.get(n) is not None:
            return i[n]
    for n in names:
        if _shared(c).get(n) is not None:
            return _shared(c)[n]
    return None


def _device(c):
    torch = _torch()
    st = c.get("state")
    if st is not None and getattr(st, "device", None) is not None:
        return st.device
    return torch.device("cuda:0" if torch.cuda.is_available() else "cpu")


def _model(i, c, required: bool = True):
    m = _pick(i, c, "model_handle", "model")
    if m is None and c.get("state") is not None and getattr(c["state"], "model", None) is not None:
        m = c["state"].model
    if m is None and required:
        raise NodeFailure("no model: connect a TriuneTransformer node's model_handle or load a model first")
    return m


def _tokenizer(c, vocab: int = 256):
    st = c.get("state")
    tok = _shared(c).get("tokenizer") or (getattr(st, "tokenizer", None) if st is not None else None)
    if tok is None:
        from ..serve.engine_state import ByteTokenizer

        tok = ByteTokenizer(min(256, vocab))
    return tok


def _as_tokens(v, c):
    """[B, T] int64 token tensor from a tensor, a list of ids or text."""
    torch = _torch()
    if isinstance(v, torch.Tensor):
        t = v.long()
        return t if t.dim() == 2 else t.reshape(1, -1)
    if isinstance(v, str):
        ids = _tokenizer(c).encode(v)
        return torch.tensor([list(getattr(ids, "ids", ids))], dtype=torch.long)
    if isinstance(v, (list, tuple)) and v:
        return torch.tensor(v, dtype=torch.long).reshape(1, -1) if not isinstance(v[0], (list, tuple)) else torch.tensor(v, dtype=torch.long)
    return None


def _hidden(i, c, p, key="hidden_states"):
    torch = _torch()
    x = _pick(i, c, key, "x")
    if x is None:
        d = int(p.get("hidden_dim") or p.get("dim") or p.get("in_features") or 64)
        g = torch.Generator().manual_seed(int(p.get("seed", 0)))
        x = torch.randn(int(p.get("batch_size", 2)), int(p.get("seq_len", 16)), d, generator=g)
    return x


def _place(mod, x):
    return mod.to(device=x.device, dtype=x.dtype if x.is_floating_point() else None)


def shallow_exit_layout(num_layers: int) -> Dict[str, int]:
    """Router prefix and the two early exits for a model shallower than the default layout needs (exits at about a
    quarter and a half of the depth); empty for 16 layers and more, where the defaults hold."""
    nl = int(num_layers)
    if nl >= 16:
        return {}
    if nl < 4:
        raise NodeFailure("a three-exit model needs at least 4 layers")
    prefix = max(1, nl // 8)
    reflex = max(prefix + 1, nl // 4)
    return {"router_prefix_layers": prefix, "reflex_exit_layer": reflex, "limbic_exit_layer": max(reflex + 1, nl // 2)}


def _out_dir(p, c, default="outputs") -> Path:
    d = Path(str(p.get("save_dir") or p.get("output_dir") or c.get("output_dir") or default)).expanduser()
    d.mkdir(parents=True, exist_ok=True)
    return d


# ---------------------------------------------------------------------------------------------------- data
@studio_node("__Inputs__", "Runtime", {}, {}, dynamic_ports=True)
def _inputs_feeder(i, p, c):
    return dict(p.get("values") or {})


def _read_local_texts(path: str, limit: int = 64) -> List[str]:
    """Up to ``limit`` documents of a file, or of the files of a directory (rows of .jsonl / .parquet give their text field)."""
    from ..data.dataset import TEXT_KEYS, iter_local_texts

    files = [path] if os.path.isfile(path) else sorted(str(f) for f in Path(path).rglob("*") if f.is_file())
    docs: List[str] = []
    for f in files:
        try:
            rows = iter_local_texts(f)
            for row in rows:
                if isinstance(row, dict):
                    row = next((row[k] for k in TEXT_KEYS if isinstance(row.get(k), str)), None)
                if isinstance(row, str) and row.strip():
                    docs.append(row)
                if len(docs) >= limit:
                    return docs
        except ValueError:
            continue  # a file type the readers do not know: skip it inside a directory
    return docs


_BUILTIN_SAMPLE = ("The quick brown fox jumps over the lazy dog. Linear attention keeps a state of fixed size, so the cost of a "
                   "token does not grow with the length of the context. ")


@studio_node("LocalFileReader", "Data", {}, {"dataset": STREAM, "dataset_stream": STREAM, "text_samples": TEXT, "text_sample": TEXT},
             {"file_path": "data/fineweb_sample.jsonl", "batch_size": 4, "seq_len": 64, "configure_runtime": True},
             "local .txt / .jsonl / .parquet corpus", aliases=("Data",))
def _local_reader(i, p, c):
    path = str(p.get("file_path") or p.get("path") or "")
    if not path or not os.path.exists(path):
        raise NodeFailure(f"LocalFileReader: no such file or directory: {path!r}")
    docs = _read_local_texts(path, int(p.get("limit", 64)))
    if not docs:
        raise NodeFailure(f"LocalFileReader: {path!r} holds no text")
    stream = {"kind": "local", "path": path, "documents": len(docs), "batch_size": int(p.get("batch_size", 4)), "seq_len": int(p.get("seq_len", 64))}
    sh = _shared(c)
    sh.update(dataset_stream=stream, text=docs[0], data_source=path)
    return {"dataset": stream, "dataset_stream": stream, "text_samples": docs, "text_sample": docs[0]}


def _offline_stream(kind: str, name: str, p, c):
    """Hub and URL sources without a network: a local path of that name is read; anything else is refused plainly."""
    local = str(p.get("local_path") or "")
    if name.startswith("file://"):
        local = name[len("file://"):]
    elif not local and os.path.exists(name):
        local = name
    if local:
        out = _local_reader({}, {**p, "file_path": local}, c)
        stream = dict(out["dataset_stream"], kind=kind, source=name)
        _shared(c)["dataset_stream"] = stream
        return {"dataset_stream": stream, "text_sample": out["text_sample"], "_info": {"source": name, "read_from": local}}
    raise NodeFailure(f"{kind} source {name!r} needs network access, which this build does not use; give 'local_path' "
                      f"(a .txt / .jsonl / .parquet file or directory) or a file:// URL")


@studio_node("HuggingFaceStreamer", "Data", {}, {"dataset_stream": STREAM, "text_sample": TEXT},
             {"dataset_name": "roneneldan/TinyStories", "split": "train", "config": "", "text_column": "text", "buffer_size": 20},
             "hub dataset stream (local mirror only in this build)")
def _hf_stream(i, p, c):
    return _offline_stream("huggingface", str(p.get("dataset_name", "")), p, c)


@studio_node("URLDatasetStreamer", "Data", {}, {"dataset_stream": STREAM, "text_sample": TEXT},
             {"url": "https://example.com/corpus.jsonl", "text_column": "text", "buffer_size": 20}, "remote corpus stream (file:// only in this build)")
def _url_stream(i, p, c):
    url = str(p.get("url", "")).strip()
    if not url:
        raise NodeFailure("URLDatasetStreamer requires a dataset URL")
    return _offline_stream("url", url, p, c)


@studio_node("BPETokenizer", "Data", {"text": TEXT}, {"tokens": TENSOR}, {"vocab_size": 32000, "pad_token": "[PAD]", "eos_token": "[EOS]"},
             "text -> token ids [1, n]")
def _bpe_tok(i, p, c):
    torch = _torch()
    text = _pick(i, c, "text", "text_sample")
    if isinstance(text, list):
        text = text[0] if text else ""
    if not isinstance(text, str) or not text.strip():
        raise NodeFailure("Tokenizer has no text input; connect a text-producing node")
    tok = None
    if p.get("tokenizer_path"):
        from ..data.tokenizer import load_tokenizer

        if not os.path.isfile(str(p["tokenizer_path"])):
            raise NodeFailure(f"configured tokenizer was not found: {p['tokenizer_path']}")
        tok = load_tokenizer(str(p["tokenizer_path"]))
        _shared(c)["tokenizer"] = tok
    tok = tok or _tokenizer(c)
    enc = tok.encode(text)
    ids = list(getattr(enc, "ids", enc))
    if not ids:
        raise NodeFailure("Tokenizer returned no token ids for the connected text")
    vocab = int(tok.get_vocab_size())
    if min(ids) < 0 or max(ids) >= vocab:
        raise NodeFailure("Tokenizer produced ids outside its declared vocabulary")
    t = torch.tensor([ids], dtype=torch.long)
    _shared(c).update(tokens=t, input_ids=t, tokenizer_vocab=vocab)
    return {"tokens": t, "_info": {"vocab_size": vocab, "seq_len": len(ids), "preview": text[:80]}}


@studio_node("CyclingDataLoader", "Data", {"tokens": TENSOR}, {"input_ids": TENSOR, "targets": TENSOR}, {"batch_size": 4, "seq_len": 64, "shuffle": True},
             "token stream -> (inputs, next-token targets) batch")
def _cycling(i, p, c):
    torch = _torch()
    t = _as_tokens(_pick(i, c, "tokens", "input_ids"), c)
    if t is None or t.dim() != 2 or t.shape[1] < 2:
        raise NodeFailure("DataLoader requires a rank-2 token tensor with at least two tokens per sequence")
    seq = int(p["seq_len"]) if p.get("seq_len") else t.shape[1] - 1
    if seq < 1:
        raise NodeFailure("DataLoader seq_len must be positive")
    flat = t.reshape(-1)
    seq = min(seq, flat.numel() - 1)
    bs = max(1, int(p.get("batch_size", 4)))
    need = bs * seq + 1
    reps = (need + flat.numel() - 1) // flat.numel()
    stream = flat.repeat(reps)[:need]  # cycle the stream until the batch is full
    x, y = stream[:-1].view(bs, seq), stream[1:].view(bs, seq)
    if p.get("shuffle"):
        perm = torch.randperm(bs, generator=torch.Generator().manual_seed(int(p.get("seed", 0))))
        x, y = x[perm], y[perm]
    _shared(c).update(input_ids=x, targets=y)
    return {"input_ids": x, "targets": y}


# ---------------------------------------------------------------------------------------------------- model and layers
@studio_node("TriuneTransformer", "Model", {"input_ids": TENSOR, "model_handle": MODEL},
             {"logits": TENSOR, "model_handle": MODEL, "exit_logits": TUPLE, "router_logits": TENSOR, "balance_loss": LOSS, "selected_depth": TENSOR},
             {"vocab_size": 32000, "hidden_dim": 384, "num_layers": 16, "num_heads": 6, "num_experts": 8, "use_fp4": False, "initialize_only": False},
             "forward pass of the active model, or of a model built from this node when use_node_config is set", aliases=("Model",))
def _triune_model(i, p, c):
    torch = _torch()
    m = _model(i, c, required=False)
    dev = _device(c)
    if m is None or p.get("use_node_config"):
        from ..models.zoo import load_model
        from ..utils import place_model

        given = {k: p[k] for k in ("vocab_size", "hidden_dim", "num_layers", "num_heads", "num_experts", "head_dim", "top_k", "use_fp4", "use_fp8")
                 if p.get(k) is not None}
        for k in ("vocab_size", "hidden_dim", "num_layers", "num_heads", "num_experts", "head_dim", "top_k"):
            if k in given:
                given[k] = int(given[k])
        if "head_dim" not in given and given.get("hidden_dim") and given.get("num_heads"):
            given["head_dim"] = given["hidden_dim"] // given["num_heads"]
        nl = given.get("num_layers")
        if nl is not None:
            for k, v in shallow_exit_layout(nl).items():
                given.setdefault(k, v)
        tok_vocab = _shared(c).get("tokenizer_vocab")
        if tok_vocab and int(given.get("vocab_size", 0)) < tok_vocab:
            given["vocab_size"] = int(tok_vocab)
        spec = str(p.get("preset_id") or p.get("preset") or "default")
        m = place_model(load_model(spec, **given), dev, torch.bfloat16 if dev.type == "cuda" else torch.float32)
    _shared(c)["model"] = m
    out = {"model_handle": m}
    ids = _as_tokens(_pick(i, c, "input_ids", "tokens"), c)
    if p.get("initialize_only") or ids is None:
        return {**out, "_info": {"parameters": sum(q.numel() for q in m.parameters()), "forward": False}}
    ids = ids.to(next(m.parameters()).device)
    if int(ids.max()) >= int(m.vocab_size):
        raise NodeFailure(f"token id {int(ids.max())} is outside the model's vocabulary of {int(m.vocab_size)}")
    was = m.training
    m.eval()
    try:
        with torch.no_grad():
            if hasattr(m, "forward_all_exits"):
                lr, ll, lc, route = m.forward_all_exits(ids)
                bal = getattr(m, "last_balance_loss", None)
                out.update(logits=lc, exit_logits=(lr, ll, lc), router_logits=route,
                           balance_loss=bal if bal is not None else torch.zeros((), device=ids.device),
                           selected_depth=route.argmax(-1))
            else:
                res = m(ids)
                out["logits"] = res[0] if isinstance(res, tuple) else getattr(res, "logits", res)
    finally:
        m.train(was)
    sh = _shared(c)
    for k in ("logits", "exit_logits", "router_logits", "balance_loss"):
        if k in out:
            sh[k] = out[k]
    return out


def _mixer(delta: bool):
    def fn(i, p, c):
        from ..models.attention import HybridAttention

        x = _hidden(i, c, p)
        d = x.shape[-1]
        heads = int(p.get("num_heads") or max(1, d // 64))
        if d % heads:
            raise NodeFailure(f"hidden width {d} is not divisible by {heads} heads")
        torch = _torch()
        torch.manual_seed(int(p.get("seed", 0)))
        mod = _place(HybridAttention(d, heads, use_delta_rule=delta or bool(p.get("use_delta_rule")), use_sdpa=bool(p.get("use_sdpa")),
                                     head_dim=d // heads), x).eval()
        with torch.no_grad():
            y = mod(x)
        y = y[0] if isinstance(y, tuple) else y
        _shared(c)["hidden_states"] = y
        return {"attention_out": y}

    return fn


studio_node("VectorisedGLA", "Model", {"hidden_states": TENSOR}, {"attention_out": TENSOR}, {"hidden_dim": 384, "num_heads": 6},
            "gated linear attention over [B, T, d]")(_mixer(False))
studio_node("HybridAttention", "Model", {"hidden_states": TENSOR}, {"attention_out": TENSOR}, {"hidden_dim": 384, "num_heads": 6},
            "attention slot of a block (GLA, delta rule or softmax)")(_mixer(False))


@studio_node("MoE_FFN", "Model", {"hidden_states": TENSOR}, {"moe_out": TENSOR}, {"num_experts": 8, "top_k": 2, "shared_expert": True},
             "routed experts plus the shared expert")
def _moe(i, p, c):
    from ..models.moe import MoE_FFN

    torch = _torch()
    x = _hidden(i, c, p)
    torch.manual_seed(int(p.get("seed", 0)))
    mod = _place(MoE_FFN(x.shape[-1], int(p["num_experts"]), int(p["top_k"]), shared_expert=bool(p["shared_expert"])), x).eval()
    with torch.no_grad():
        y = mod(x)
    y = y[0] if isinstance(y, tuple) else y
    _shared(c)["hidden_states"] = y
    return {"moe_out": y, "_info": {"experts": int(p["num_experts"]), "top_k": int(p["top_k"])}}


@studio_node("DepthRouter", "Model", {"hidden_states": TENSOR}, {"exit_choice": TENSOR, "router_logits": TENSOR, "balance_loss": LOSS},
             {"target_depth_dist": [0.34, 0.33, 0.33], "temperature": 1.0}, "three-way depth router on pooled hidden states")
def _router(i, p, c):
    from ..models.router import GumbelSoftmaxRouter

    torch = _torch()
    x = _hidden(i, c, p)
    torch.manual_seed(int(p.get("seed", 0)))
    mod = _place(GumbelSoftmaxRouter(x.shape[-1], p["target_depth_dist"]), x).eval()
    with torch.no_grad():
        logits, y, bal = mod(x, temperature=float(p["temperature"]))
    _shared(c).update(router_logits=logits, balance_loss=bal)
    return {"exit_choice": y.argmax(-1), "router_logits": logits, "balance_loss": bal}


def _quant_linear(kind: str):
    def fn(i, p, c):
        from ..models.quant_linear import FP4Linear, FP8Linear

        torch = _torch()
        x = _hidden(i, c, p, "x")
        fin = x.shape[-1]
        fout = int(p.get("out_features") or fin)
        torch.manual_seed(int(p.get("seed", 0)))
        ref = torch.nn.Linear(fin, fout, bias=bool(p.get("bias", True)))
        mod = (FP8Linear if kind == "fp8" else FP4Linear)(fin, fout, bias=bool(p.get("bias", True)))
        with torch.no_grad():
            if hasattr(mod, "load_from_linear"):
                mod.load_from_linear(ref)
            elif hasattr(mod, "weight") and mod.weight.shape == ref.weight.shape:
                mod.weight.copy_(ref.weight)
                if getattr(mod, "bias", None) is not None and ref.bias is not None:
                    mod.bias.copy_(ref.bias)
        mod, ref = _place(mod, x).eval(), _place(ref, x).eval()
        with torch.no_grad():
            y, y_ref = mod(x), ref(x)
        err = float((y.float() - y_ref.float()).norm() / y_ref.float().norm().clamp_min(1e-12))
        return {"linear_out": y, "_info": {"format": kind, "relative_error_vs_full_precision": err}}

    return fn


studio_node("FP8Linear", "Model", {"x": TENSOR}, {"linear_out": TENSOR}, {"in_features": 384, "out_features": 384, "bias": True},
            "linear layer with an E4M3 block-scaled weight")(_quant_linear("fp8"))
studio_node("FP4Linear", "Model", {"x": TENSOR}, {"linear_out": TENSOR}, {"in_features": 384, "out_features": 384, "bias": True},
            "linear layer with a 4-bit block-scaled weight")(_quant_linear("fp4"))


@studio_node("TensorInspector", "Analysis", {"x": TENSOR}, {"metrics": METRICS}, {}, "shape, dtype, moments and a finite check")
def _tensor_inspector(i, p, c):
    torch = _torch()
    x = _pick(i, c, "x", "hidden_states", "logits")
    if not isinstance(x, torch.Tensor):
        raise NodeFailure("TensorInspector needs a tensor input")
    f = x.detach().float()
    m = {"shape": list(x.shape), "dtype": str(x.dtype).replace("torch.", ""), "numel": x.numel(), "mean": float(f.mean()),
         "std": float(f.std()) if f.numel() > 1 else 0.0, "min": float(f.min()), "max": float(f.max()),
         "finite": bool(torch.isfinite(f).all()), "l2_norm": float(f.norm())}
    return {"metrics": m}


@studio_node("TokenBatchInspector", "Analysis", {"tokens": TENSOR}, {"metrics": METRICS}, {}, "range, unique count and repetition of a token batch")
def _token_inspector(i, p, c):
    t = _as_tokens(_pick(i, c, "tokens", "input_ids"), c)
    if t is None:
        raise NodeFailure("TokenBatchInspector needs a token tensor")
    flat = t.reshape(-1)
    uniq = int(flat.unique().numel())
    return {"metrics": {"shape": list(t.shape), "min_id": int(flat.min()), "max_id": int(flat.max()), "unique": uniq,
                        "repetition": 1.0 - uniq / max(1, flat.numel())}}


@studio_node("RMSNorm", "Model", {"x": TENSOR}, {"norm_out": TENSOR}, {"dim": 384, "eps": 1e-6}, "RMS normalisation with a unit weight")
def _rmsnorm(i, p, c):
    from .. import ops

    torch = _torch()
    x = _hidden(i, c, p, "x")
    w = i.get("weight")
    if w is None:
        w = torch.ones(x.shape[-1], device=x.device, dtype=x.dtype)
    return {"norm_out": ops.rmsnorm(x, w.to(x.device, x.dtype), float(p.get("eps", 1e-6)))}


studio_node("FastRMSNorm", "Kernel", {"x": TENSOR, "weight": TENSOR}, {"norm_out": TENSOR}, {"eps": 1e-6}, "RMS normalisation kernel")(_rmsnorm)


@studio_node("FastRoPE", "Kernel", {"q": TENSOR, "k": TENSOR}, {"q_rot": TENSOR, "k_rot": TENSOR}, {"dim": 64, "max_seq_len": 8192, "base": 10000.0},
             "rotary position embedding of q and k [B, T, H, D]")
def _rope(i, p, c):
    from ..models.rotary import RotaryEmbedding

    torch = _torch()
    D = int(p["dim"])
    g = torch.Generator().manual_seed(int(p.get("seed", 0)))
    q = i.get("q") if i.get("q") is not None else torch.randn(2, 16, 2, D, generator=g)
    k = i.get("k") if i.get("k") is not None else torch.randn(2, 16, 2, D, generator=g)
    if q.dim() != 4 or q.shape[-1] % 2:
        raise NodeFailure("FastRoPE expects q and k of shape [batch, seq, heads, even head_dim]")
    from .. import ops

    rot = RotaryEmbedding(q.shape[-1], max_seq_len=max(int(p["max_seq_len"]), q.shape[1]), base=float(p["base"]))
    cos, sin = rot(q.shape[1], q.device)
    return {"q_rot": ops.apply_rope(q, cos, sin), "k_rot": ops.apply_rope(k.to(q.device), cos, sin)}


@studio_node("LoRAAdapter", "Model", {"base_layer": MODEL}, {"adapted_layer": MODEL}, {"rank": 16, "alpha": 32.0, "dropout": 0.0, "target_modules": "all"},
             "attach low-rank adapters to a model or a linear layer")
def _lora(i, p, c):
    from ..trainer.finetune import LoRAConfig, TriuneFineTuner

    torch = _torch()
    base = i.get("base_layer")
    if base is None:
        base = _model(i, c, required=False)
    if base is None:
        base = torch.nn.Sequential(torch.nn.Linear(64, 64))
    if isinstance(base, torch.nn.Linear):
        base = torch.nn.Sequential(base)
    ft = TriuneFineTuner(base, LoRAConfig(rank=int(p["rank"]), alpha=float(p["alpha"]), dropout=float(p.get("dropout", 0.0))))
    c.setdefault("finetuners", []).append(ft)
    return {"adapted_layer": base, "_info": {"adapters": len(ft.applied_adapters), "trainable": ft.count_trainable_parameters()}}


# ---------------------------------------------------------------------------------------------------- optimizers, losses
def _optimizer(kind: Optional[str]):
    def fn(i, p, c):
        from ..optim import build_optimizer

        m = _model(i, c)
        k = kind or str(p.get("optimizer") or p.get("optimizer_type") or p.get("name") or "centroid_steer").lower()
        k = "centroid_steer" if "centroid" in k or "galore" in k else ("muon" if "muon" in k else ("adamw" if "adam" in k else k))
        cfg = {"optimizer": k, "lr": float(p.get("lr", 1e-4)), "weight_decay": float(p.get("weight_decay", 0.05))}
        if isinstance(p.get("betas"), (list, tuple)) and len(p["betas"]) == 2:
            cfg["betas"] = (float(p["betas"][0]), float(p["betas"][1]))
        for src, dst in (("momentum", "muon_momentum"), ("ns_steps", "ns_steps"), ("galore_rank", "galore_rank"), ("steer_scale", "steer_scale")):
            if p.get(src) is not None:
                cfg[dst] = p[src]
        opt = build_optimizer(m, cfg)
        _shared(c)["optimizer"] = opt
        metrics = {"optimizer": type(opt).__name__, "lr": cfg["lr"], "parameters": sum(q.numel() for g in opt.param_groups for q in g["params"])}
        loss = _pick(i, c, "loss")
        if loss is not None and getattr(loss, "requires_grad", False) and p.get("apply_step"):
            opt.zero_grad()
            loss.backward()
            opt.step()
            metrics["stepped"] = True
        return {"optimizer_handle": opt, "metrics": metrics}

    return fn


_OPT_PORTS = ({"model_handle": MODEL, "loss": LOSS}, {"optimizer_handle": OPT, "metrics": METRICS})
studio_node("CentroidSteerOptimizer", "Optimizer", *_OPT_PORTS, {"lr": 1e-4, "betas": [0.9, 0.99], "weight_decay": 0.05, "steer_scale": 0.18, "galore_rank": 256},
            "three-tier optimizer")(_optimizer("centroid_steer"))
studio_node("MuonOptimizer", "Optimizer", *_OPT_PORTS, {"lr": 0.02, "momentum": 0.95, "ns_steps": 5}, "Newton-Schulz orthogonalised momentum")(_optimizer("muon"))
studio_node("AdamWOptimizer", "Optimizer", *_OPT_PORTS, {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.1}, "AdamW")(_optimizer("adamw"))
studio_node("Optimizer", "Optimizer", *_OPT_PORTS, {"optimizer": "centroid_steer", "lr": 1e-4}, "optimizer chosen by the 'optimizer' parameter")(_optimizer(None))


@studio_node("CosineLRScheduler", "Optimizer", {"optimizer": OPT}, {"scheduled_lr": METRICS}, {"warmup_steps": 100, "total_steps": 10000, "min_lr_ratio": 0.1},
             "warm-up + cosine learning rate; applied to the connected optimizer")
def _cosine(i, p, c):
    from ..trainer.rescue import cosine_lr

    opt = _pick(i, c, "optimizer", "optimizer_handle")
    base = float(p.get("lr") or (opt.param_groups[0].get("initial_lr", opt.param_groups[0]["lr"]) if opt is not None else 1e-4))
    step = int(p.get("step", 0))
    lr = cosine_lr(step, int(p["total_steps"]), int(p["warmup_steps"]), base, base * float(p["min_lr_ratio"]))
    if opt is not None and p.get("apply", True):
        for g in opt.param_groups:
            g.setdefault("initial_lr", g["lr"])
            g["lr"] = lr * (g["initial_lr"] / base if base else 1.0)
    return {"scheduled_lr": {"step": step, "lr": lr, "base_lr": base, "applied": opt is not None and bool(p.get("apply", True))}}


@studio_node("FastCrossEntropy", "Loss", {"logits": TENSOR, "targets": TENSOR, "balance_loss": LOSS, "router_logits": TENSOR}, {"loss": LOSS, "lm_loss": LOSS},
             {"ignore_index": -100, "chunk_size": 4096, "label_smoothing": 0.0, "balance_loss_weight": 0.01, "router_z_loss_weight": 0.001},
             "next-token cross entropy plus the weighted router terms", aliases=("Loss",))
def _cross_entropy(i, p, c):
    import torch.nn.functional as F

    torch = _torch()
    logits, targets = _pick(i, c, "logits"), _pick(i, c, "targets", "labels")
    if not isinstance(logits, torch.Tensor) or not isinstance(targets, torch.Tensor):
        raise NodeFailure("the loss needs logits [B, T, V] and targets [B, T]")
    T = min(logits.shape[-2], targets.shape[-1])
    lg = logits[..., :T, :].reshape(-1, logits.shape[-1]).float()
    tg = targets[..., :T].reshape(-1).to(lg.device)
    lm = F.cross_entropy(lg, tg, ignore_index=int(p["ignore_index"]), label_smoothing=float(p["label_smoothing"]))
    loss = lm
    bal, route = i.get("balance_loss"), i.get("router_logits")
    if isinstance(bal, torch.Tensor):
        loss = loss + float(p["balance_loss_weight"]) * bal.float().to(lm.device)
    if isinstance(route, torch.Tensor):
        loss = loss + float(p["router_z_loss_weight"]) * torch.logsumexp(route.float(), dim=-1).pow(2).mean().to(lm.device)
    _shared(c)["loss"] = loss
    return {"loss": loss, "lm_loss": lm, "_info": {"perplexity": math.exp(min(float(lm.detach()), 50.0))}}


@studio_node("JointExitLoss", "Loss", {"exit_logits": TUPLE, "targets": TENSOR, "z_loss": LOSS}, {"joint_loss": LOSS, "per_exit_loss": METRICS},
             {"lambda_reflex": 0.3, "lambda_limbic": 0.5, "lambda_cortex": 1.0, "label_smoothing": 0.0}, "weighted sum of the three exits' losses")
def _joint_loss(i, p, c):
    import torch.nn.functional as F

    torch = _torch()
    exits, targets = _pick(i, c, "exit_logits"), _pick(i, c, "targets", "labels")
    if not isinstance(exits, (tuple, list)) or len(exits) != 3 or not isinstance(targets, torch.Tensor):
        raise NodeFailure("JointExitLoss needs the three exits' logits and targets")
    lam = [float(p["lambda_reflex"]), float(p["lambda_limbic"]), float(p["lambda_cortex"])]
    parts = []
    for lg in exits:
        T = min(lg.shape[-2], targets.shape[-1])
        parts.append(F.cross_entropy(lg[..., :T, :].reshape(-1, lg.shape[-1]).float(), targets[..., :T].reshape(-1).to(lg.device),
                                     label_smoothing=float(p["label_smoothing"])))
    joint = sum(a * b for a, b in zip(lam, parts)) / max(sum(lam), 1e-12)
    z = i.get("z_loss")
    if isinstance(z, torch.Tensor):
        joint = joint + z.to(joint.device)
    _shared(c)["loss"] = joint
    return {"joint_loss": joint, "per_exit_loss": {"reflex": float(parts[0].detach()), "limbic": float(parts[1].detach()), "cortex": float(parts[2].detach())}}


@studio_node("RouterZLoss", "Loss", {"router_logits": TENSOR}, {"z_loss": LOSS}, {"coeff": 0.001}, "coeff x mean squared log-partition of the router logits")
def _z_loss(i, p, c):
    torch = _torch()
    r = _pick(i, c, "router_logits")
    if not isinstance(r, torch.Tensor):
        raise NodeFailure("RouterZLoss needs router logits")
    return {"z_loss": float(p["coeff"]) * torch.logsumexp(r.float(), dim=-1).pow(2).mean()}


# ---------------------------------------------------------------------------------------------------- runtime
@studio_node("Runtime", "Runtime", {}, {"runtime_info": METRICS}, {}, "device, precision and kernel facts of this process")
def _runtime(i, p, c):
    from .. import _ext

    torch = _torch()
    dev = _device(c)
    info = {"device": str(dev), "torch": torch.__version__, "cuda": torch.cuda.is_available(), "kernels_loaded": bool(_ext.ext_available())}
    if dev.type == "cuda":
        pr = torch.cuda.get_device_properties(dev)
        info.update(name=pr.name, sms=pr.multi_processor_count, memory_gb=round(pr.total_memory / 2**30, 1), capability=f"{pr.major}.{pr.minor}")
    return {"runtime_info": info}


@studio_node("LayerStreamingEngine", "Runtime", {"model_handle": MODEL}, {"streaming_model": MODEL}, {"prefetch": True, "pin_memory": True, "chunk_size": 1},
             "keep layers in host memory and stream them through the device")
def _layer_streaming(i, p, c):
    from ..runtime.streaming import StreamingConfig, enable_layer_streaming

    m = _model(i, c)
    dev = _device(c)
    eng = enable_layer_streaming(m, str(dev), config=StreamingConfig(resident_gpu_layers=int(p.get("resident_layers", max(1, int(p["chunk_size"])))),
                                                                      pin_memory=bool(p["pin_memory"]) and dev.type == "cuda"))
    c.setdefault("streaming_engines", []).append(eng)
    return {"streaming_model": m, "_info": dict(eng.get_telemetry())}


@studio_node("GradientAccumulator", "Runtime", {"loss": LOSS}, {"accum_status": METRICS}, {"grad_accum_steps": 4},
             "backward of loss / steps; reports when the window is full")
def _grad_accum(i, p, c):
    torch = _torch()
    loss = _pick(i, c, "loss")
    n = max(1, int(p["grad_accum_steps"]))
    st = c.setdefault("accumulation", {"micro_step": 0})
    did = False
    if isinstance(loss, torch.Tensor) and loss.requires_grad:
        (loss / n).backward()
        did = True
    st["micro_step"] += 1
    ready = st["micro_step"] % n == 0
    return {"accum_status": {"micro_step": st["micro_step"], "grad_accum_steps": n, "backward": did, "ready_to_step": ready,
                             "loss": float(loss.detach()) if isinstance(loss, torch.Tensor) else None}}


@studio_node("CheckpointManager", "Runtime", {"model_handle": MODEL, "optimizer_handle": OPT}, {"checkpoint_path": FILE}, {"save_dir": "checkpoints_full", "keep_last_n": 3},
             "write a checkpoint and keep the newest few")
def _checkpoint_manager(i, p, c):
    from ..trainer import checkpoint as ckpt

    m = _model(i, c)
    opt = _pick(i, c, "optimizer_handle", "optimizer")
    d = _out_dir(p, c, "checkpoints_full")
    step = int(p.get("step", c.get("accumulation", {}).get("micro_step", 0)))
    path = ckpt.save_checkpoint(str(d / f"dag_step_{step:08d}.pt"), model=m, optimizer=opt, step=step, config=dict(p.get("config", {})))
    keep = max(1, int(p["keep_last_n"]))
    old = sorted(d.glob("dag_step_*.pt"), key=lambda f: f.stat().st_mtime)[:-keep]
    for f in old:
        f.unlink()
    return {"checkpoint_path": str(path), "_info": {"removed": len(old)}}


@studio_node("DynamicResourceManager", "Runtime", {}, {"feasibility_report": METRICS}, {"target_device": "auto", "safety_margin_gb": 1.0},
             "hardware profile and whether the active model fits")
def _resource_manager(i, p, c):
    from dataclasses import asdict

    from ..runtime.resource_manager import DynamicResourceManager

    dev = None if str(p["target_device"]) in ("auto", "") else str(p["target_device"])
    prof = asdict(DynamicResourceManager.probe_hardware(dev))
    rep: Dict[str, Any] = {"hardware": prof, "safety_margin_gb": float(p["safety_margin_gb"])}
    m = _model(i, c, required=False)
    if m is not None:
        n = sum(q.numel() for q in m.parameters())
        need = n * (2 + 4 + 8) / 2**30  # bf16 weights, fp32 master, two fp32 moments
        free = float(prof.get("free_vram_gb") or 0.0)
        rep.update(parameters=n, training_state_gb=round(need, 3), feasible=bool(need + float(p["safety_margin_gb"]) <= free) if free else None)
    return {"feasibility_report": rep}


@studio_node("VRAMProfiler", "Runtime", {}, {"vram_stats": METRICS}, {"device": "cuda", "alert_threshold_gb": 0.0}, "device memory statistics")
def _vram(i, p, c):
    from ..runtime.vram import VRAMProfiler

    st = dict(VRAMProfiler.get_vram_stats(str(p.get("device", "cuda"))))
    thr = float(p.get("alert_threshold_gb") or 0.0)
    if thr > 0:
        used = float(st.get("allocated_gb") or st.get("used_gb") or 0.0)
        st["alert"] = used > thr
    return {"vram_stats": st}


@studio_node("PythonSandbox", "Runtime", {"code": TEXT}, {"result": ANY, "stdout": TEXT}, {"timeout": 10, "max_memory_mb": 256},
             "user code in an isolated interpreter (allow-listed imports, no dunder access)")
def _sandbox(i, p, c):
    from ..runtime.sandbox import PythonSandbox

    code = i.get("code") or p.get("code")
    if not isinstance(code, str) or not code.strip():
        raise NodeFailure("PythonSandbox needs code")
    res = PythonSandbox(timeout=float(p["timeout"]), max_memory_mb=int(p["max_memory_mb"])).execute_code(code, p.get("inputs") or {})
    if not res.get("success", False):
        raise NodeFailure(f"sandboxed code failed: {res.get('error') or res.get('stderr')}")
    return {"result": res.get("result"), "stdout": res.get("stdout", "")}


@studio_node("WandbLogger", "Runtime", {"metrics": METRICS}, {"log_status": METRICS}, {"step": 0}, "append metrics to a local JSON-lines run log")
def _wandb(i, p, c):
    m = _pick(i, c, "metrics")
    if m is None:
        raise NodeFailure("WandbLogger needs metrics")
    d = _out_dir(p, c, "runs")
    path = d / f"{p.get('project', 'dag')}.jsonl"
    rec = {"step": int(p.get("step", 0)), "time": time.time(), "metrics": summarise(m)}
    with open(path, "a", encoding="utf-8") as f:
        f.write(json.dumps(rec) + "\n")
    return {"log_status": {"logged": True, "path": str(path), "mode": "offline file (no network)", "step": rec["step"]}}


# ---------------------------------------------------------------------------------------------------- inference, agents
@studio_node("AutoregressiveGenerator", "Model", {"model_handle": MODEL, "prompt": TEXT}, {"generated_text": TEXT, "tokens_per_sec": METRICS},
             {"max_tokens": 64, "temperature": 0.7, "top_k": 40, "repetition_penalty": 1.1, "force_depth": None}, "sampled or greedy generation")
def _generator(i, p, c):
    from ..inference import generate_response

    m = _model(i, c)
    prompt = _pick(i, c, "prompt", "text", "text_sample")
    if not isinstance(prompt, str) or not prompt:
        raise NodeFailure("the generator needs a prompt")
    kw: Dict[str, Any] = {"max_new_tokens": int(p["max_tokens"]), "temperature": float(p["temperature"]), "template": bool(p.get("template", False))}
    if p.get("top_k") is not None:
        kw["top_k"] = int(p["top_k"])
    if p.get("repetition_penalty") is not None:
        kw["repetition_penalty"] = float(p["repetition_penalty"])
    if p.get("force_depth") not in (None, "", "auto"):
        kw["decode_depth"] = int(p["force_depth"])
    import inspect

    allowed = set(inspect.signature(generate_response).parameters)
    t0 = time.perf_counter()
    out = generate_response(m, _tokenizer(c, int(getattr(m, "vocab_size", 256))), prompt, **{k: v for k, v in kw.items() if k in allowed})
    dt = time.perf_counter() - t0
    n = len(out.get("tokens") or [])
    return {"generated_text": out["text"], "tokens_per_sec": {"tokens": n, "seconds": dt, "tok_s": n / dt if dt > 0 and n else None,
                                                               "telemetry": out.get("telemetry", {})}}


@studio_node("BYOKChatRouter", "Agent", {"prompt": TEXT}, {"provider_config": METRICS}, {"provider": "openai", "model": "gpt-4o-mini", "temperature": 0.7, "max_tokens": 512},
             "provider settings for a bring-your-own-key chat call (no request is sent from here)")
def _byok(i, p, c):
    cfg = {"provider": str(p["provider"]), "model": str(p["model"]), "temperature": float(p["temperature"]), "max_tokens": int(p["max_tokens"]),
           "has_key": bool(c.get("provider_keys", {}).get(str(p["provider"]))), "prompt_chars": len(i.get("prompt") or "")}
    return {"provider_config": cfg, "_specification": True}


@studio_node("RerouteNode", "Reroute", {"in": ANY}, {"out": ANY}, {"label": "reroute"},
             "a junction that passes its input on unchanged (keeps long wires of the canvas tidy)")
def _reroute(i, p, c):
    return {"out": i.get("in", next(iter(i.values()), None))}


# ---------------------------------------------------------------------------------------------------- training, evaluation
@studio_node("TrainingStep", "Evaluation", {"dataset_stream": STREAM, "model_handle": MODEL, "optimizer_handle": OPT, "tokens": TENSOR},
             {"step_metrics": METRICS, "loss": LOSS, "model_handle": MODEL}, {"grad_accum_steps": 1, "max_grad_norm": 1.0},
             "forward, backward, clip and optimizer step on the connected batch")
def _training_step(i, p, c):
    torch = _torch()
    m = _model(i, c)
    opt = _pick(i, c, "optimizer_handle", "optimizer")
    if opt is None:
        from ..optim import build_optimizer

        opt = build_optimizer(m, {"optimizer": "centroid_steer", "lr": float(p.get("lr", 1e-4))})
        _shared(c)["optimizer"] = opt
    x, y = _shared(c).get("input_ids"), _shared(c).get("targets")
    tok = _as_tokens(i.get("tokens"), c)
    if tok is not None:
        x, y = tok[:, :-1], tok[:, 1:]
    if x is None or y is None or x.shape != y.shape:
        if x is not None and x.shape[1] >= 2:
            x, y = x[:, :-1], x[:, 1:]
        else:
            raise NodeFailure("TrainingStep needs tokens (or a CyclingDataLoader upstream)")
    dev = next(m.parameters()).device
    x, y = x.to(dev).contiguous(), y.to(dev).contiguous()
    n = max(1, int(p["grad_accum_steps"]))
    depth = int(p.get("force_depth", 2))
    m.train()
    opt.zero_grad()
    t0 = time.perf_counter()
    total = 0.0
    for k in range(n):
        loss = m.forward_loss(x, y, force_depth=depth) if hasattr(m, "forward_loss") else _generic_lm_loss(m, x, y)
        (loss / n).backward()
        total += float(loss.detach()) / n
    gn = float(torch.nn.utils.clip_grad_norm_([q for q in m.parameters() if q.grad is not None], float(p["max_grad_norm"])))
    opt.step()
    dt = time.perf_counter() - t0
    metrics = {"loss": total, "grad_norm": gn, "tokens": int(x.numel()) * n, "seconds": dt, "tok_s": x.numel() * n / dt}
    lt = torch.tensor(total)
    _shared(c)["loss"] = lt
    return {"step_metrics": metrics, "loss": lt, "model_handle": m}


def _generic_lm_loss(m, x, y):
    import torch.nn.functional as F

    out = m(x)
    lg = out[0] if isinstance(out, tuple) else getattr(out, "logits", out)
    return F.cross_entropy(lg.reshape(-1, lg.shape[-1]).float(), y.reshape(-1))


@studio_node("PerplexityEvaluator", "Evaluation", {"model_handle": MODEL, "tokens": TENSOR, "targets": TENSOR, "exit_logits": TUPLE},
             {"perplexity": METRICS, "val_loss": LOSS, "per_exit_metrics": METRICS}, {}, "loss and perplexity at every exit", aliases=("Evaluation",))
def _evaluator(i, p, c):
    import torch.nn.functional as F

    torch = _torch()
    targets = _pick(i, c, "targets")
    exits = i.get("exit_logits")
    names = ("reflex", "limbic", "cortex")
    per: Dict[str, Any] = {}
    if isinstance(exits, (tuple, list)) and isinstance(targets, torch.Tensor):
        for nm, lg in zip(names, exits):
            T = min(lg.shape[-2], targets.shape[-1])
            l = float(F.cross_entropy(lg[..., :T, :].reshape(-1, lg.shape[-1]).float(), targets[..., :T].reshape(-1).to(lg.device)))
            per[nm] = {"loss": l, "perplexity": math.exp(min(l, 50.0))}
    else:
        m = _model(i, c)
        tok = _as_tokens(_pick(i, c, "tokens", "input_ids"), c)
        if tok is None or tok.shape[1] < 2:
            raise NodeFailure("the evaluator needs tokens, or exit logits with targets")
        dev = next(m.parameters()).device
        if isinstance(targets, torch.Tensor) and targets.shape == tok.shape:
            x, y = tok.to(dev), targets.to(dev)
        else:
            x, y = tok[:, :-1].to(dev).contiguous(), tok[:, 1:].to(dev).contiguous()
        was = m.training
        m.eval()
        try:
            with torch.no_grad():
                if hasattr(m, "forward_loss"):
                    for d, nm in enumerate(names):
                        l = float(m.forward_loss(x, y, force_depth=d))
                        per[nm] = {"loss": l, "perplexity": math.exp(min(l, 50.0))}
                else:
                    l = float(_generic_lm_loss(m, x, y))
                    per["cortex"] = {"loss": l, "perplexity": math.exp(min(l, 50.0))}
        finally:
            m.train(was)
    last = per[next(reversed(per))]
    mono = all(per[a]["loss"] >= per[b]["loss"] for a, b in zip(list(per)[:-1], list(per)[1:]))
    return {"perplexity": {"perplexity": last["perplexity"], "monotone_over_exits": mono}, "val_loss": torch.tensor(last["loss"]), "per_exit_metrics": per}


@studio_node("LoRAFineTuner", "Evaluation", {"model_handle": MODEL, "tokens": TENSOR}, {"finetuned_adapter": FILE, "final_loss": LOSS},
             {"rank": 8, "alpha": 16.0, "lr": 2e-4, "max_grad_norm": 1.0}, "a few LoRA steps on the connected tokens; saves the adapter")
def _lora_finetune(i, p, c):
    from ..trainer.finetune import LoRAConfig, TriuneFineTuner

    torch = _torch()
    m = _model(i, c)
    tok = _as_tokens(_pick(i, c, "tokens", "input_ids"), c)
    if tok is None or tok.shape[1] < 2:
        raise NodeFailure("LoRAFineTuner needs tokens")
    dev = next(m.parameters()).device
    x, y = tok[:, :-1].to(dev).contiguous(), tok[:, 1:].to(dev).contiguous()
    ft = TriuneFineTuner(m, LoRAConfig(rank=int(p["rank"]), alpha=float(p["alpha"])))
    params = [q for q in m.parameters() if q.requires_grad]
    opt = torch.optim.AdamW(params, lr=float(p["lr"]))
    m.train()
    loss_v = float("nan")
    for _ in range(max(1, int(p.get("steps", 3)))):
        opt.zero_grad()
        loss = m.forward_loss(x, y, force_depth=2) if hasattr(m, "forward_loss") else _generic_lm_loss(m, x, y)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, float(p["max_grad_norm"]))
        opt.step()
        loss_v = float(loss.detach())
    d = _out_dir(p, c, "adapters") / str(p.get("adapter_name", "dag_adapter"))
    ft.save_adapter(str(d))
    return {"finetuned_adapter": str(d), "final_loss": torch.tensor(loss_v), "_info": {"trainable": len(params)}}


# ---------------------------------------------------------------------------------------------------- export
@studio_node("SafeTensorsExport", "Export", {"model_handle": MODEL}, {"safetensors_file": FILE}, {"filename": "model.safetensors", "include_optimizer": False, "adapter_only": False},
             "weights as one .safetensors file", aliases=("Export",))
def _export_st(i, p, c):
    from ..export.exporter import export_model

    m = _model(i, c)
    path = _out_dir(p, c, "exports") / str(p["filename"])
    fmt = "lora" if p.get("adapter_only") else "safetensors"
    return {"safetensors_file": str(export_model(m, str(path), fmt))}


@studio_node("GGUFExport", "Export", {"model_handle": MODEL}, {"gguf_file": FILE}, {"quantization": "Q4_K_M", "filename": "model.gguf"},
             "GGUF export settings (configuration only: no file is written, as in the reference)")
def _export_gguf(i, p, c):
    # The multi-exit MoE layout has no GGUF architecture to be written as; the node records the settings a later
    # conversion would use, and reports itself as a specification node.
    return {"format": "GGUF (llama.cpp / Ollama)", "quantization": str(p.get("quantization", "Q4_K_M")), "filename": str(p.get("filename", "model.gguf")),
            "compatible_runtimes": ["Ollama", "llama.cpp", "LM Studio"], "real_computation": False, "_specification": True}


@studio_node("ONNXExport", "Export", {"model_handle": MODEL}, {"onnx_file": FILE}, {"opset_version": 17, "dynamic_axes": True}, "ONNX graph of the forward pass")
def _export_onnx(i, p, c):
    from ..export.exporter import export_model

    path = _out_dir(p, c, "exports") / str(p.get("filename", "model.onnx"))
    return {"onnx_file": str(export_model(_model(i, c), str(path), "onnx"))}


# ---------------------------------------------------------------------------------------------------- subgraphs
@studio_node("SubgraphInput", "Runtime", {}, {"value": ANY}, {"public_name": ""}, "one named value of the parent graph, inside a subgraph", dynamic_ports=True)
def _subgraph_input(i, p, c):
    name = p.get("public_name")
    offered = c.get("_subgraph_inputs", {})
    if not isinstance(name, str) or name not in offered:
        raise NodeFailure(f"subgraph input '{name}' was not supplied")
    return {"value": offered[name]}


@studio_node("Subgraph", "Runtime", {}, {}, {}, "a nested graph with declared input and output sockets", dynamic_ports=True)
def _subgraph(i, p, c):
    node = c["_node"]
    d = node.get("subgraph")
    if not isinstance(d, dict) or not isinstance(d.get("nodes"), list) or not isinstance(d.get("edges"), list):
        raise NodeFailure("a Subgraph node requires a nested nodes / edges graph")
    depth = int(c.get("_subgraph_depth", 0))
    if depth >= MAX_SUBGRAPH_DEPTH:
        raise NodeFailure(f"nested subgraph depth exceeds the limit ({MAX_SUBGRAPH_DEPTH})")
    missing = [str(s.get("name", "?")) for s in d.get("inputs", []) if isinstance(s, dict) and s.get("required", True) and s.get("name") not in i]
    if missing:
        raise NodeFailure(f"subgraph is missing required input(s): {', '.join(missing)}")
    child_ctx = {k: v for k, v in c.items() if not k.startswith("_")}
    child_ctx.update(_subgraph_depth=depth + 1, _subgraph_inputs=dict(i))
    res = StudioGraphRunner(c["_runner"].emit).run({"nodes": d["nodes"], "edges": d["edges"]}, child_ctx, _keep_values=True)
    if res["status"] == "failed":
        raise NodeFailure(f"subgraph '{node.get('title', node.get('id'))}' failed at '{res['failed_node']}': {res['error']}")
    out: Dict[str, Any] = {}
    for s in d.get("outputs", []):
        name, sn, sp = s.get("name"), s.get("source_node"), s.get("source_port")
        if not name or not sn or not sp:
            raise NodeFailure("each subgraph output must declare name, source_node and source_port")
        ports = res["_values"].get(sn, {})
        if sp not in ports:
            if s.get("required", True):
                raise NodeFailure(f"subgraph output '{name}' has no value from {sn}:{sp}")
            continue
        out[name] = ports[sp]
    out["_info"] = {"nested_nodes_executed": len(res["results"]), "outputs": [k for k in out]}
    return out


# ---------------------------------------------------------------------------------------------------- graph -> training settings
def compile_to_training(graph: Dict[str, Any]) -> Dict[str, Any]:
    """Read a canvas graph as a training recipe (``triune/api/routes.py:4200-4530``): the model node's architecture, a
    precision node, the optimizer node's hyper-parameters, the schedule, the loader's batch shape, the loss weights,
    gradient accumulation and clipping. Returns ``{"model": {...}, "run": {...}, "data": {...}, "applied": [...]}``; the
    caller decides what to do with it (the server applies it to the live engine state)."""
    if not isinstance(graph, dict) or not isinstance(graph.get("nodes"), list):
        raise StudioGraphError("a graph is an object with a nodes array")
    model: Dict[str, Any] = {}
    run: Dict[str, Any] = {}
    data: Dict[str, Any] = {}
    applied: List[str] = []

    def first(p, *keys):
        for k in keys:
            if p.get(k) is not None and p.get(k) != "":
                return p[k]
        return None

    for node in graph["nodes"]:
        if not isinstance(node, dict):
            continue
        kind, p = resolve_kind(node), node_params(node)
        if kind in ("TriuneTransformer", "Model"):
            for dst, keys, cast in (("num_layers", ("num_layers", "layers"), int), ("hidden_dim", ("hidden_dim", "hiddenDim", "dim"), int),
                                    ("num_heads", ("num_heads", "heads"), int), ("head_dim", ("head_dim", "headDim"), int),
                                    ("num_experts", ("num_experts", "experts_routed", "experts"), int), ("vocab_size", ("vocab_size",), int),
                                    ("use_fp8", ("use_fp8",), bool), ("use_fp4", ("use_fp4",), bool)):
                v = first(p, *keys)
                if v is not None:
                    model[dst] = cast(v)
            preset = first(p, "preset_id", "preset", "model_preset")
            if preset:
                model["preset"] = str(preset)
            dm = first(p, "depth_mode", "depth")
            if dm:
                run["depth_mode"] = str(dm).lower()
            bw = first(p, "balance_loss_weight", "balance_weight")
            if bw is not None:
                run["balance_coef"] = float(bw)
            prec = first(p, "precision", "dtype")
            if prec:
                run["precision"] = str(prec).lower()
            applied.append("model_architecture")
        elif kind in ("FP8Linear", "FP4Linear"):
            run["precision"] = "fp8" if kind == "FP8Linear" else "fp4"
            applied.append("precision")
        elif kind in ("CentroidSteerOptimizer", "MuonOptimizer", "AdamWOptimizer", "Optimizer"):
            name = {"CentroidSteerOptimizer": "centroid_steer", "MuonOptimizer": "muon", "AdamWOptimizer": "adamw"}.get(kind) or str(p.get("optimizer", "centroid_steer"))
            run["optimizer"] = name
            for k in ("lr", "weight_decay", "eps", "momentum", "steer_scale"):
                if p.get(k) is not None:
                    run[k if k != "momentum" else "muon_momentum"] = float(p[k])
            for k in ("ns_steps", "galore_rank"):
                if p.get(k) is not None:
                    run[k] = int(p[k])
            if isinstance(p.get("betas"), (list, tuple)) and len(p["betas"]) == 2:
                run["beta1"], run["beta2"] = float(p["betas"][0]), float(p["betas"][1])
            applied.append("optimizer")
        elif kind == "CosineLRScheduler":
            for k in ("warmup_steps", "total_steps"):
                if p.get(k) is not None:
                    run[k] = int(p[k])
            if p.get("min_lr_ratio") is not None:
                run["min_lr_ratio"] = float(p["min_lr_ratio"])
            applied.append("schedule")
        elif kind in ("CyclingDataLoader", "LocalFileReader", "Data"):
            for k in ("batch_size", "seq_len"):
                if p.get(k) is not None:
                    run[k] = int(p[k])
            fp = first(p, "file_path", "path")
            if fp:
                data["path"] = str(fp)
            applied.append("data")
        elif kind in ("HuggingFaceStreamer", "URLDatasetStreamer"):
            data["source"] = str(first(p, "dataset_name", "url") or "")
            if p.get("local_path"):
                data["path"] = str(p["local_path"])
            applied.append("data_source")
        elif kind == "JointExitLoss":
            run["depth_mode"] = "joint"
            run["exit_weights"] = [float(p.get("lambda_reflex", 0.3)), float(p.get("lambda_limbic", 0.5)), float(p.get("lambda_cortex", 1.0))]
            applied.append("joint_loss")
        elif kind in ("FastCrossEntropy", "Loss"):
            if p.get("label_smoothing") is not None:
                run["label_smoothing"] = float(p["label_smoothing"])
            if p.get("router_z_loss_weight") is not None:
                run["z_loss_coef"] = float(p["router_z_loss_weight"])
            applied.append("loss")
        elif kind == "RouterZLoss":
            if p.get("coeff") is not None:
                run["z_loss_coef"] = float(p["coeff"])
            applied.append("router_z_loss")
        elif kind in ("GradientAccumulator", "TrainingStep"):
            if p.get("grad_accum_steps") is not None:
                run["grad_accum_steps"] = int(p["grad_accum_steps"])
            if p.get("max_grad_norm") is not None:
                run["grad_clip"] = float(p["max_grad_norm"])
            applied.append("accumulation")
        elif kind == "LayerStreamingEngine":
            run["layer_streaming"] = True
            applied.append("layer_streaming")
        elif kind == "CheckpointManager":
            if p.get("save_dir"):
                run["checkpoint_dir"] = str(p["save_dir"])
            if p.get("keep_last_n") is not None:
                run["keep_last_n"] = int(p["keep_last_n"])
            applied.append("checkpoints")
    if "min_lr_ratio" in run and "lr" in run:
        run["min_lr"] = run["lr"] * run.pop("min_lr_ratio")
    return {"model": model, "run": run, "data": data, "applied": applied}
