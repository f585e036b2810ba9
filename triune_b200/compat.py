"""Import paths of the reference project, served by this framework.

``triune_b200.compat.install()`` registers a package named ``triune`` whose sub-packages (``triune.model``,
``triune.optim``, ``triune.kernels``, ``triune.runtime``, ``triune.trainer``, ``triune.data``, ``triune.export``,
``triune.api``, ``triune.agents``, ``triune.plugins``, ``triune.execution`` ...) export, under the names of the
reference's ``__init__`` files, the objects of this framework that do the same job. Scripts written against the
reference then run with one extra line at the top::

    import triune_b200.compat; triune_b200.compat.install()
    from triune.model import TriuneTransformer
    from triune.kernels import fast_chunk_gla, chunked_cross_entropy_from_hidden
    from triune.optim import CentroidSteerOptimizer

Nothing is copied: every name resolves, when first touched, to an object defined elsewhere in this package; the few
names that have no object of their own here (aliases such as ``Engine``, ``MemoryPlan``, ``muon_orthogonalize``, small
helpers such as ``rotate_half`` and ``is_main_process``, and the registry / engine classes that front
``execution/studio.py``) are defined below. ``coverage()`` lists, per reference package, which names resolve. If the real
``triune`` package is already imported, ``install`` refuses rather than shadow it.
"""

from __future__ import annotations

import importlib
import importlib.util
import os
import sys
import types
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

# reference package -> [(module of this framework, names exported under the same name)], plus renames {ref name: "module:attr"}
_SAME: Dict[str, List[Tuple[str, Tuple[str, ...]]]] = {
    "optim": [("optim.centroid", ("CentroidSteerOptimizer",)), ("optim.manifold", ("LowSpaceWeightProjector", "QuantumUnitaryOptimizer", "UnitaryManifoldOptimizer")),
              ("optim.muon", ("Muon",)), ("optim.factory", ("build_optimizer",))],
    "model": [("models.zoo", ("CANONICAL_MODEL_SPECS", "MODEL_REGISTRY", "ModelSpec", "build_model_from_spec", "get_model_spec", "load_model", "register_model")),
              ("models.transformer", ("TriuneTransformer",)), ("models.speculative", ("SelfSpeculativeGenerator",)), ("models.block", ("TransformerBlock",)),
              ("models.attention", ("HybridAttention", "VectorisedGLA")), ("models.moe", ("MoE_FFN", "RoutingResult")), ("models.norms", ("RMSNorm",)),
              ("models.rotary", ("RotaryEmbedding",)), ("models.router", ("GumbelSoftmaxRouter",)), ("models.quant_linear", ("FP4Linear", "FP8Linear")),
              ("models.factory", ("build_model",)), ("models.adapters", ("WeightTiedExitProjection", "attach_early_exits", "generate_adaptive")),
              ("models.manifold_embedding", ("UniversalAdaptiveEmbedding",)),
              ("models.jev", ("JEVLatentPredictor", "JEVObjective", "JEVExitRouter", "JEVRoutingResult", "TriuneLatentPredictor", "TriuneLatentObjective",
                              "TriuneContinuousExitRouter", "ContinuousLatentExitRouter", "JointEmbeddingObjective", "LatentPredictor"))],
    "runtime": [("runtime.memory_planner", ("MemoryEstimate", "MemoryPlanner")),
                ("runtime.resource_manager", ("DynamicResourceManager", "LiveVRAMMonitor", "AllotmentPlan", "HardwareProfile", "VRAMBudgetExceededError")),
                ("runtime.streaming", ("LayerStreamingEngine", "StreamingConfig", "enable_layer_streaming")), ("runtime.capabilities", ("PrecisionCapabilities",)),
                ("runtime.staging", ("ParameterStager", "StagingBuffer", "FP8StagingBuffer")), ("runtime.sandbox", ("PythonSandbox", "SandboxResult")),
                ("runtime.vram", ("VRAMProfiler", "AutoOffloader")), ("runtime.cuda_graph", ("CUDAGraphEngine",)), ("runtime.neuron_scope", ("NeuronScope",)),
                ("runtime.parallel_engine", ("ParallelEngine", "GLAPipelineBlock", "MoERoutingBlock"))],
    "ops": [("ops._c_bridge", ("NativeTriuneEngine", "get_native_c_info")),
            ("ops", ("gla", "muon_ns", "rmsnorm", "swiglu", "cross_entropy", "lora_linear")),
            ("runtime.neuron_scope", ("TIER_NAMES",)), ("kernels", ("FastChunkedCrossEntropyLoss",))],
    "agents": [("agents", ("Agent", "Tool", "ToolRegistry")), ("agents.extras", ("ProviderManager",))],
    "recipes": [("recipes", ("bf16_autocast", "build_fp8_precision_context", "build_precision_context", "build_mxfp8_precision_context"))],
    "trainer": [("trainer.engine", ("TrainingEngine",)), ("parallel.dist", ("DistributedContext", "setup_distributed", "cleanup_distributed", "all_reduce_tensor")),
                ("trainer.trainer", ("Trainer",)), ("trainer.logger", ("NullLogger", "WandbLogger")),
                ("trainer.finetune", ("LoRAConfig", "LoRALayer", "TriuneFineTuner", "list_adapters", "export_adapter"))],
    "kernels": [("kernels", ())],  # every public name of kernels.py, see _names_of
    "export": [("export.exporter", ("export_gguf", "export_onnx", "export_safetensors", "export_model")), ("export.hf_compat", ("export_to_huggingface",))],
    "api": [("serve", ("create_app", "run_server"))],
    "callbacks": [("callbacks.base", ("Callback", "CallbackList")), ("callbacks.telemetry", ("TelemetryCallback",)), ("callbacks.events", ("EventEmitter", "global_emitter"))],
    "configs": [("config", ("build_config", "validate_config"))],
    "data": [("data.dataloader", ("AsyncDevicePrefetcher", "CyclingDataLoader")), ("data.dynamic_tokenizer", ("DynamicTokenizer", "DynamicTokenizerOutput")),
             ("data.dataset", ("TokenStreamDataset", "build_dataloader")), ("data.tokenizer", ("TriuneTokenizer", "build_tokenizer", "load_tokenizer"))],
    "plugins": [("execution.dag", ("register_node",))],
    "execution": [],
    "modules": [],
    "utils": [],
}
_RENAMED: Dict[str, Dict[str, str]] = {
    "optim": {"AdamW8bit": "compat:AdamW8bit", "HAS_8BIT": "compat:HAS_8BIT", "zeropower_via_newtonschulz5": "compat:zeropower_via_newtonschulz5"},
    "model": {"TriuneModel": "compat:TriuneModel", "apply_rotary": "compat:apply_rotary", "rotate_half": "compat:rotate_half"},
    "runtime": {"MemoryPlan": "runtime.memory_planner:MemoryEstimate", "apply_layer_streaming_if_requested": "compat:apply_layer_streaming_if_requested"},
    "ops": {"is_native_c_available": "ops._c_bridge:is_available", "c_centroid_steer_update_f32": "ops._c_bridge:c_centroid_steer_update",
            "c_route_tiers_f32": "ops._c_bridge:c_route_tiers", "c_compute_neuron_heatmap_f32": "ops._c_bridge:c_neuron_heatmap",
            "c_gla_recurrent_step_f32": "ops._c_bridge:c_gla_recurrent_step", "muon_orthogonalize": "compat:muon_orthogonalize", "norm": "ops:rmsnorm", "rope": "ops:apply_rope",
            "batched_qr": "compat:batched_qr", "cholesky_qr": "compat:cholesky_qr", "subspace_projection": "compat:subspace_projection",
            "batched_subspace_projection": "compat:batched_subspace_projection", "triangular_steer_update": "compat:triangular_steer_update",
            "route_tiers": "compat:route_tiers",
            "gelu": "ops:gelu_tanh", "chunked_cross_entropy": "kernels:chunked_cross_entropy_from_hidden", "lora_forward": "kernels:fast_lora_forward",
            "upgrade": "models.universal:upgrade_model", "TIER_REFLEX": "compat:TIER_REFLEX", "TIER_LIMBIC": "compat:TIER_LIMBIC", "TIER_CORTEX": "compat:TIER_CORTEX"},
    "agents": {"AgentHarness": "compat:AgentHarness", "AgentMemoryStore": "compat:AgentMemoryStore", "SkillLibrary": "compat:SkillLibrary",
               "MultiAgentOrchestrator": "compat:MultiAgentOrchestrator", "build_integrated_toolbelt": "compat:build_integrated_toolbelt",
               "AgentSkill": "agents.extras:Skill", "BUILTIN_PERSONAS": "agents.harness:PERSONAS", "PersonaProfile": "agents.harness:PersonaSpec",
               "ProviderConfig": "agents.extras:Provider", "StateController": "compat:StateController", "CognitiveState": "compat:CognitiveState",
               "LearnedLesson": "compat:LearnedLesson", "ToolStats": "compat:ToolStats", "UserPreference": "compat:UserPreference"},
    "trainer": {"all_reduce_dict": "compat:all_reduce_dict", "merge_adapter_checkpoint": "compat:merge_adapter_checkpoint", "Engine": "trainer.engine:TrainingEngine", "DistributedTrainingEngine": "compat:DistributedTrainingEngine", "is_distributed": "compat:is_distributed",
                "get_rank": "compat:get_rank", "get_world_size": "compat:get_world_size", "get_local_rank": "compat:get_local_rank",
                "is_main_process": "compat:is_main_process", "wrap_distributed_model": "compat:wrap_distributed_model"},
    "configs": {"default_config": "compat:default_config"},
    "plugins": {"NodeRegistry": "compat:NodeRegistry", "NODE_REGISTRY": "compat:global_registry", "global_registry": "compat:global_registry",
                "node_registry": "compat:global_registry", "get_node_executor": "compat:get_node_executor", "list_registered_nodes": "compat:list_registered_nodes"},
    "execution": {"DAGParser": "compat:DAGParser", "ExecutionEngine": "compat:ExecutionEngine", "NodeExecutionError": "execution.studio:StudioGraphError"},
    "modules": {"ModuleManager": "compat:ModuleManager"},
}
# deeper import paths that scripts use directly: reference module -> module of this framework
_MODULE_ALIASES = {
    "model.transformer": "models.transformer", "model.moe": "models.moe", "model.attention": "models.attention", "model.router": "models.router",
    "model.config": "config", "optim.centroid": "optim.centroid", "optim.muon": "optim.muon", "trainer.finetune": "trainer.finetune",
    "trainer.engine": "trainer.engine", "runtime.streaming": "runtime.streaming", "runtime.sandbox": "runtime.sandbox",
    "runtime.gguf_loader": "runtime.gguf_loader", "runtime.model_scanner": "runtime.model_scanner", "data.tokenizer": "data.tokenizer",
    "data.dynamic_tokenizer": "data.dynamic_tokenizer", "data.dataset": "data.dataset", "data.dataloader": "data.dataloader", "export.exporter": "export.exporter",
    "export.hf_compat": "export.hf_compat", "profiling": "profiling", "desktop": "desktop", "packaging": "packaging", "cli": "cli",
    "api.server": "serve.server", "api.routes": "serve.routes", "api.srsm": "serve.srsm", "execution.dag": "compat", "kernels.fast_gla": "kernels",
    "kernels.fast_cross_entropy": "kernels", "kernels.fast_rmsnorm": "kernels", "kernels.fast_rope": "kernels", "kernels.fast_swiglu": "kernels",
    "kernels.fast_muon": "kernels", "kernels.fast_lora": "kernels", "kernels.fast_nvfp4": "kernels", "kernels.fast_fp8": "kernels",
}

# every other module path of the reference -> the modules of this framework its names are looked up in, in order ("compat":
# this module). Looked up when a name is first touched, so importing one of these paths imports nothing heavy.
_DEEP: Dict[str, Tuple[str, ...]] = {
    "agents._storage": ("compat",), "agents.engine": ("compat", "agents", "agents.extras"), "agents.memory": ("compat", "agents.extras"),
    "agents.personas": ("compat", "agents.harness"), "agents.providers": ("compat", "agents.extras"), "agents.skills": ("compat", "agents.extras"),
    "agents.tools": ("compat", "agents", "agents.harness", "agents.extras"),
    "callbacks.base": ("callbacks.base",), "callbacks.events": ("callbacks.events",), "callbacks.telemetry": ("callbacks.telemetry",),
    "cli_ui": ("cli_ui",), "inference": ("compat", "inference"), "trainer.checkpoint": ("compat", "trainer.checkpoint"), "configs.config": ("compat", "config"), "execution.dag": ("compat", "execution.dag", "execution.studio", "execution.nodes"),
    "kernels.dispatcher": ("kernels", "compat"), "kernels.fast_triangular": ("compat", "kernels"), "kernels.fast_muon": ("compat", "kernels"),
    "kernels.fast_nvfp4": ("compat", "kernels"),
    "model.adapters": ("models.adapters",), "model.base": ("models.zoo", "compat"), "model.block": ("models.block",),
    "model.config": ("compat", "config"), "model.early_exit": ("models.adapters", "models.transformer"), "model.factory": ("models.factory", "models.zoo"),
    "model.fp4": ("models.quant_linear", "kernels"), "model.fp8": ("models.quant_linear", "kernels"), "model.jev": ("models.jev",),
    "model.manifold_embedding": ("models.manifold_embedding",), "model.norms": ("models.norms",), "model.rotary": ("compat", "models.rotary"),
    "model.speculative": ("models.speculative",), "model.transmuter": ("models.transmuter",), "model.vectorised_gla": ("models.attention",),
    "model.zoo": ("models.zoo",), "modules.manager": ("compat", "execution.studio"), "modules.github_client": ("plugins.repo_search",),
    "modules.curated.custom_loss_nodes.custom_loss_nodes": ("plugins.curated.custom_loss_nodes.custom_loss_nodes",),
    "ops._c_bridge": ("compat", "ops._c_bridge"), "ops.centroid_steer": ("compat", "ops"), "ops.gla": ("compat", "ops", "kernels"), "ops.muon": ("compat", "ops"),
    "ops.norm": ("compat", "ops"), "ops.router": ("compat", "ops"), "ops.swiglu": ("compat", "ops"),
    "optim.factory": ("optim.factory",), "optim.manifold": ("optim.manifold",),
    "plugins.node_schema": ("compat", "execution.studio", "execution.dag"), "plugins.registry": ("compat", "execution.dag", "plugins.registry"),
    "recipes.bf16": ("recipes",), "recipes.fp8": ("recipes",), "recipes.mxfp8": ("recipes",), "recipes.nvfp4": ("recipes",),
    "runtime.capabilities": ("runtime.capabilities",), "runtime.cuda_graph": ("runtime.cuda_graph",), "runtime.disk_streaming": ("compat", "runtime.disk_streaming"),
    "runtime.memory_planner": ("compat", "runtime.memory_planner"), "runtime.neuron_scope": ("runtime.neuron_scope",),
    "runtime.parallel_engine": ("runtime.parallel_engine",), "runtime.resource_manager": ("runtime.resource_manager",), "runtime.staging": ("runtime.staging",),
    "runtime.vram": ("runtime.vram",), "trainer.callbacks": ("trainer.callbacks", "callbacks.base"), "trainer.distributed": ("compat", "parallel.dist"),
    "trainer.evaluation": ("trainer.evaluation",), "trainer.logger": ("trainer.logger",), "trainer.scheduler": ("trainer.scheduler",),
    "trainer.trainer": ("trainer.trainer",), "universal": ("compat", "models.universal"), "utils.device": ("compat", "utils"), "utils.seed": ("compat", "utils"),
}
# names of the reference's top-level package that are not simply a name of one of its sub-packages
_ROOT: Dict[str, str] = {"__version__": "compat:__version__", "Model": "models.factory:build_model", "Config": "config:build_config",
                         "CentroidSteer": "optim.centroid:CentroidSteerOptimizer", "UniversalDenseTransformer": "models.universal:UniversalDenseTransformer",
                         "UniversalMoETransformer": "models.universal:UniversalMoETransformer", "TriuneUniversalEngine": "models.universal:TriuneUniversalEngine",
                         "upgrade_model": "models.universal:upgrade_model", "upgrade": "models.universal:upgrade_model"}
# names that modules aliased one-to-one (``_MODULE_ALIASES``) lack here but the reference's module has
_ALIAS_FALLBACKS: Dict[str, Tuple[str, ...]] = {
    "api.routes": ("compat", "serve.routes_shell", "serve.engine_state"), "api.server": ("compat",), "inference": ("compat",), "cli": ("compat",),
    "packaging": ("compat",), "optim.centroid": ("compat", "optim.subspace"), "trainer.checkpoint": ("compat",), "runtime.model_scanner": ("compat",),
    "runtime.gguf_loader": ("compat",), "model.attention": ("compat", "ops.reference"), "model.moe": ("compat",), "model.transformer": ("compat",),
    "trainer.engine": ("compat",), "trainer.finetune": ("compat",), "runtime.streaming": ("compat", "runtime.staging"), "data.dynamic_tokenizer": ("compat",),
    "model.router": ("compat",), "optim.muon": ("compat",), "desktop": ("compat",), "profiling": ("compat",),
}

_PKG = __name__.rsplit(".", 1)[0]


def _resolve(target: str) -> Any:
    mod, _, attr = target.partition(":")
    m = sys.modules[__name__] if mod == "compat" else importlib.import_module(f"{_PKG}.{mod}" if mod else _PKG)
    return getattr(m, attr) if attr else m


def _names_of(pkg: str) -> Dict[str, str]:
    out: Dict[str, str] = {}
    for mod, names in _SAME.get(pkg, []):
        if not names:  # the whole public surface of that module
            names = tuple(getattr(importlib.import_module(f"{_PKG}.{mod}"), "__all__", ()))
        for n in names:
            out[n] = f"{mod}:{n}"
    out.update(_RENAMED.get(pkg, {}))
    return out


class _Lazy(types.ModuleType):
    """A module whose attributes are looked up in this framework when first touched."""

    def __init__(self, name: str, table: Dict[str, str], doc: str):
        super().__init__(name, doc)
        self.__dict__["_table"] = table
        self.__all__ = sorted(table)
        self.__path__ = []  # a package: sub-modules may be imported from it

    def __getattr__(self, name: str) -> Any:
        table = self.__dict__["_table"]
        if name not in table:
            for other in self.__dict__.get("_also", ()):  # the top-level package re-exports names of its sub-packages
                if name in other.__dict__["_table"]:
                    val = getattr(other, name)
                    setattr(self, name, val)
                    return val
            raise AttributeError(f"module {self.__name__!r} has no attribute {name!r}")
        try:
            val = _resolve(table[name])
        except Exception as e:
            raise AttributeError(f"{self.__name__}.{name} could not be resolved ({type(e).__name__}: {e})") from e
        setattr(self, name, val)
        return val

    def __dir__(self):
        return sorted(set(self.__dict__["_table"]) | set(super().__dir__()))


def _search(mods: Tuple[str, ...], name: str) -> Any:
    """``name`` from the first of ``mods`` (modules of this framework; "compat" is this one) that has it."""
    if name.startswith("__") and name.endswith("__"):
        raise AttributeError(name)
    for m in mods:
        try:
            mod = sys.modules[__name__] if m == "compat" else importlib.import_module(f"{_PKG}.{m}")
        except ImportError:
            continue
        if name in vars(mod):
            return vars(mod)[name]
        if m == "compat" and name in _LAZY_VALUES:
            return _LAZY_VALUES[name]()
    raise AttributeError(name)


def _engine_state():
    from .serve.engine_state import get_state

    return get_state()


def _attr(path: str) -> Callable[[], Any]:
    return lambda: _resolve(path)


# names of this module that are objects made (or imported) when first asked for
_LAZY_VALUES: Dict[str, Callable[[], Any]] = {
    "pytorch_state": _engine_state, "RealPyTorchEngineState": _attr("serve.engine_state:EngineState"),
    "ChatCompletionRequest": _attr("serve.routes:ChatRequest"), "FineTuneRequest": _attr("serve.routes:FinetuneRequest"),
    "ModelLoadRequest": _attr("serve.routes:LoadRequest"), "TrainingConfigRequest": _attr("serve.routes:TrainRequest"),
    "HAS_FASTAPI": lambda: importlib.util.find_spec("fastapi") is not None,
    "module_manager": lambda: _shared("module_manager", lambda: ModuleManager()),
    "AgentSkill": _attr("agents.extras:Skill"), "BUILTIN_PERSONAS": _attr("agents.harness:PERSONAS"), "PersonaProfile": _attr("agents.harness:PersonaSpec"),
    "ProviderConfig": _attr("agents.extras:Provider"), "IncrementalStreamingDecoder": _attr("inference:IncrementalStreamingDecoder"),
    "atomic_write_text": _attr("agents.storage:atomic_write_text"), "atomic_write_json": _attr("agents.storage:atomic_write_json"),
    "load_validated_json_dict": _attr("agents.storage:load_validated_json_dict"), "tokenize_terms": _attr("agents.storage:tokenize_terms"),
    "compute_tfidf_cosine_scores": _attr("agents.storage:compute_tfidf_cosine_scores"),
    "seed_everything": _attr("utils:seed_everything"), "device_diagnostic": _attr("utils:device_diagnostic"),
}
_SHARED: Dict[str, Any] = {}


def _shared(key: str, make: Callable[[], Any]) -> Any:
    if key not in _SHARED:
        _SHARED[key] = make()
    return _SHARED[key]


class _Deep(types.ModuleType):
    """A module path of the reference whose names are spread over one or more modules here."""

    def __init__(self, name: str, mods: Tuple[str, ...]):
        super().__init__(name, f"{name}: looked up in {', '.join(mods)} of {_PKG}")
        self.__dict__["_mods"] = mods
        self.__path__ = []

    def __getattr__(self, name: str) -> Any:
        try:
            val = _search(self.__dict__["_mods"], name)
        except AttributeError:
            val, found = None, False
            parent = self.__name__
            while "." in parent and not found:  # a name the enclosing package exports lives in one of its modules
                parent = parent.rpartition(".")[0]
                pm = sys.modules.get(parent)
                if isinstance(pm, _Lazy) and name in pm.__dict__["_table"]:
                    val, found = getattr(pm, name), True
            if not found:
                raise AttributeError(f"module {self.__name__!r} has no attribute {name!r}") from None
        setattr(self, name, val)
        return val


_PATCHED: List[types.ModuleType] = []  # modules of this framework that were given a fallback ``__getattr__`` by install()


def install(name: str = "triune", force: bool = False) -> types.ModuleType:
    """Register the alias package in ``sys.modules`` and return it. Idempotent; refuses to shadow a real package of that
    name that is already imported unless ``force``."""
    cur = sys.modules.get(name)
    if cur is not None and not isinstance(cur, _Lazy) and not force:
        raise RuntimeError(f"a real package named {name!r} is already imported; not shadowing it")
    if isinstance(cur, _Lazy):
        return cur
    root = _Lazy(name, dict(_ROOT), f"{name}: import paths of the reference, served by {_PKG}")
    sys.modules[name] = root
    subs = []
    for pkg in _SAME:
        sub = _Lazy(f"{name}.{pkg}", _names_of(pkg), f"{name}.{pkg} on {_PKG}")
        sys.modules[f"{name}.{pkg}"] = sub
        setattr(root, pkg, sub)
        subs.append(sub)
    root.__dict__["_also"] = subs
    for ref_mod, ours in _MODULE_ALIASES.items():
        full = f"{name}.{ref_mod}"
        if full in sys.modules:
            continue
        target = sys.modules[__name__] if ours == "compat" else importlib.import_module(f"{_PKG}.{ours}")
        sys.modules[full] = target
        parent, _, leaf = full.rpartition(".")
        if parent in sys.modules and isinstance(sys.modules[parent], _Lazy):
            if leaf not in sys.modules[parent].__dict__["_table"]:  # a function of the same name wins over its module, as in the reference
                sys.modules[parent].__dict__.setdefault(leaf, target)
        elif parent == name:
            setattr(root, leaf, target)
        extra = _ALIAS_FALLBACKS.get(ref_mod)
        if extra and ours != "compat" and "__getattr__" not in vars(target):
            target.__getattr__ = (lambda mods, modname: lambda attr: _fallback(mods, modname, attr))(extra, target.__name__)
            _PATCHED.append(target)
    for ref_mod, mods in _DEEP.items():
        full = f"{name}.{ref_mod}"
        if full in sys.modules:
            continue
        parts = ref_mod.split(".")
        for k in range(1, len(parts)):  # intermediate packages the reference has but nothing is imported from
            mid = f"{name}.{'.'.join(parts[:k])}"
            if mid not in sys.modules:
                sys.modules[mid] = _Deep(mid, ())
                setattr(sys.modules[mid.rpartition('.')[0]], parts[k - 1], sys.modules[mid])
        mod = _Deep(full, mods)
        sys.modules[full] = mod
        parent, _, leaf = full.rpartition(".")
        par = sys.modules[parent]
        if isinstance(par, _Lazy):
            if leaf not in par.__dict__["_table"]:
                par.__dict__.setdefault(leaf, mod)
        elif leaf not in vars(par):
            setattr(par, leaf, mod)
    return root


def _fallback(mods: Tuple[str, ...], modname: str, attr: str) -> Any:
    try:
        return _search(mods, attr)
    except AttributeError:
        raise AttributeError(f"module {modname!r} has no attribute {attr!r}") from None


def uninstall(name: str = "triune") -> None:
    """Remove the alias package again (a real package of that name is left alone)."""
    if not isinstance(sys.modules.get(name), _Lazy):
        return
    for k in [k for k in sys.modules if k == name or k.startswith(name + ".")]:
        del sys.modules[k]
    while _PATCHED:
        vars(_PATCHED.pop()).pop("__getattr__", None)


def coverage() -> Dict[str, Dict[str, Any]]:
    """Per reference package: the names it exports that resolve here, and the ones that do not."""
    rep: Dict[str, Dict[str, Any]] = {}
    for pkg in _SAME:
        ok, bad = [], {}
        for n, target in _names_of(pkg).items():
            try:
                _resolve(target)
                ok.append(n)
            except Exception as e:
                bad[n] = f"{type(e).__name__}: {e}"
        rep[pkg] = {"resolved": sorted(ok), "unresolved": bad}
    return rep


__version__ = "1.0.0"
TIER_REFLEX, TIER_LIMBIC, TIER_CORTEX = 0, 1, 2


# ---------------------------------------------------------------------------------------------------- model helpers
class TriuneModel(nn.Module):
    """Base of model classes registered in the zoo: ``forward(input_ids, force_depth) -> (logits, aux)`` and a parameter
    count (``triune/model/base.py:474-487``)."""

    def forward(self, input_ids: torch.Tensor, force_depth: Optional[int] = None):  # pragma: no cover - interface
        raise NotImplementedError

    def get_num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """(x1, x2) -> (-x2, x1) over the two halves of the last dimension."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(q, k) -> (q cos + rotate_half(q) sin, k cos + rotate_half(k) sin) with tables that broadcast against them."""
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def apply_layer_streaming_if_requested(model: nn.Module, device, config: Dict[str, Any], optimizer: Optional[Any] = None):
    """Attach a layer-streaming engine when ``config["streaming"]`` is set (the reference's flat ``streaming_*`` keys)."""
    if not config.get("streaming", False):
        return None
    from .runtime.streaming import StreamingConfig, enable_layer_streaming

    cfg = StreamingConfig(enabled=True, chunk_size=int(config.get("streaming_chunk_size", 1)), pin_memory=config.get("streaming_pin_memory"),
                          async_prefetch=bool(config.get("streaming_prefetch", True)), fp8_weights=bool(config.get("streaming_fp8_weights", False)),
                          resident_gpu_layers=int(config.get("streaming_resident_gpu_layers", 0)), grad_clip=float(config.get("grad_clip", 1.0)),
                          instant_optimizer=True, forward_snapshots=bool(config.get("streaming_capture_forward_snapshots", True)),
                          activation_checkpointing=bool(config.get("streaming_activation_checkpointing", True)))
    return enable_layer_streaming(model, device, cfg)


def default_config() -> Dict[str, Any]:
    from .config import build_config

    return build_config({})


# ---------------------------------------------------------------------------------------------------- optimizer
HAS_8BIT = True  # 8-bit moments are part of this framework (``optim/adam8bit.py``); no external package is involved


def AdamW8bit(params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
    from .optim.adam8bit import AdamW8bit as _Impl

    return _Impl(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)



# ---------------------------------------------------------------------------------------------------- operator signatures
def muon_orthogonalize(G: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    from . import ops

    return ops.muon_ns(G, steps)


def zeropower_via_newtonschulz5(G: torch.Tensor, steps: int = 5, eps: float = 1e-7, scratch_buffer: Any = None, return_scratch: bool = False):
    from . import ops

    X = ops.muon_ns(G, steps)
    return (X, scratch_buffer) if return_scratch else X


def triangular_steer_update(P: torch.Tensor, Grad_proj: torch.Tensor, steer_scale: float = 1.0, momentum: float = 0.9, retract_stiefel: bool = False) -> torch.Tensor:
    """The reference's argument order (scale before momentum); optionally retracts the result onto orthonormal columns."""
    from . import ops

    out = ops.triangular_steer_update(P, Grad_proj, momentum, steer_scale)
    if retract_stiefel:
        from .optim.subspace import polar_stiefel_retraction

        out = polar_stiefel_retraction(out)
    return out


def route_tiers(logits: torch.Tensor, reflex_threshold: float = 0.70) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (probabilities [B, 3], selected tier [B])."""
    from . import ops

    return torch.softmax(logits.float(), dim=-1), ops.route_tiers(logits.float(), reflex_threshold)


def batched_qr(Y_mat: torch.Tensor, cond_threshold: float = 1e4, eps_shift: float = 1e-7, orth_tol: float = 1e-4, return_fallback_mask: bool = False,
               return_diagnostics: bool = False, out_dtype: Optional[torch.dtype] = None):
    from .optim.subspace import batched_qr as _qr

    Q, info = _qr(Y_mat, cond_threshold, eps_shift, orth_tol, return_info=True)
    if out_dtype is not None:
        Q = Q.to(out_dtype)
    if return_diagnostics:
        return Q, info
    if return_fallback_mask:
        return Q, info["fallback_mask"]
    return Q


def cholesky_qr(Y_f: torch.Tensor, cond_threshold: float = 1e4, eps_shift: float = 1e-7, orth_tol: float = 1e-4) -> torch.Tensor:
    return batched_qr(Y_f, cond_threshold, eps_shift, orth_tol)


def subspace_projection(grad: torch.Tensor, rank: int, niter: int = 2, cond_threshold: float = 1e4, eps_shift: float = 1e-7, orth_tol: float = 1e-4) -> torch.Tensor:
    from .optim.subspace import subspace_projection as _sp

    return _sp(grad, rank, power_iters=max(0, int(niter) - 1))


def batched_subspace_projection(grads: torch.Tensor, rank: int, niter: int = 2, cond_threshold: float = 1e4, eps_shift: float = 1e-7, orth_tol: float = 1e-4,
                                return_diagnostics: bool = False):
    """-> (bases [K, d, rank], name of the path taken) and, on request, per-call diagnostics."""
    from .optim.subspace import batched_subspace_projection as _bsp
    from .optim.subspace import flush_qr_telemetry, new_qr_telemetry  # noqa: F401

    Q = _bsp(grads, rank, power_iters=max(0, int(niter) - 1))
    path = "batched_scholqr2"
    return (Q, path, []) if return_diagnostics else (Q, path)


def fast_subspace_projection(grad: torch.Tensor, rank: int, niter: int = 2, cond_threshold: float = 1e4, eps_shift: float = 1e-7,
                            orth_tol: float = 1e-4) -> Tuple[torch.Tensor, str]:
    """-> (orthonormal basis of the dominant subspace on the short side of ``grad``, "left" or "right")."""
    m, n = grad.shape
    return subspace_projection(grad, rank, niter, cond_threshold, eps_shift, orth_tol), ("left" if m <= n else "right")


def polar_stiefel_retraction(P: torch.Tensor, eps: float = 1e-7) -> torch.Tensor:
    """``P [.., d, r]`` with its columns made orthonormal again (Cholesky QR with its condition check and Householder
    fall-back); the span is kept."""
    return batched_qr(P.float(), eps_shift=eps).to(P.dtype)


def generate_response(model, tokenizer, prompt: str, *, device=None, pad_token_id: Optional[int] = None, eos_token_id: Optional[int] = None,
                      force_depth: Optional[int] = None, temperature: float = 0.7, top_k: int = 50, repetition_penalty: float = 1.1,
                      max_new_tokens: int = 100, prompt_is_formatted: bool = False, cancel_event=None, on_text=None, return_info: bool = False,
                      cache=None):
    """``inference.generate_response`` under the reference's keyword-only signature (``triune/inference.py:833-1052``):
    returns the reply text, or with ``return_info`` a dict with the text, token count, rates, latencies, the exit tier
    that decoded and the cache."""
    import time

    from .inference import generate_response as _gen

    if temperature < 0:
        raise ValueError("temperature must be non-negative")
    if top_k <= 0:
        raise ValueError("top_k must be a positive integer")
    if repetition_penalty <= 0:
        raise ValueError("repetition_penalty must be greater than zero")
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be positive")
    t0 = time.perf_counter()
    out = _gen(model, tokenizer, prompt, max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k,
               repetition_penalty=repetition_penalty, decode_depth=force_depth, stream_callback=on_text, cancel_event=cancel_event, cache=cache,
               template=not prompt_is_formatted, device=device, eos_token_id=eos_token_id, pad_token_id=pad_token_id)
    text = out["text"].strip()
    if not return_info:
        return text
    dt = max(1e-9, time.perf_counter() - t0)
    tele, n = out["telemetry"], len(out["tokens"])
    depth = force_depth if force_depth is not None else tele.get("depth")
    route = ("REFLEX", "LIMBIC", "CORTEX")[int(depth)] if isinstance(depth, int) and 0 <= depth <= 2 else "AUTO"
    return {"text": text, "tokens_count": n, "tokens_per_sec": n / dt, "latency_ms": round(dt * 1e3, 1),
            "ttft_ms": round(1e3 * float(tele.get("ttft_s", 0.0)), 1), "decode_tokens_per_sec": round(float(tele.get("decode_tok_s", 0.0)), 2),
            "route": route, "cancelled": bool(cancel_event is not None and cancel_event.is_set()), "cache": out["cache"]}


def build_nvfp4_disk_cache(model_id_or_dir, cache_dir=None, *, hadamard: bool = True, protect_sensitive: bool = True, quantize_lm_head: bool = False,
                           compute_device=None, force: bool = False, local_files_only: bool = False):
    """-> the cache directory (the reference's return value; this framework's own function returns the manifest)."""
    from .runtime import disk_streaming as ds

    src = ds.resolve_hf_model_dir(model_id_or_dir, local_files_only=local_files_only)
    target = ds.Path(cache_dir) if cache_dir is not None else ds.default_nvfp4_cache_dir(src, hadamard)
    ds.build_nvfp4_disk_cache(src, target, hadamard=hadamard, protect_sensitive=protect_sensitive, quantize_lm_head=quantize_lm_head,
                              device=None if compute_device is None else str(compute_device), force=force)
    return target


def _save_for_trainer(which: str, trainer, engine, step: int, loss: float):
    from pathlib import Path

    from .trainer import checkpoint as ck

    fn = ck.save_latest if which == "latest" else ck.save_best
    if isinstance(trainer, (str, os.PathLike)):  # this framework's own calling form
        return fn(trainer, **({} if engine is None else {"model": engine}))
    best = getattr(engine, "best_eval_loss", None)
    return Path(fn(str(trainer.config["checkpoint_dir"]), model=trainer.model, optimizer=getattr(trainer, "optimizer", None), step=step, loss=loss,
                   best_eval_loss=float("inf") if best is None else float(best), config=dict(getattr(trainer, "config", {}) or {}),
                   depth_usage_ema=getattr(engine, "depth_usage_ema", None), wandb_run_id=getattr(getattr(trainer, "logger", None), "run_id", None)))


def save_latest(trainer, engine=None, step: int = 0, loss: float = 0.0):
    """``latest.pt`` in the trainer's checkpoint directory (``triune/trainer/checkpoint.py:138-146`` of the reference)."""
    return _save_for_trainer("latest", trainer, engine, step, loss)


def save_best(trainer, engine=None, step: int = 0, loss: float = 0.0):
    return _save_for_trainer("best", trainer, engine, step, loss)


def load_checkpoint(trainer, path=None, *, load_optimizer: bool = True, **kw):
    """``load_checkpoint(trainer, path, load_optimizer=...)`` of the reference: restores the trainer's model (and
    optimizer) after the fingerprint check against the trainer's configuration, and returns the checkpoint dict. A path
    as first argument is this framework's own calling form and is passed through."""
    from .trainer import checkpoint as ck

    if isinstance(trainer, (str, os.PathLike)):
        return ck.load_checkpoint(trainer, *(() if path is None else (path,)), **kw)
    cfg = getattr(trainer, "config", None)
    return ck.load_checkpoint(str(path), model=trainer.model, optimizer=getattr(trainer, "optimizer", None) if load_optimizer else None,
                              config=dict(cfg) if isinstance(cfg, dict) else None)


def all_reduce_dict(metrics: Dict[str, float], op: Any = None) -> Dict[str, float]:
    """Average (the default) or sum of scalar metrics over the ranks."""
    from .parallel.dist import all_reduce_dict as _ard

    out = _ard({k: float(v) for k, v in metrics.items()})
    if op is not None and "SUM" in str(op).upper():
        out = {k: v * get_world_size() for k, v in out.items()}
    return out


def merge_adapter_checkpoint(adapter_path, checkpoint_path, output_path=None, tokenizer_path="triune_tokenizer.json"):
    """Load the checkpoint's model, fold the adapter into its weights, write a checkpoint of the merged model; -> its path."""
    from pathlib import Path

    from .inference import load_checkpoint_model
    from .trainer.checkpoint import save_checkpoint
    from .trainer.finetune import merge_adapter_checkpoint as _merge

    model = load_checkpoint_model(str(checkpoint_path))[0]
    _merge(model, adapter_path)
    out = Path(output_path) if output_path else Path(checkpoint_path).with_name(Path(checkpoint_path).stem + "_merged.pt")
    save_checkpoint(str(out), model=model, step=0, config={})
    return out


# ---------------------------------------------------------------------------------------------------- agents, reference signatures
def AgentMemoryStore(store_dir="checkpoints/agent_harness"):
    from pathlib import Path

    from .agents.extras import AgentMemoryStore as _Impl

    return _Impl(str(Path(store_dir) / "memory.json"))


def SkillLibrary(store_dir="checkpoints/agent_harness/skills", extra_skill_dirs=None):
    from pathlib import Path

    from .agents.extras import SkillLibrary as _Impl

    Path(store_dir).mkdir(parents=True, exist_ok=True)
    lib = _Impl(str(store_dir))
    for d in extra_skill_dirs or []:
        if Path(d).is_dir():
            lib.load_directory(str(d))
    return lib


def build_integrated_toolbelt(*, workspace=".", memory=None, skills=None, state_controller=None, subagent_runner=None, allow_shell: bool = False,
                              allow_writes: bool = True, allow_local_http: bool = False):
    """The workspace-confined tools (read-only unless ``allow_writes``; a shell only with ``allow_shell``); requests to
    loopback or private addresses stay refused whatever ``allow_local_http`` says."""
    from .agents import Tool
    from .agents.harness import workspace_tools

    reg = workspace_tools(str(workspace), read_only=not allow_writes, allow_shell=allow_shell)
    if memory is not None:
        reg.register(Tool("remember", "keep a note for later runs", lambda text: (memory.add_lesson(str(text)), memory.save(), "noted")[2], {"text": "str"}))
        reg.register(Tool("recall", "notes of earlier runs that match a query", lambda query: [t for _, t in memory.recall(str(query))], {"query": "str"}))
    if subagent_runner is not None:
        reg.register(Tool("delegate", "hand a sub-task to another persona", lambda task, persona=None: subagent_runner(str(task), persona), {"task": "str", "persona": "str"}))
    return reg


from .agents.harness import AgentHarness as _HarnessImpl  # noqa: E402


class AgentHarness(_HarnessImpl):
    """The reference's keyword-only constructor over ``agents.harness.AgentHarness``. ``completion_fn(prompt=...)`` returns
    the text (or a dictionary with a ``text`` / ``content`` entry); without it ``model`` names a local model that is loaded
    on first use."""

    def __init__(self, *, workspace=".", store_dir="checkpoints/agent_harness", model: Optional[str] = None, allow_shell: bool = False,
                 allow_writes: bool = True, allow_local_http: bool = False, completion_fn: Optional[Callable[..., Any]] = None, providers=None,
                 depth: int = 0, persona: str = "auto", max_steps: int = 3):
        state: Dict[str, Any] = {}

        def generate(prompt: str) -> str:
            if completion_fn is not None:
                out = completion_fn(prompt=prompt)
                return out if isinstance(out, str) else str(out.get("text") or out.get("content") or "")
            if "st" not in state:
                from .serve.engine_state import EngineState

                state["st"] = EngineState()
                state["st"].load_model(model or "triune-nano")
            return state["st"].generate(prompt, max_new_tokens=256, template=False)["text"]

        super().__init__(generate, str(store_dir), workspace=str(workspace), persona=persona, read_only=not allow_writes, allow_shell=allow_shell,
                         max_steps=max_steps)
        self.providers, self.depth = providers, depth


class MultiAgentOrchestrator:
    """Specialists that take a goal in turn (``execute``) or side by side (``execute_parallel``) through one harness."""

    def __init__(self, harness=None):
        self.harness = harness
        self.team: List[str] = []

    def add_agent(self, persona: str) -> None:
        if persona not in self.team:
            self.team.append(persona)

    def execute_pipeline(self, goal: str, personas: Optional[List[str]] = None) -> List[Dict[str, Any]]:
        return self.execute(goal, list(personas or self.team))

    def orchestrate_team(self, goal: str, personas: Optional[List[str]] = None, parallel: bool = False, max_workers: int = 4) -> Dict[str, Any]:
        names = list(personas or self.team)
        steps = self.execute_parallel(goal, names, max_workers) if parallel else self.execute(goal, names)
        return {"goal": goal, "team": names, "parallel": bool(parallel), "steps": steps, "final": steps[-1]["text"] if steps else ""}

    def execute(self, goal: str, personas: List[str]) -> List[Dict[str, Any]]:
        return self.harness.run_team(goal, list(personas))

    def execute_parallel(self, goal: str, personas: List[str], max_workers: int = 4) -> List[Dict[str, Any]]:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=max(1, int(max_workers))) as ex:
            outs = list(ex.map(lambda p: {"agent": p, **self.harness.run(goal, persona=p)}, personas))
        return outs


# ---------------------------------------------------------------------------------------------------- distributed helpers
def is_distributed() -> bool:
    import torch.distributed as dist

    return dist.is_available() and dist.is_initialized()


def get_rank() -> int:
    import torch.distributed as dist

    return dist.get_rank() if is_distributed() else int(os.environ.get("RANK", 0))


def get_world_size() -> int:
    import torch.distributed as dist

    return dist.get_world_size() if is_distributed() else int(os.environ.get("WORLD_SIZE", 1))


def get_local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", 0))


def is_main_process() -> bool:
    return get_rank() == 0


def wrap_distributed_model(model: nn.Module, device_ids: Optional[List[int]] = None, find_unused_parameters: bool = True):
    """DistributedDataParallel around the model (the library baseline; this framework's own data parallelism is
    ``parallel.data_parallel.ShardedDataParallel``, which the trainer uses when given a ``dp`` object)."""
    if not is_distributed():
        raise RuntimeError("Cannot wrap model in DDP when distributed mode is not initialized.")
    from torch.nn.parallel import DistributedDataParallel as DDP

    return DDP(model, device_ids=device_ids, find_unused_parameters=find_unused_parameters, broadcast_buffers=False)


from .trainer.engine import TrainingEngine as _TrainingEngine  # noqa: E402


class DistributedTrainingEngine(_TrainingEngine):
    """``TrainingEngine`` whose step results also carry the loss and token count reduced over all ranks
    (``global_loss``, ``global_lm_loss``, ``global_tokens``; ``triune/trainer/distributed.py:159-181``)."""

    def __init__(self, trainer):
        super().__init__(trainer)
        self.is_distributed = is_distributed()

    def step_once(self, *a, **k):
        res = super().step_once(*a, **k)
        if self.is_distributed and isinstance(res, dict):
            red = all_reduce_dict({"loss": float(res.get("loss", 0.0)), "lm_loss": float(res.get("lm", res.get("loss", 0.0))), "tokens": float(res.get("tokens", 0))})
            res["global_loss"], res["global_lm_loss"], res["global_tokens"] = red["loss"], red["lm_loss"], int(red["tokens"])
        return res


# ---------------------------------------------------------------------------------------------------- agents records
class UserPreference(dict):
    """One stored preference: ``{"key", "value", "updated"}``."""


class LearnedLesson(dict):
    """One stored lesson: ``{"text", "tags", "time"}``."""


class ToolStats(dict):
    """Per-tool counters: ``{"calls", "failures", "seconds"}`` with the derived figures the reference's record offers."""

    @property
    def success_rate(self) -> float:
        c = float(self.get("calls", 0))
        return (c - float(self.get("failures", 0))) / c if c else 0.0

    @property
    def avg_latency_ms(self) -> float:
        c = float(self.get("calls", 0))
        return 1e3 * float(self.get("seconds", 0.0)) / c if c else 0.0

    @property
    def calibrated_reliability(self) -> float:
        """Success rate shrunk towards one half while there are few calls (one prior success and one prior failure)."""
        c = float(self.get("calls", 0))
        return (c - float(self.get("failures", 0)) + 1.0) / (c + 2.0)


class CognitiveState(dict):
    """What the state controller reports: persona, depth tier, temperature."""


class StateController:
    """Chooses persona and depth for a goal (``triune/agents/personas.py``): persona by the goal's words, depth by its
    length (short questions leave at the Reflex exit, long tasks use the full depth)."""

    def __init__(self, store_dir=None, persona: str = "auto", depth: str = "auto"):
        self.store_dir, self.persona, self.depth = store_dir, persona, depth

    # ---- persona book-keeping under the reference's method names
    def register_persona(self, name: str, system_prompt: str, temperature: float = 0.7, keywords=()) -> None:
        from .agents.harness import PERSONAS, PersonaSpec

        PERSONAS[name.lower()] = PersonaSpec(name.lower(), system_prompt, float(temperature), tuple(keywords))

    def delete_persona(self, name: str) -> bool:
        from .agents.harness import PERSONAS

        return PERSONAS.pop(name.lower(), None) is not None

    def shift(self, persona: str) -> CognitiveState:
        """Switch to a persona by name and report the new state."""
        self.persona = persona
        return self.assess("")

    def adapt_for_goal(self, goal: str) -> CognitiveState:
        return self.assess(goal)

    def adapt_after_tool(self, tool: str, ok: bool) -> CognitiveState:
        """A failing tool call moves an automatic persona to the debugger for the rest of the goal."""
        if not ok and self.persona in ("auto", ""):
            self.persona = "debugger"
        return self.assess("")

    @property
    def active_profile(self):
        from .agents.harness import DEFAULT_PERSONA, PERSONAS

        return PERSONAS.get(self.persona.lower(), DEFAULT_PERSONA)

    def assess(self, goal: str) -> CognitiveState:
        from .agents.harness import resolve_persona

        p = resolve_persona(self.persona, goal)
        words = len(goal.split())
        depth = self.depth if self.depth != "auto" else ("reflex" if words < 8 else "limbic" if words < 40 else "cortex")
        return CognitiveState(persona=p.name, system_prompt=p.system_prompt, temperature=p.temperature, depth=depth,
                              force_depth={"reflex": 0, "limbic": 1, "cortex": 2}[depth])


# ---------------------------------------------------------------------------------------------------- node registry, DAG engine
class NodeRegistry:
    """The node catalogue behind the canvas (``triune/plugins/registry.py:46-176``): built-in kinds come from
    ``execution/studio.py``; ``register`` adds a kind with a handler ``(inputs, params, context) -> outputs``."""

    def register_builtin_nodes(self) -> None:
        from .execution import studio  # noqa: F401 - importing registers the built-in kinds

    def register(self, name: str, handler: Callable, inputs: Optional[Dict[str, str]] = None, outputs: Optional[Dict[str, str]] = None,
                 category: str = "Custom", parameters: Optional[Dict[str, Any]] = None, description: str = "") -> None:
        from .execution.studio import studio_node

        studio_node(name, category, inputs or {}, outputs or {}, parameters or {}, description)(handler)

    def get(self, name: str):
        from .execution.studio import STUDIO_NODES

        return STUDIO_NODES.get(name)

    def get_catalog(self) -> List[Dict[str, Any]]:
        from .execution.studio import studio_catalog

        return studio_catalog()

    def list_nodes(self) -> List[str]:
        return sorted(n["name"] for n in self.get_catalog())

    def get_core_node_names(self) -> List[str]:
        """The built-in kinds (everything except ``Custom`` registrations)."""
        return sorted(n["name"] for n in self.get_catalog() if n["category"] != "Custom")

    def get_node(self, name: str) -> Optional[Dict[str, Any]]:
        return next((n for n in self.get_catalog() if n["name"] == name), None)

    def get_schema(self, name: str) -> Optional[Dict[str, Any]]:
        n = self.get_node(name)
        return None if n is None else {"inputs": n["typed_inputs"], "outputs": n["typed_outputs"], "parameters": n["parameters"]}

    def __contains__(self, name: str) -> bool:
        return self.get(name) is not None


global_registry = NodeRegistry()


def list_registered_nodes() -> List[str]:
    return sorted(n["name"] for n in global_registry.get_catalog())


def get_node_executor(name: str) -> Optional[Callable]:
    spec = global_registry.get(name)
    return None if spec is None else spec.fn


class DAGParser:
    """Validation and ordering of canvas graphs (``triune/execution/dag.py:39-216``)."""

    @classmethod
    def parse(cls, graph_json: Dict[str, Any]) -> Dict[str, Any]:
        from .execution.studio import parse_studio_graph

        g = parse_studio_graph(graph_json)
        adj: Dict[str, List[str]] = {}
        for e in g.edges:
            adj.setdefault(e["source"], []).append(e["target"])
        return {"execution_order": g.order, "node_map": g.nodes, "adj": adj}

    @classmethod
    def from_json(cls, graph_json: Dict[str, Any]) -> Dict[str, Any]:
        from .execution.studio import parse_studio_graph

        g = parse_studio_graph(graph_json)
        deps: Dict[str, List[str]] = {n: [] for n in g.nodes}
        for e in g.edges:
            deps[e["target"]].append(e["source"])
        return {n: {"id": n, "type": node.get("type"), "details": node.get("details"), "dependencies": deps[n]} for n, node in g.nodes.items()}


class ExecutionEngine:
    """Runs canvas graphs (``triune/execution/dag.py:271-3160``): ``execute_graph`` / ``run`` for whole graphs,
    ``execute_node`` / ``execute_single_node`` for one node, event callbacks per node, extra handlers by name."""

    def __init__(self):
        self.event_callbacks: List[Callable[[Dict[str, Any]], None]] = []

    def register_event_callback(self, cb) -> None:
        if cb not in self.event_callbacks:
            self.event_callbacks.append(cb)

    def unregister_event_callback(self, cb) -> None:
        if cb in self.event_callbacks:
            self.event_callbacks.remove(cb)

    def _emit(self, ev: Dict[str, Any]) -> None:
        for cb in list(self.event_callbacks):
            try:
                cb(ev)
            except Exception:
                pass

    def register_handler(self, node_type: str, handler: Callable) -> None:
        """``handler(node, context) -> dict`` in the reference's convention: ``context["current_inputs"]`` holds the port
        values; the returned dictionary's entries become the node's output ports."""
        def adapted(inputs, params, ctx):
            context = {"current_inputs": dict(inputs), "port_data": {}, **{k: v for k, v in ctx.items() if not k.startswith("_")}}
            out = handler(dict(ctx.get("_node") or {}, params=params), context) or {}
            if out.get("status") in ("failed", "error"):
                from .execution.studio import NodeFailure

                raise NodeFailure(str(out.get("error", "node reported failure")))
            ports = dict(context["port_data"].get((ctx.get("_node") or {}).get("id"), {}))
            return {**ports, "_info": {k: v for k, v in out.items() if k not in ports}}

        global_registry.register(node_type, adapted, category="Custom")
        from .execution.studio import STUDIO_NODES

        STUDIO_NODES[node_type].dynamic_ports = True

    def execute_graph(self, graph_json: Dict[str, Any], *, initial_context: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        from .execution.studio import StudioGraphRunner

        return StudioGraphRunner(self._emit).run(graph_json, dict(initial_context or {}))

    def run(self, graph_json: Dict[str, Any]) -> Dict[str, Any]:
        return self.execute_graph(graph_json)["results"]

    def execute_node(self, node_or_name, inputs: Optional[Dict[str, Any]] = None, context: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        from .execution.studio import run_studio_node

        node = {"type": node_or_name, "title": node_or_name} if isinstance(node_or_name, str) else dict(node_or_name)
        return run_studio_node(node, inputs, context)

    def execute_single_node(self, node: Dict[str, Any], context: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        return self.execute_node(node, None, context)


from .execution.studio import StudioGraphError as NodeExecutionError  # noqa: E402  (the error type graph validation raises)


# ---------------------------------------------------------------------------------------------------- modules
class ModuleManager:
    """Life cycle of local modules (plugin directories with signed manifests) inside one directory: install from a local
    directory, list, activate (verify and load), uninstall, scaffold. Remote catalogues are not contacted
    (``triune/modules/manager.py:345-1757`` of the reference also clones from the network)."""

    def __init__(self, directory: str = "plugins", key: Optional[str] = None, config_dir: Optional[str] = None):
        from .plugins.registry import PluginRegistry

        self.directory = directory = str(config_dir or directory)
        self.registry = PluginRegistry(key)
        os.makedirs(directory, exist_ok=True)
        self.registry.discover(directory)

    def get_installed_modules(self) -> List[Dict[str, Any]]:
        self.registry.discover(self.directory)
        return self.registry.list()

    def scan_workspace_plugins(self, path: Optional[str] = None) -> Dict[str, Any]:
        found = self.registry.discover(path or self.directory)
        return {"found": [p.name for p in found], "plugins": self.registry.list()}

    def install_module(self, req: Dict[str, Any]) -> Dict[str, Any]:
        import shutil
        from pathlib import Path

        origin = str(req.get("download_url") or req.get("path") or req.get("url") or req.get("source") or "")
        if origin.startswith("builtin://") or (not origin and req.get("id")):  # a module that ships with the framework
            from .plugins.curated import curated_path

            try:
                origin = str(curated_path(origin[len("builtin://"):] if origin else str(req["id"])))
            except KeyError:
                return {"status": "error", "message": f"no curated module named {origin or req.get('id')!r}"}
            req = {**req, "name": req.get("name") or Path(origin).name}
        src = Path(origin).expanduser()
        if "://" in str(src) or not src.is_dir():
            return {"status": "error", "message": "only local module directories can be installed (no network access)"}
        name = str(req.get("name") or src.name)
        dst = (Path(self.directory) / name).resolve()
        if Path(self.directory).resolve() not in dst.parents:
            return {"status": "error", "message": "the module name escapes the module directory"}
        if dst.exists():
            return {"status": "error", "message": f"module {name!r} is already installed"}
        shutil.copytree(src, dst)
        self.registry.discover(self.directory)
        return {"status": "installed", "id": name, "path": str(dst)}

    def activate_module(self, name: str) -> Dict[str, Any]:
        info = self.registry.load(name)
        return {"status": "active", "id": info.name, "nodes": info.nodes}

    def uninstall_module(self, module_id: str) -> Dict[str, Any]:
        import shutil
        from pathlib import Path

        dst = (Path(self.directory) / module_id).resolve()
        if Path(self.directory).resolve() not in dst.parents or not dst.is_dir():
            return {"status": "error", "message": f"module {module_id!r} is not installed"}
        shutil.rmtree(dst)
        self.registry.plugins.pop(module_id, None)
        return {"status": "uninstalled", "id": module_id}

    # ---- the rest of the reference manager's surface; what would need the network says so
    def _config_path(self):
        from pathlib import Path

        return Path(self.directory) / "modules.json"

    def get_config(self) -> Dict[str, Any]:
        import json

        p = self._config_path()
        return json.loads(p.read_text()) if p.is_file() else {"directory": self.directory, "active": []}

    def save_config(self, config: Dict[str, Any]) -> Dict[str, Any]:
        import json

        self._config_path().write_text(json.dumps(config, indent=1))
        return config

    def inspect_directory(self, path: str) -> Dict[str, Any]:
        """What a directory holds, without importing anything from it."""
        from pathlib import Path

        d = Path(path)
        if not d.is_dir():
            return {"status": "error", "message": f"no such directory: {path}"}
        files = [f for f in d.rglob("*") if f.is_file()]
        return {"status": "ok", "path": str(d), "files": len(files), "python_files": sum(f.suffix == ".py" for f in files),
                "has_manifest": (d / "plugin.json").is_file(), "is_git": (d / ".git").exists(),
                "weights": sorted(f.name for f in files if f.suffix in (".safetensors", ".pt", ".gguf"))[:20]}

    def discover_and_register_nodes(self, module_id: str) -> Dict[str, Any]:
        return self.activate_module(module_id)

    def create_custom_plugin_template(self, name: str) -> Dict[str, Any]:
        return self.create_plugin_template(name)

    def scan_hardware_and_software(self) -> Dict[str, Any]:
        from .installer import probe_machine

        return probe_machine().to_dict()

    def search_marketplace(self, query: str = "", source: str = "all") -> Dict[str, Any]:
        """The curated modules that match ``query`` (they install offline from ``builtin://<id>``); remote catalogues are
        not contacted."""
        from .plugins.curated import CURATED

        q = (query or "").lower()
        hits = [dict(c, source="curated") for c in CURATED if not q or q in (c["id"] + " " + c["name"] + " " + c["description"]).lower()]
        return {"results": hits, "curated": hits, "github": [], "huggingface": [],
                "note": "remote catalogues need network access, which this framework does not use"}

    def check_updates(self) -> Dict[str, Any]:
        return {"updates": [], "note": "remote catalogues need network access, which this framework does not use"}

    def clone_repository(self, url: str, mod_type: str = "auto", branch: str = "main", name: Optional[str] = None) -> Dict[str, Any]:
        """Clone a LOCAL git repository (a path or ``file://`` URL) into the module directory."""
        import subprocess
        from pathlib import Path

        src = url[len("file://"):] if url.startswith("file://") else url
        if "://" in src or src.startswith("git@") or not (Path(src) / ".git").exists():
            return {"status": "error", "message": "only local git repositories can be cloned (no network access)"}
        dst = (Path(self.directory) / (name or Path(src).name)).resolve()
        if Path(self.directory).resolve() not in dst.parents or dst.exists():
            return {"status": "error", "message": "the target exists already or escapes the module directory"}
        r = subprocess.run(["git", "clone", "--quiet", "--depth", "1", src, str(dst)], capture_output=True, text=True, timeout=120)
        if r.returncode != 0:
            return {"status": "error", "message": r.stderr.strip()[:300]}
        self.registry.discover(self.directory)
        return {"status": "cloned", "id": dst.name, "path": str(dst)}

    def git_pull(self, module_id: str) -> Dict[str, Any]:
        import subprocess
        from pathlib import Path

        dst = (Path(self.directory) / module_id).resolve()
        if Path(self.directory).resolve() not in dst.parents or not (dst / ".git").exists():
            return {"status": "error", "message": f"no git module {module_id!r} is installed"}
        r = subprocess.run(["git", "-C", str(dst), "pull", "--quiet", "--ff-only"], capture_output=True, text=True, timeout=120)
        return {"status": "updated", "id": module_id} if r.returncode == 0 else {"status": "error", "message": r.stderr.strip()[:300]}

    def create_plugin_template(self, name: str) -> Dict[str, Any]:
        from .plugins.registry import create_plugin

        path = create_plugin(self.directory, name, self.registry.key)
        self.registry.discover(self.directory)
        return {"status": "created", "path": str(path)}
