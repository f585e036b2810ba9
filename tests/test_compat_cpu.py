"""The reference's import paths served by this framework (``triune_b200.compat``)."""

import importlib
import sys

import pytest
import torch

from triune_b200 import compat

REFERENCE_EXPORTS = {
    "optim": "AdamW8bit CentroidSteerOptimizer HAS_8BIT LowSpaceWeightProjector Muon QuantumUnitaryOptimizer UnitaryManifoldOptimizer build_optimizer zeropower_via_newtonschulz5",
    "model": "CANONICAL_MODEL_SPECS MODEL_REGISTRY ModelSpec TriuneModel TriuneTransformer SelfSpeculativeGenerator TransformerBlock HybridAttention VectorisedGLA MoE_FFN "
             "RoutingResult RMSNorm RotaryEmbedding apply_rotary rotate_half GumbelSoftmaxRouter FP4Linear FP8Linear build_model build_model_from_spec get_model_spec load_model "
             "register_model WeightTiedExitProjection attach_early_exits generate_adaptive UniversalAdaptiveEmbedding JEVLatentPredictor JEVObjective JEVExitRouter "
             "JEVRoutingResult TriuneLatentPredictor TriuneLatentObjective TriuneContinuousExitRouter ContinuousLatentExitRouter JointEmbeddingObjective LatentPredictor",
    "runtime": "MemoryEstimate MemoryPlan MemoryPlanner DynamicResourceManager LiveVRAMMonitor AllotmentPlan HardwareProfile VRAMBudgetExceededError LayerStreamingEngine "
               "StreamingConfig enable_layer_streaming apply_layer_streaming_if_requested PrecisionCapabilities ParameterStager StagingBuffer FP8StagingBuffer PythonSandbox "
               "SandboxResult VRAMProfiler AutoOffloader CUDAGraphEngine NeuronScope ParallelEngine GLAPipelineBlock MoERoutingBlock",
    "ops": "NativeTriuneEngine is_native_c_available get_native_c_info c_centroid_steer_update_f32 c_route_tiers_f32 c_compute_neuron_heatmap_f32 c_gla_recurrent_step_f32 "
           "batched_qr cholesky_qr subspace_projection batched_subspace_projection triangular_steer_update gla muon_orthogonalize muon_ns norm rmsnorm rope swiglu gelu "
           "cross_entropy chunked_cross_entropy FastChunkedCrossEntropyLoss lora_forward lora_linear upgrade route_tiers TIER_REFLEX TIER_LIMBIC TIER_CORTEX TIER_NAMES",
    "agents": "Agent AgentHarness AgentMemoryStore AgentSkill BUILTIN_PERSONAS CognitiveState LearnedLesson MultiAgentOrchestrator PersonaProfile ProviderConfig "
              "ProviderManager SkillLibrary StateController Tool ToolRegistry ToolStats UserPreference build_integrated_toolbelt",
    "recipes": "bf16_autocast build_fp8_precision_context build_precision_context build_mxfp8_precision_context",
    "trainer": "Engine TrainingEngine DistributedTrainingEngine DistributedContext setup_distributed cleanup_distributed is_distributed get_rank get_world_size "
               "get_local_rank is_main_process all_reduce_tensor all_reduce_dict wrap_distributed_model Trainer NullLogger WandbLogger LoRAConfig LoRALayer TriuneFineTuner "
               "list_adapters export_adapter merge_adapter_checkpoint",
    "kernels": "is_triton_available get_kernel_backend get_triton_error is_turbo_mode_enabled set_turbo_mode get_kernel_telemetry fast_rmsnorm fast_fused_add_rmsnorm "
               "FastRMSNorm fast_rope fast_swiglu fast_gelu FastSwiGLU FastGELU fast_cross_entropy chunked_cross_entropy_from_hidden FastChunkedCrossEntropyLoss fast_chunk_gla "
               "fast_chunk_gated_deltanet fast_recurrent_gated_deltanet fast_zeropower_via_newtonschulz5 fast_lora_forward fast_lora_linear fast_qkv_lora_linear "
               "fast_gate_up_lora_linear is_fp8_available fast_fp8_linear FastFP8Linear nvfp4_quantize nvfp4_dequantize nvfp4_linear fwht_16 NVFP4Linear",
    "export": "export_gguf export_onnx export_safetensors export_model export_to_huggingface",
    "api": "create_app run_server",
    "callbacks": "Callback CallbackList TelemetryCallback EventEmitter global_emitter",
    "configs": "build_config default_config validate_config",
    "data": "AsyncDevicePrefetcher CyclingDataLoader DynamicTokenizer DynamicTokenizerOutput TokenStreamDataset TriuneTokenizer build_dataloader build_tokenizer load_tokenizer",
    "plugins": "NodeRegistry NODE_REGISTRY global_registry node_registry get_node_executor list_registered_nodes register_node",
    "execution": "DAGParser ExecutionEngine NodeExecutionError",
    "modules": "ModuleManager",
}


@pytest.fixture()
def triune():
    compat.uninstall()
    root = compat.install()
    yield root
    compat.uninstall()


def test_every_exported_name_of_the_reference_resolves(triune):
    cov = compat.coverage()
    for pkg, names in REFERENCE_EXPORTS.items():
        assert cov[pkg]["unresolved"] == {}, (pkg, cov[pkg]["unresolved"])
        mod = importlib.import_module(f"triune.{pkg}")
        for n in names.split():
            assert getattr(mod, n) is not None or n in ("NODE_REGISTRY",), (pkg, n)
    assert compat.install() is triune  # idempotent
    with pytest.raises(AttributeError):
        importlib.import_module("triune.model").no_such_name


def test_a_script_written_against_the_reference_runs(triune, tmp_path):
    """Imports by the reference's paths (package level and deep modules), builds the model, trains a step, exports."""
    from triune.configs import build_config, default_config
    from triune.export import export_model
    from triune.kernels import fast_cross_entropy
    from triune.model import TriuneModel, TriuneTransformer, apply_rotary, rotate_half
    from triune.model.transformer import TriuneTransformer as Deep
    from triune.optim import HAS_8BIT, AdamW8bit, CentroidSteerOptimizer
    from triune.trainer import get_rank, get_world_size, is_distributed, is_main_process

    import triune_b200.models.transformer as ours

    assert Deep is TriuneTransformer is ours.TriuneTransformer and issubclass(TriuneModel, torch.nn.Module)
    assert default_config() == build_config({}) and HAS_8BIT is True
    assert (get_rank(), get_world_size(), is_distributed(), is_main_process()) == (0, 1, False, True)
    x = torch.arange(8.0).view(1, 8)
    assert rotate_half(x).tolist() == [[-4.0, -5.0, -6.0, -7.0, 0.0, 1.0, 2.0, 3.0]]
    qr, kr = apply_rotary(x, 2 * x, torch.ones(8), torch.zeros(8))
    assert torch.allclose(qr, x) and torch.allclose(kr, 2 * x)
    torch.manual_seed(0)
    model = TriuneTransformer(vocab_size=64, hidden_dim=32, num_layers=5, num_heads=1, head_dim=32, num_experts=2, router_prefix_layers=1,
                              reflex_exit_layer=2, limbic_exit_layer=3)
    ids = torch.randint(0, 64, (2, 17))
    opt = CentroidSteerOptimizer(model, lr=1e-3)
    logits = model(ids[:, :-1], force_depth=2)[0]
    loss = fast_cross_entropy(logits.reshape(-1, 64), ids[:, 1:].reshape(-1))
    loss.backward()
    opt.step()
    assert torch.isfinite(loss)
    out = export_model(model, str(tmp_path / "m.safetensors"), "safetensors")
    assert (tmp_path / "m.safetensors").is_file() and str(out).endswith("m.safetensors")
    # 8-bit AdamW: follows fp32 AdamW closely on a quadratic and keeps two bytes per parameter
    w8, w32 = torch.nn.Parameter(torch.full((600,), 2.0)), torch.nn.Parameter(torch.full((600,), 2.0))
    o8, o32 = AdamW8bit([w8], lr=0.05, weight_decay=0.0), torch.optim.AdamW([w32], lr=0.05, weight_decay=0.0)
    for _ in range(30):
        for w, o in ((w8, o8), (w32, o32)):
            o.zero_grad()
            (w * w).sum().backward()
            o.step()
    assert float((w8 - w32).abs().max()) < 0.05 and float(w8.abs().max()) < 1.2
    assert o8.state_bytes() == 2 * 768 + 8 * 3  # 600 elements in 3 blocks of 256


def test_graph_engine_registry_and_modules_under_reference_names(triune, tmp_path):
    from triune.execution import DAGParser, ExecutionEngine, NodeExecutionError
    from triune.execution.dag import ExecutionEngine as Deep
    from triune.modules import ModuleManager
    from triune.plugins import get_node_executor, global_registry, list_registered_nodes
    from triune.agents import BUILTIN_PERSONAS, StateController

    assert Deep is ExecutionEngine and "TriuneTransformer" in list_registered_nodes() and callable(get_node_executor("RMSNorm"))
    assert "architect" in BUILTIN_PERSONAS and StateController().assess("why does it crash with a traceback")["persona"] == "debugger"
    assert StateController(depth="auto").assess("hi")["depth"] == "reflex"
    g = {"nodes": [{"id": "a", "type": "PythonSandbox", "params": {"code": "result = 'abc'"}}, {"id": "b", "type": "BPETokenizer"}],
         "edges": [{"source": "a", "target": "b", "source_port": "result", "target_port": "text"}]}
    assert DAGParser.parse(g)["execution_order"] == ["a", "b"] and DAGParser.from_json(g)["b"]["dependencies"] == ["a"]
    with pytest.raises(NodeExecutionError):
        DAGParser.parse({"nodes": [{"id": "a", "type": "X"}], "edges": [{"source": "a", "target": "zz"}]})
    eng = ExecutionEngine()
    events = []
    eng.register_event_callback(events.append)
    res = eng.execute_graph(g)
    assert res["status"] == "success" and [e["event"] for e in events] == ["node_started", "node_finished"] * 2
    assert eng.run(g)["b"]["status"] == "completed"
    # a handler in the reference's convention: (node, context) -> dict, ports through context["port_data"]
    def doubler(node, context):
        context["port_data"].setdefault(node["id"], {})["doubled"] = 2 * context["current_inputs"]["value"]
        return {"status": "completed", "note": "ok"}

    eng.register_handler("Doubler", doubler)
    out = eng.execute_node({"id": "d", "type": "Doubler"}, {"value": 21})
    assert out["status"] == "success" and out["output"]["ports"]["doubled"] == 42
    assert "Doubler" in global_registry
    from triune_b200.execution.studio import STUDIO_NODES

    STUDIO_NODES.pop("Doubler")  # leave the process-wide catalogue as it was
    from triune_b200.plugins.registry import create_plugin

    src = create_plugin(tmp_path / "src", "my_nodes")
    mm = ModuleManager(str(tmp_path / "mods"))
    assert mm.install_module({"path": str(src)})["status"] == "installed"
    assert [m["name"] for m in mm.get_installed_modules()] == ["my_nodes"]
    assert mm.install_module({"url": "https://github.com/a/b"})["status"] == "error"
    assert mm.uninstall_module("my_nodes")["status"] == "uninstalled" and mm.uninstall_module("my_nodes")["status"] == "error"


def test_a_real_package_of_that_name_is_not_shadowed():
    compat.uninstall()
    import types

    sys.modules["triune"] = types.ModuleType("triune")
    try:
        with pytest.raises(RuntimeError):
            compat.install()
    finally:
        del sys.modules["triune"]


def test_reference_signatures_of_operators_and_agents(triune, tmp_path):
    """Where the two projects order or name arguments differently, the names under ``triune.*`` follow the reference."""
    from triune.agents import AgentHarness, AgentMemoryStore, MultiAgentOrchestrator, SkillLibrary, build_integrated_toolbelt
    from triune.ops import batched_qr, batched_subspace_projection, muon_orthogonalize, route_tiers, subspace_projection, triangular_steer_update
    from triune.optim import zeropower_via_newtonschulz5
    from triune.trainer import all_reduce_dict

    from triune_b200 import ops

    torch.manual_seed(0)
    P, G = torch.randn(2, 6, 6), torch.randn(2, 6, 6)
    want = ops.triangular_steer_update(P.clone(), G, 0.9, 0.25)  # this framework: (P, G, momentum, scale)
    assert torch.allclose(triangular_steer_update(P.clone(), G, 0.25, 0.9), want)  # the reference: (P, G, scale, momentum)
    assert torch.allclose(triangular_steer_update(P.clone(), G, steer_scale=0.25, momentum=0.9), want)
    R = triangular_steer_update(torch.randn(2, 8, 4), torch.randn(2, 8, 4), 0.1, 0.9, retract_stiefel=True)
    assert torch.allclose(R.transpose(1, 2) @ R, torch.eye(4).expand(2, 4, 4), atol=1e-3)
    probs, tiers = route_tiers(torch.tensor([[4.0, 0.0, 0.0], [0.0, 0.0, 3.0]]), reflex_threshold=0.7)
    assert torch.allclose(probs.sum(-1), torch.ones(2)) and tiers.tolist() == [0, 2]
    A = torch.randn(3, 20, 4)
    Q = batched_qr(A)
    Q2, mask = batched_qr(A, return_fallback_mask=True)
    Q3, info = batched_qr(A, return_diagnostics=True, out_dtype=torch.float64)
    assert torch.allclose(Q, Q2) and mask.shape == (3,) and Q3.dtype == torch.float64 and "orth_err" in info
    assert subspace_projection(torch.randn(16, 12), 4).shape[-1] == 4
    Qb, path = batched_subspace_projection(torch.randn(2, 16, 12), 4)
    assert Qb.shape[0] == 2 and isinstance(path, str) and len(batched_subspace_projection(torch.randn(2, 16, 12), 4, return_diagnostics=True)) == 3
    Gm = torch.randn(8, 12)
    assert torch.allclose(muon_orthogonalize(Gm, 5), zeropower_via_newtonschulz5(Gm, steps=5))
    X, scratch = zeropower_via_newtonschulz5(Gm, 5, 1e-7, "buf", True)
    assert scratch == "buf" and X.shape == Gm.shape
    assert all_reduce_dict({"loss": 2.0, "tokens": 10}) == {"loss": 2.0, "tokens": 10.0}

    ws = tmp_path / "ws"
    ws.mkdir()
    (ws / "a.txt").write_text("hello")
    mem = AgentMemoryStore(tmp_path / "store")
    tools = build_integrated_toolbelt(workspace=ws, memory=mem, allow_writes=False, subagent_runner=lambda task, persona: f"{persona}: {task}")
    assert "write_file" not in tools.tools and tools.call("read_file", path="a.txt") == "hello"
    assert tools.call("remember", text="the corpus lives in a.txt") == "noted" and "a.txt" in tools.call("recall", query="where is the corpus")[0]
    assert tools.call("delegate", task="check", persona="sentinel") == "sentinel: check"
    assert (tmp_path / "store" / "memory.json").is_file()
    lib = SkillLibrary(tmp_path / "skills", extra_skill_dirs=[tmp_path / "none"])
    assert lib.skills == {}
    seen = []
    h = AgentHarness(workspace=ws, store_dir=tmp_path / "store", completion_fn=lambda prompt: (seen.append(prompt), {"text": "done"})[1], allow_writes=False)
    out = h.run("explain why the file exists")
    assert out["text"] == "done" and out["persona"] == "researcher" and "write_file" not in out["tools_offered"]
    orch = MultiAgentOrchestrator(h)
    assert [o["agent"] for o in orch.execute("plan then review", ["architect", "sentinel"])] == ["architect", "sentinel"]
    par = orch.execute_parallel("look at it", ["engineer", "tutor"], max_workers=2)
    assert [o["agent"] for o in par] == ["engineer", "tutor"] and all(o["text"] == "done" for o in par)


def test_method_names_of_the_reference_on_core_classes(triune):
    """Methods that callers of the reference use on the engine, optimizer, layer and loader classes exist here and do the
    same job (CPU: the graph engine captures nothing and falls back)."""
    from triune.data import CyclingDataLoader
    from triune.kernels import NVFP4Linear
    from triune.model import FP4Linear, FP8Linear, MoE_FFN, RotaryEmbedding, SelfSpeculativeGenerator, TriuneTransformer
    from triune.optim import CentroidSteerOptimizer
    from triune.runtime import CUDAGraphEngine, LayerStreamingEngine, StreamingConfig
    from triune.trainer import Trainer

    torch.manual_seed(0)
    model = TriuneTransformer(vocab_size=64, hidden_dim=32, num_layers=5, num_heads=1, head_dim=32, num_experts=2, router_prefix_layers=1,
                              reflex_exit_layer=2, limbic_exit_layer=3)
    opt = CentroidSteerOptimizer(model, lr=1e-3)
    opt.param_groups[0]["lr"] = 5e-4  # what an outer PyTorch scheduler does
    opt.sync_lr_from_param_groups()
    assert opt.lr == 5e-4 and opt.muon_lr == pytest.approx(opt.initial_muon_lr * 0.5)
    moe = MoE_FFN(32, 4, 2).eval()
    x = torch.randn(2, 6, 32)
    with torch.no_grad():
        assert torch.allclose(moe.sparse_forward(x), moe(x, update_stats=False))
    f4 = FP4Linear(32, 16)
    q4 = f4.to_nvfp4_inference()
    assert q4(torch.randn(3, 32)).shape == (3, 16)
    with pytest.raises(ValueError):
        FP4Linear(24, 8).to_nvfp4_inference()
    f8 = FP8Linear(32, 16)
    w0 = f8.weight.clone()
    f8.reset_parameters()
    assert not torch.equal(w0, f8.weight)
    assert NVFP4Linear.empty_skeleton(32, 16).weight.shape == (16, 32)
    assert RotaryEmbedding(dim=16).head_dim == 16 and RotaryEmbedding(16).head_dim == 16
    gen = SelfSpeculativeGenerator(model, None, 2, 0.7)  # (model, tokenizer, k_draft, temperature): the reference's positional order
    assert gen.temperature == 0.7 and gen.k_draft == 2
    it = CyclingDataLoader([1, 2])
    assert [it.next(), it.next(), it.next()] == [1, 2, 1]

    tr = Trainer(model=model, optimizer=opt, train_loader=None, eval_loader=None, tokenizer=None, config={"vocab_size": 64, "lr": 1e-3},
                 device="cpu", precision_context=None, logger=None, sample_prompt="Once")
    assert tr.sample_prompt == "Once"
    with tr.bf16_autocast():
        pass
    eng = LayerStreamingEngine(model, torch.device("cpu"), StreamingConfig(), optimizer=None, layers_path=None)
    eng.attach()
    try:
        roots = eng.get_root_parameters()
        inside = {id(p) for l in eng.layers for p in l.parameters()}
        assert roots and all(id(p) not in inside for p in roots)
        eng.set_optimizer(opt)
        tr.engine.sync_streaming_engine()
        eng.flush_d2h_transfers()
        eng.zero_grad()
        ids = torch.randint(0, 64, (2, 9))
        model.forward_loss(ids[:, :-1], ids[:, 1:], force_depth=2).backward()
        norm = eng.step_optimizer(None)
        assert norm > 0
        eng.cleanup_resident_layers()
    finally:
        eng.detach()

    g = CUDAGraphEngine("cpu")
    lin = torch.nn.Linear(4, 4)
    sgd = torch.optim.SGD(lin.parameters(), lr=0.1)
    xb, yb = torch.randn(2, 4), torch.randn(2, 4)
    assert g.capture_training_step(lin, sgd, xb, yb) is False and g.capture_inference_step(lin, xb) is False and not g.can_replay(xb, yb)
    assert g.step(xb, yb, sync=True, fallback_fn=lambda a, b: 1.5) == 1.5
    assert float(g.step(xb, yb, fallback_fn=lambda a, b: 2.5)) == 2.5
    assert torch.equal(g.inference_step(xb, fallback_fn=lambda a: a * 2), xb * 2)
    with pytest.raises(RuntimeError):
        g.step(xb, yb)
    g.invalidate()
    assert g.current_loss_item() == 0.0 and g.is_captured is False


def test_reference_method_names_on_agents_registry_and_modules(triune, tmp_path):
    from triune.agents import AgentHarness, MultiAgentOrchestrator, PersonaProfile, ProviderManager, StateController, ToolStats, build_integrated_toolbelt
    from triune.modules import ModuleManager
    from triune.plugins import NodeRegistry

    tools = build_integrated_toolbelt(workspace=tmp_path, allow_writes=True)
    assert "read_file" in tools.names() and tools.get("clock").run().endswith("Z") and tools.get("nope") is None
    ok = tools.execute("write_file", {"path": "a.txt", "content": "x"})
    bad = tools.execute("read_file", {"path": "../outside"})
    assert ok["ok"] and not bad["ok"] and "PermissionError" in bad["error"] and tools.stats["read_file"] == {"calls": 1, "failures": 1, "seconds": bad["seconds"]}
    spec = {t["function"]["name"]: t for t in tools.to_openai_tools()}["read_file"]
    assert spec["type"] == "function" and spec["function"]["parameters"]["properties"]["start"] == {"type": "integer"}
    assert "- read_file(path, start, length)" in tools.format_prompt_catalog() and len(tools.list_tools()) == len(tools.names())
    st = ToolStats(calls=4, failures=1, seconds=0.2)
    assert st.success_rate == 0.75 and st.avg_latency_ms == pytest.approx(50.0) and st.calibrated_reliability == pytest.approx(4 / 6)
    assert ToolStats().success_rate == 0.0 and ToolStats().calibrated_reliability == 0.5

    sc = StateController(tmp_path)
    sc.register_persona("poet", "Answer in verse.", 0.9, ("poem", "verse"))
    assert sc.adapt_for_goal("a poem in verse, please")["persona"] == "poet" and sc.shift("sentinel")["persona"] == "sentinel"
    assert sc.active_profile.name == "sentinel" and isinstance(sc.active_profile, PersonaProfile) and sc.active_profile.to_dict()["name"] == "sentinel"
    sc2 = StateController()
    assert sc2.adapt_after_tool("search", ok=False)["persona"] == "debugger"
    assert sc.delete_persona("poet") and not sc.delete_persona("poet")

    pm = ProviderManager(transport=lambda p, msgs, opt: f"{p.name}/{opt.get('model', p.model)}: {msgs[-1]['content']}")
    pm.register_provider("local", "http://127.0.0.1:11434", "gemma3:4b")
    pm.register_provider("cloud", "https://api.example.com", "big", api_key="")
    assert pm.list_active_providers() == ["local"] and pm.pick_default_model() == "local:gemma3:4b" and pm.get_provider("LOCAL").model == "gemma3:4b"
    assert pm.complete_chat([{"role": "user", "content": "hi"}]) == {"text": "local/gemma3:4b: hi", "provider": "local", "model": "gemma3:4b"}
    with pytest.raises(KeyError):
        pm.complete_chat([], model="nobody:x")

    h = AgentHarness(workspace=tmp_path, store_dir=tmp_path / "store", completion_fn=lambda prompt: "fine")
    assert h.run_goal("say something")["text"] == "fine"
    orch = MultiAgentOrchestrator(h)
    orch.add_agent("architect")
    orch.add_agent("engineer")
    orch.add_agent("architect")
    assert [s["agent"] for s in orch.execute_pipeline("build it")] == ["architect", "engineer"]
    team = orch.orchestrate_team("build it", parallel=True, max_workers=2)
    assert team["team"] == ["architect", "engineer"] and team["final"] == "fine" and team["parallel"] is True

    reg = NodeRegistry()
    assert "TriuneTransformer" in reg.list_nodes() and reg.get_core_node_names() == reg.list_nodes()
    assert [p["name"] for p in reg.get_schema("RouterZLoss")["inputs"]] == ["router_logits"] and reg.get_node("nope") is None

    mm = ModuleManager(config_dir=str(tmp_path / "mods"))
    assert mm.save_config({"directory": str(tmp_path / "mods"), "active": ["a"]}) == mm.get_config()
    assert mm.inspect_directory(str(tmp_path))["files"] >= 1 and mm.inspect_directory(str(tmp_path / "zz"))["status"] == "error"
    assert mm.search_marketplace("zzz")["results"] == [] and mm.check_updates()["updates"] == []
    assert [r["download_url"] for r in mm.search_marketplace("loss")["results"]] == ["builtin://custom_loss_nodes"]
    assert mm.clone_repository("https://github.com/a/b")["status"] == "error" and mm.git_pull("none")["status"] == "error"
    assert "os_type" in mm.scan_hardware_and_software()
    assert mm.create_custom_plugin_template("my_plug")["status"] == "created" and mm.discover_and_register_nodes("my_plug")["status"] == "active"


def test_run_config_keys_and_exploration_schedule_follow_the_reference():
    """Every key of the reference's default run config exists here (its 48 keys, read from its ``build_config``), and the
    exploration schedule accepts the reference's names as well as a starting rate."""
    from types import SimpleNamespace

    from triune_b200.config import build_config
    from triune_b200.trainer.engine import TrainingEngine

    ref_keys = """vocab_size hidden_dim num_layers num_heads num_experts top_k router_prefix_layers reflex_exit_layer limbic_exit_layer target_depth_dist
    depth_mode exploration exploration_steps use_fp4 use_fp8 batch_size seq_len grad_accum_steps total_steps lr min_lr warmup_steps betas weight_decay grad_clip
    galore galore_rank galore_update_gap galore_lr galore_betas steer_scale use_triangular_core use_muon muon_lr muon_momentum log_every save_every eval_every
    eval_batches checkpoint_dir shuffle_buffer dataset_name dataset_config num_workers""".split()
    cfg = build_config({})
    assert [k for k in ref_keys if k not in cfg] == [] and cfg["exploration"] == "linear" and cfg["dataset_config"] == "sample-10BT"

    def rate(conf, step):
        eng = SimpleNamespace(config=conf, step=step)
        return TrainingEngine._exploration(eng)

    lin = {"exploration": "linear", "exploration_steps": 100}
    assert rate(lin, 0) == 1.0 and rate(lin, 25) == 0.75 and rate(lin, 100) == 0.0 and rate(lin, 500) == 0.0
    cos = {"exploration": "cosine", "exploration_steps": 100}
    assert rate(cos, 0) == 1.0 and rate(cos, 50) == pytest.approx(0.5) and rate(cos, 100) == 0.0
    assert rate({"exploration": "none", "exploration_steps": 100}, 0) == 0.0 and rate({"exploration": "linear", "exploration_steps": 0}, 0) == 0.0
    num = {"exploration": 0.2, "exploration_steps": 100}
    assert rate(num, 0) == pytest.approx(0.2) and rate(num, 50) == pytest.approx(0.1) and rate(num, 100) == 0.0
    assert rate({"exploration": 0.4, "exploration_steps": 100, "exploration_schedule": "cosine"}, 50) == pytest.approx(0.2)


def test_every_module_path_of_the_reference_imports_and_top_level_names_resolve():
    """Deep import paths (``triune.runtime.staging``, ``triune.model.manifold_embedding``, ``triune.agents.tools`` ...) and
    the names the reference's top-level package re-exports resolve, and uninstalling removes the fall-back lookups that
    were attached to this framework's modules."""
    import importlib

    import triune_b200.compat as compat

    compat.install()
    try:
        import triune

        assert triune.Model is importlib.import_module("triune_b200.models.factory").build_model
        assert triune.CentroidSteer is triune.CentroidSteerOptimizer and triune.TriuneTransformer is triune.model.TriuneTransformer
        assert callable(triune.upgrade) and callable(triune.fast_rope) and triune.Trainer is triune.trainer.Trainer
        for path, names in {
            "triune.runtime.staging": ["ParameterStager", "FP8StagingBuffer"], "triune.model.manifold_embedding": ["UniversalAdaptiveEmbedding"],
            "triune.agents.tools": ["validate_http_url", "ToolRegistry"], "triune.agents._storage": ["atomic_write_json", "compute_tfidf_cosine_scores"],
            "triune.agents.personas": ["BUILTIN_PERSONAS", "PersonaProfile"], "triune.kernels.fast_muon": ["NS5_COEFFS", "compute_muon_update_scale"],
            "triune.kernels.fast_triangular": ["fast_triangular_adamw"], "triune.model.config": ["checkpoint_bwd_ctx", "BATCH_SIZE", "HIDDEN_DIM"],
            "triune.plugins.node_schema": ["PortType", "NodeSchema", "is_port_compatible"], "triune.trainer.checkpoint": ["compute_checkpoint_fingerprint"],
            "triune.universal": ["DenseTransformerBlock", "UniversalDenseTransformer", "upgrade_model"], "triune.utils.seed": ["seed_everything"],
            "triune.api.routes": ["ChatCompletionRequest", "pytorch_state", "sanitize_text", "router"], "triune.api.server": ["lifespan", "create_app"],
            "triune.cli_ui": ["render_table", "route_badge_markup"], "triune.modules.github_client": ["RepoSearchClient"],
            "triune.modules.curated.custom_loss_nodes.custom_loss_nodes": ["FocalCrossEntropyLoss", "anneal_temperature"],
            "triune.runtime.model_scanner": ["parse_gguf_header", "scan_pc_models"], "triune.inference": ["IncrementalStreamingDecoder"],
            "triune.optim.centroid": ["profile_rank_sensitivity", "fast_subspace_projection", "CentroidSteerOptimizer"],
            "triune.ops.centroid_steer": ["polar_stiefel_retraction", "batched_qr"], "triune.packaging": ["build_linux_native", "TRIUNE_SVG_ICON"],
        }.items():
            mod = importlib.import_module(path)
            for n in names:
                assert getattr(mod, n) is not None, f"{path}.{n}"
        with pytest.raises(AttributeError):
            importlib.import_module("triune.runtime.staging").no_such_name
        import triune_b200.serve.routes as routes

        assert routes.ChatCompletionRequest is routes.ChatRequest  # the fall-back attached to the aliased module
    finally:
        compat.uninstall()
    import triune_b200.serve.routes as routes

    assert not hasattr(routes, "pytorch_state")


def test_reference_helper_functions_compute_what_they_name():
    import torch

    from triune_b200.agents import validate_http_url
    from triune_b200.agents.storage import atomic_write_json, compute_tfidf_cosine_scores, load_validated_json_dict, tokenize_terms
    from triune_b200.kernels import compute_muon_update_scale, fast_triangular_adamw, fast_zeropower_via_newtonschulz5_batched
    from triune_b200.optim.centroid import profile_rank_sensitivity
    from triune_b200.serve.routes import sanitize_text

    with pytest.raises(ValueError):
        validate_http_url("ftp://example.com/x")
    with pytest.raises(ValueError):
        validate_http_url("http://user:pw@127.0.0.1/")
    with pytest.raises(PermissionError):
        validate_http_url("http://127.0.0.1:9/")
    assert validate_http_url(" http://127.0.0.1:11434/api/tags ", allow_local_services=True) == "http://127.0.0.1:11434/api/tags"
    with pytest.raises(PermissionError):
        validate_http_url("http://10.1.2.3/")
    assert "#oke" in tokenize_terms("the tokenizer") and "the" not in tokenize_terms("the tokenizer")
    s = compute_tfidf_cosine_scores("gpu memory planner", ["plan memory of a gpu", "bake bread", ""])
    assert s[0] > s[1] == 0.0 and s[2] == 0.0 and all(0.0 <= v <= 1.0 for v in s)
    import tempfile
    from pathlib import Path

    d = Path(tempfile.mkdtemp())
    atomic_write_json(d / "a" / "x.json", {"k": [1, 2]})
    assert load_validated_json_dict(d / "a" / "x.json") == {"k": [1, 2]} and not list((d / "a").glob(".*tmp"))
    (d / "bad.json").write_text("{not json")
    assert load_validated_json_dict(d / "bad.json") == {} and load_validated_json_dict(d / "none.json") == {}
    broken = "it’s “here” — café".encode("utf-8").decode("cp1252", errors="replace")
    assert sanitize_text(broken) == 'it\'s "here" -- café' and sanitize_text("plain ‘x’ é") == "plain ‘x’ é" and sanitize_text(None) == ""
    assert compute_muon_update_scale(64, 16) == 2.0 and compute_muon_update_scale(16, 64, 0.2) == pytest.approx(0.2)
    X = fast_zeropower_via_newtonschulz5_batched(torch.randn(2, 8, 24), steps=8)
    assert torch.allclose(X @ X.transpose(1, 2), torch.eye(8).expand(2, 8, 8), atol=1e-2)
    with pytest.raises(ValueError):
        fast_zeropower_via_newtonschulz5_batched(torch.randn(8, 24))
    R, m, v, out = torch.randn(3, 5, 5), torch.zeros(3, 5, 5), torch.zeros(3, 5, 5), torch.empty(3, 5, 5)
    fast_triangular_adamw(R, m, v, out, torch.tensor([1, 1, 1]), 0.9, 0.999, mask_mode="triu")
    assert torch.allclose(out, torch.sign(R).triu(), atol=1e-3) and torch.allclose(m, 0.1 * R)  # first step of Adam: the sign of the gradient
    lin = torch.nn.Linear(32, 16, bias=False)
    with torch.no_grad():
        lin.weight.copy_(torch.outer(torch.randn(16), torch.randn(32)))  # rank one
    rep = profile_rank_sensitivity(lin, target_energy=0.9, min_rank=1)
    assert rep["layers"]["weight"]["recommended_rank"] == 1 and rep["layers"]["weight"]["captured_energy"] > 0.99


def test_reference_calling_forms_of_generation_checkpoints_and_cache(tmp_path):
    """``generate_response`` with the reference's keyword-only arguments returns text (a dict with ``return_info``);
    ``save_latest`` / ``load_checkpoint`` take a trainer; ``build_nvfp4_disk_cache`` returns the cache directory; layer
    constructors take ``device`` / ``dtype``; attribute names of the reference read back."""
    import torch

    import triune_b200.compat as compat
    from triune_b200.config import ModelConfig
    from triune_b200.models import TriuneTransformer

    cfg = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, top_k=2, router_prefix_layers=1,
               reflex_exit_layer=2, limbic_exit_layer=3, expert_hidden=96, dense_hidden=80)

    class Tok:
        pad_token_id, sep_token_id, eos_token_id = None, None, None

        def encode(self, s):
            return [ord(ch) % 256 for ch in s]

        def decode(self, ids):
            return "".join(chr(32 + i % 90) for i in ids)

    compat.install()
    try:
        from triune.inference import generate_response
        from triune.model.fp8 import FP8Linear
        from triune.model.jev import JEVObjective
        from triune.model.rotary import RotaryEmbedding
        from triune.runtime.parallel_engine import MoERoutingBlock
        from triune.trainer.checkpoint import compute_checkpoint_fingerprint, load_checkpoint, save_latest

        torch.manual_seed(0)
        model = TriuneTransformer.from_config(ModelConfig(**cfg)).eval()
        text = generate_response(model, Tok(), "hi", device="cpu", pad_token_id=0, eos_token_id=255, max_new_tokens=4, temperature=0.0)
        info = generate_response(model, Tok(), "hi", device="cpu", pad_token_id=0, eos_token_id=255, max_new_tokens=4, temperature=0.0,
                                 force_depth=1, return_info=True)
        assert isinstance(text, str) and info["route"] == "LIMBIC" and info["tokens_count"] <= 4 and not info["cancelled"] and "cache" in info
        with pytest.raises(ValueError):
            generate_response(model, Tok(), "hi", device="cpu", pad_token_id=0, eos_token_id=255, top_k=0)

        class Trainer:
            pass

        t = Trainer()
        t.model, t.config = model, dict(cfg, checkpoint_dir=str(tmp_path))
        t.optimizer = torch.optim.AdamW(model.parameters())
        eng = type("Engine", (), {"best_eval_loss": 1.5, "depth_usage_ema": [0.3, 0.3, 0.4]})()
        path = save_latest(t, eng, 7, 2.5)
        assert path == tmp_path / "latest.pt" and path.is_file()
        t2 = Trainer()
        t2.model, t2.optimizer, t2.config = TriuneTransformer.from_config(ModelConfig(**cfg)), None, dict(t.config)
        ck = load_checkpoint(t2, path, load_optimizer=False)
        key = next(iter(model.state_dict()))
        assert ck["step"] == 7 and ck["best_eval_loss"] == 1.5 and ck["fingerprint"] == compute_checkpoint_fingerprint(t.config)
        assert torch.equal(t2.model.state_dict()[key], model.state_dict()[key])
        t2.config["hidden_dim"] = 128
        with pytest.raises(ValueError):
            load_checkpoint(t2, path, load_optimizer=False)
        assert FP8Linear(32, 16, device="cpu", dtype=torch.float32).weight.shape == (16, 32)
        assert RotaryEmbedding(dim=16, max_seq_len=32).cos_cached.shape[0] == 32 and MoERoutingBlock(dim=32, num_experts=2, top_k=1, mode="batched").mode == "batched"
        obj = JEVObjective()
        obj(torch.randn(4, 8), torch.randn(4, 8))
        assert all(isinstance(v, float) for v in (obj.last_sim_loss, obj.last_stp_loss, obj.last_cov_loss, obj.last_total_loss))
    finally:
        compat.uninstall()
