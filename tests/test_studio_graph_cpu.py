"""Graphs in the Studio canvas format (node, port and parameter names of the reference's catalogue) on the CPU."""

import json
import os

import pytest
import torch

from triune_b200.execution import studio
from triune_b200.execution.studio import (STUDIO_NODES, StudioGraphError, compile_to_training, node_params, parse_studio_graph,
                                          resolve_kind, run_studio_graph, run_studio_node, studio_catalog)

REFERENCE_KINDS = """Data HuggingFaceStreamer URLDatasetStreamer LocalFileReader BPETokenizer CyclingDataLoader Model TriuneTransformer
VectorisedGLA HybridAttention MoE_FFN DepthRouter FP8Linear FP4Linear TensorInspector TokenBatchInspector RMSNorm LoRAAdapter Optimizer
CentroidSteerOptimizer MuonOptimizer AdamWOptimizer CosineLRScheduler Loss FastCrossEntropy JointExitLoss RouterZLoss FastRoPE FastRMSNorm
Runtime LayerStreamingEngine GradientAccumulator CheckpointManager DynamicResourceManager VRAMProfiler PythonSandbox WandbLogger
AutoregressiveGenerator BYOKChatRouter Subgraph SubgraphInput Evaluation TrainingStep PerplexityEvaluator LoRAFineTuner Export
SafeTensorsExport GGUFExport ONNXExport""".split()

MODEL_CFG = {"hidden_dim": 64, "num_layers": 4, "num_heads": 1, "num_experts": 4, "vocab_size": 256, "use_node_config": True}


def _corpus(tmp_path):
    p = tmp_path / "corpus.txt"
    p.write_text("hello world, this is a tiny corpus for the graph.\n\nsecond paragraph of text here.\n")
    return str(p)


def test_every_node_kind_of_the_canvas_is_known_with_its_ports():
    assert len(REFERENCE_KINDS) == 49
    for k in REFERENCE_KINDS:
        assert k in STUDIO_NODES, k
    cat = {n["name"]: n for n in studio_catalog()}
    assert [p["name"] for p in cat["TriuneTransformer"]["typed_outputs"]] == [
        "logits", "model_handle", "exit_logits", "router_logits", "balance_loss", "selected_depth"]
    assert cat["FastCrossEntropy"]["inputs"] == ["logits", "targets", "balance_loss", "router_logits"]
    assert cat["TrainingStep"]["outputs"] == ["step_metrics", "loss", "model_handle"]
    assert set(cat["CentroidSteerOptimizer"]["parameters"]) == {"lr", "betas", "weight_decay", "steer_scale", "galore_rank"}
    assert "__Inputs__" not in cat


def test_kind_resolution_and_parameter_layers():
    assert resolve_kind({"type": "Model", "title": "TriuneTransformer"}) == "TriuneTransformer"
    assert resolve_kind({"type": "Model", "title": "My network"}) == "Model"
    assert resolve_kind({"type": "Custom", "title": "Muon step"}) == "MuonOptimizer"
    assert resolve_kind({"type": "Custom", "title": "GGUF writer"}) == "GGUFExport"
    assert resolve_kind({"type": "", "title": ""}) is None
    p = node_params({"details": "lr=0.01\nname=adam\nbad line\nflag=true", "params": {"lr": 0.02}, "config": {"wd": {"value": 0.1}, "k": 3}})
    assert p == {"lr": 0.02, "name": "adam", "flag": True, "wd": 0.1, "k": 3}


def test_validation_of_edges_ports_types_and_cycles():
    a = {"id": "a", "type": "BPETokenizer"}
    b = {"id": "b", "type": "CyclingDataLoader"}
    ok = {"nodes": [a, b], "edges": [{"source": "a", "target": "b", "source_port": "tokens", "target_port": "tokens"}]}
    assert parse_studio_graph(ok).order == ["a", "b"]
    with pytest.raises(StudioGraphError, match="no output port"):
        parse_studio_graph({"nodes": [a, b], "edges": [{"source": "a", "target": "b", "source_port": "nope", "target_port": "tokens"}]})
    with pytest.raises(StudioGraphError, match="no input port"):
        parse_studio_graph({"nodes": [a, b], "edges": [{"source": "a", "target": "b", "source_port": "tokens", "target_port": "nope"}]})
    with pytest.raises(StudioGraphError, match="both ports or neither"):
        parse_studio_graph({"nodes": [a, b], "edges": [{"source": "a", "target": "b", "source_port": "tokens"}]})
    with pytest.raises(StudioGraphError, match="more than one incoming"):
        parse_studio_graph({"nodes": [a, b, {"id": "c", "type": "BPETokenizer"}], "edges": [
            {"source": "a", "target": "b", "source_port": "tokens", "target_port": "tokens"},
            {"source": "c", "target": "b", "source_port": "tokens", "target_port": "tokens"}]})
    with pytest.raises(StudioGraphError, match="type mismatch"):
        parse_studio_graph({"nodes": [a, {"id": "g", "type": "AutoregressiveGenerator"}], "edges": [
            {"source": "a", "target": "g", "source_port": "tokens", "target_port": "model_handle"}]})
    with pytest.raises(StudioGraphError, match="cycle"):
        parse_studio_graph({"nodes": [a, b], "edges": [{"source": "a", "target": "b"}, {"source": "b", "target": "a"}]})
    with pytest.raises(StudioGraphError, match="duplicate node id"):
        parse_studio_graph({"nodes": [a, dict(a)], "edges": []})
    with pytest.raises(StudioGraphError, match="missing node"):
        parse_studio_graph({"nodes": [a], "edges": [{"source": "a", "target": "zzz"}]})


def test_training_graph_end_to_end(tmp_path):
    """data -> tokenizer -> loader -> model -> losses / optimizer / schedule -> training step -> evaluation, generation,
    export and checkpoint, with typed edges, one untyped edge and the three ways of giving parameters."""
    g = {"nodes": [
        {"id": "data", "type": "Data", "title": "LocalFileReader", "params": {"file_path": _corpus(tmp_path)}},
        {"id": "tok", "type": "Data", "title": "BPETokenizer"},
        {"id": "dl", "type": "CyclingDataLoader", "details": "batch_size=2\nseq_len=16\nshuffle=false"},
        {"id": "model", "type": "Model", "title": "TriuneTransformer", "config": {k: {"value": v} for k, v in MODEL_CFG.items()}},
        {"id": "ce", "type": "Loss", "title": "FastCrossEntropy"},
        {"id": "z", "type": "RouterZLoss"},
        {"id": "jl", "type": "JointExitLoss"},
        {"id": "opt", "type": "Optimizer", "title": "AdamWOptimizer", "params": {"lr": 1e-3}},
        {"id": "sched", "type": "CosineLRScheduler", "params": {"step": 5, "warmup_steps": 10, "total_steps": 100}},
        {"id": "step", "type": "TrainingStep"},
        {"id": "eval", "type": "PerplexityEvaluator"},
        {"id": "gen", "type": "AutoregressiveGenerator", "params": {"max_tokens": 4, "temperature": 0.0}},
        {"id": "exp", "type": "Export", "title": "SafeTensorsExport", "params": {"save_dir": str(tmp_path)}},
        {"id": "ck", "type": "CheckpointManager", "params": {"save_dir": str(tmp_path / "ck")}},
    ], "edges": [
        {"source": "data", "target": "tok", "source_port": "text_sample", "target_port": "text"},
        {"source": "tok", "target": "dl", "source_port": "tokens", "target_port": "tokens"},
        {"source": "dl", "target": "model", "source_port": "input_ids", "target_port": "input_ids"},
        {"source": "model", "target": "ce", "source_port": "logits", "target_port": "logits"},
        {"source": "dl", "target": "ce", "source_port": "targets", "target_port": "targets"},
        {"source": "model", "target": "ce", "source_port": "router_logits", "target_port": "router_logits"},
        {"source": "model", "target": "z", "source_port": "router_logits", "target_port": "router_logits"},
        {"source": "model", "target": "jl", "source_port": "exit_logits", "target_port": "exit_logits"},
        {"source": "dl", "target": "jl", "source_port": "targets", "target_port": "targets"},
        {"source": "z", "target": "jl", "source_port": "z_loss", "target_port": "z_loss"},
        {"source": "model", "target": "opt", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "opt", "target": "sched", "source_port": "optimizer_handle", "target_port": "optimizer"},
        {"source": "model", "target": "step", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "opt", "target": "step", "source_port": "optimizer_handle", "target_port": "optimizer_handle"},
        {"source": "tok", "target": "step", "source_port": "tokens", "target_port": "tokens"},
        {"source": "step", "target": "eval", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "tok", "target": "eval", "source_port": "tokens", "target_port": "tokens"},
        {"source": "step", "target": "gen", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "data", "target": "gen", "source_port": "text_sample", "target_port": "prompt"},
        {"source": "step", "target": "exp", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "step", "target": "ck"},  # an edge without ports passes every output on
    ]}
    events = []
    r = run_studio_graph(g, emit=events.append)
    assert r["status"] == "success", r
    json.dumps(r)  # the response is JSON-safe although tensors and modules travelled between the nodes
    out = {k: v["output"] for k, v in r["results"].items()}
    assert out["model"]["ports"]["logits"]["tensor"] == [2, 16, 256]
    ce = out["ce"]["ports"]["lm_loss"]["value"]
    assert 4.5 < ce < 6.5  # about ln(256) on an untrained model
    assert out["sched"]["ports"]["scheduled_lr"]["lr"] == pytest.approx(1e-3 * 6 / 10)
    assert out["step"]["ports"]["step_metrics"]["grad_norm"] > 0
    assert set(out["eval"]["ports"]["per_exit_metrics"]) == {"reflex", "limbic", "cortex"}
    assert os.path.isfile(out["exp"]["ports"]["safetensors_file"]) and os.path.isfile(out["ck"]["ports"]["checkpoint_path"])
    assert [e["event"] for e in events].count("node_finished") == len(g["nodes"])
    # the same graph read as a training recipe
    rec = compile_to_training(g)
    assert rec["model"] == {k: v for k, v in MODEL_CFG.items() if k != "use_node_config"}
    assert rec["run"]["optimizer"] == "adamw" and rec["run"]["lr"] == 1e-3 and rec["run"]["depth_mode"] == "joint"
    assert rec["run"]["batch_size"] == 2 and rec["run"]["seq_len"] == 16 and rec["run"]["warmup_steps"] == 10
    assert rec["data"]["path"].endswith("corpus.txt")


def test_a_failing_node_stops_the_run_and_is_reported(tmp_path):
    g = {"nodes": [{"id": "r", "type": "LocalFileReader", "params": {"file_path": str(tmp_path / "missing.txt")}},
                   {"id": "t", "type": "BPETokenizer"}], "edges": [{"source": "r", "target": "t"}]}
    r = run_studio_graph(g)
    assert r["status"] == "failed" and r["failed_node"] == "r" and "no such file" in r["error"]
    assert "t" not in r["results"]
    r = run_studio_graph({"nodes": [{"id": "x", "type": "Mystery", "title": "???"}], "edges": []})
    assert r["status"] == "failed" and "no handler" in r["error"]
    # sources that would need the network say so, and read a local mirror when one is given
    r = run_studio_node({"type": "HuggingFaceStreamer"})
    assert r["status"] == "failed" and "network" in r["error"]
    r = run_studio_node({"type": "URLDatasetStreamer", "params": {"url": "file://" + _corpus(tmp_path)}})
    assert r["status"] == "success" and r["output"]["ports"]["text_sample"].startswith("hello world")
    r = run_studio_node({"type": "GGUFExport", "params": {"save_dir": str(tmp_path)}}, {"model_handle": torch.nn.Linear(4, 4)})
    assert r["node_status"] == "specification" and not list(tmp_path.glob("*.gguf"))  # settings only, as in the reference: nothing is written


def test_layer_and_kernel_nodes_compute():
    x = torch.randn(2, 16, 64)
    for kind, port in (("VectorisedGLA", "attention_out"), ("HybridAttention", "attention_out"), ("MoE_FFN", "moe_out")):
        r = run_studio_node({"type": kind, "params": {"num_heads": 1, "num_experts": 4}}, {"hidden_states": x})
        assert r["status"] == "success", r
        assert r["output"]["ports"][port]["tensor"] == [2, 16, 64] and r["output"]["ports"][port]["finite"]
    r = run_studio_node({"type": "DepthRouter"}, {"hidden_states": x})
    assert r["output"]["ports"]["router_logits"]["tensor"] == [2, 3] and r["output"]["ports"]["exit_choice"]["tensor"] == [2]
    for kind, bar in (("FP8Linear", 0.08), ("FP4Linear", 0.3)):
        r = run_studio_node({"type": kind, "params": {"out_features": 128}}, {"x": torch.randn(4, 128)})
        assert r["status"] == "success", r
        assert r["output"]["ports"]["linear_out"]["tensor"] == [4, 128] and r["output"]["relative_error_vs_full_precision"] < bar
    r = run_studio_node({"type": "RMSNorm"}, {"x": x})
    assert r["output"]["ports"]["norm_out"]["std"] == pytest.approx(1.0, abs=0.05)
    r = run_studio_node({"type": "FastRMSNorm"}, {"x": x, "weight": torch.full((64,), 2.0)})
    assert r["output"]["ports"]["norm_out"]["std"] == pytest.approx(2.0, abs=0.1)
    q = torch.randn(1, 8, 2, 32)
    r = studio.StudioGraphRunner().run({"nodes": [{"id": "i", "type": "__Inputs__", "params": {"values": {"q": q, "k": q}}},
                                                  {"id": "r", "type": "FastRoPE", "params": {"dim": 32}}],
                                        "edges": [{"source": "i", "target": "r"}]}, _keep_values=True)
    qr = r["_values"]["r"]["q_rot"]
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-4) and torch.allclose(qr[:, 0], q[:, 0], atol=1e-5)
    r = run_studio_node({"type": "TokenBatchInspector"}, {"tokens": torch.tensor([[1, 2, 2, 3]])})
    assert r["output"]["ports"]["metrics"]["unique"] == 3 and r["output"]["ports"]["metrics"]["repetition"] == 0.25
    r = run_studio_node({"type": "LoRAAdapter", "params": {"rank": 4, "target_modules": "all"}}, {"base_layer": torch.nn.Linear(16, 16)})
    assert r["status"] == "success", r


def test_runtime_nodes(tmp_path):
    r = run_studio_node({"type": "Runtime"})
    assert r["output"]["ports"]["runtime_info"]["torch"] == torch.__version__
    r = run_studio_node({"type": "VRAMProfiler"})
    assert "allocated_gb" in r["output"]["ports"]["vram_stats"]
    r = run_studio_node({"type": "DynamicResourceManager"})
    assert "hardware" in r["output"]["ports"]["feasibility_report"]
    r = run_studio_node({"type": "PythonSandbox", "params": {"code": "result = sum(range(5))\nprint('hi')"}})
    assert r["status"] == "success", r
    assert r["output"]["ports"]["result"] == 10 and "hi" in r["output"]["ports"]["stdout"]
    r = run_studio_node({"type": "PythonSandbox", "params": {"code": "import socket"}})
    assert r["status"] == "failed"
    r = run_studio_node({"type": "WandbLogger", "params": {"save_dir": str(tmp_path), "step": 3}}, {"metrics": {"loss": 1.5}})
    rec = json.loads(open(r["output"]["ports"]["log_status"]["path"]).read().splitlines()[-1])
    assert rec["step"] == 3 and rec["metrics"] == {"loss": 1.5}
    r = run_studio_node({"type": "BYOKChatRouter", "params": {"provider": "anthropic"}}, {"prompt": "hi"})
    assert r["status"] == "partial" and r["output"]["ports"]["provider_config"]["has_key"] is False
    w = torch.nn.Parameter(torch.ones(3))
    loss = (w * 2).sum()
    r = run_studio_node({"type": "GradientAccumulator", "params": {"grad_accum_steps": 2}}, {"loss": loss})
    assert r["output"]["ports"]["accum_status"]["backward"] and torch.allclose(w.grad, torch.ones(3))
    g = {"nodes": [{"id": "m", "type": "TriuneTransformer", "params": {**MODEL_CFG, "initialize_only": True}},
                   {"id": "s", "type": "LayerStreamingEngine"},
                   {"id": "f", "type": "LoRAFineTuner", "params": {"rank": 2, "steps": 2, "save_dir": str(tmp_path)}},
                   {"id": "t", "type": "__Inputs__", "params": {"values": {"tokens": torch.randint(0, 256, (2, 17))}}}],
         "edges": [{"source": "m", "target": "s", "source_port": "model_handle", "target_port": "model_handle"},
                   {"source": "m", "target": "f", "source_port": "model_handle", "target_port": "model_handle"},
                   {"source": "t", "target": "f"}]}
    r = run_studio_graph(g)
    assert r["status"] == "success", r
    assert os.path.isdir(r["results"]["f"]["output"]["ports"]["finetuned_adapter"])


def test_subgraphs_with_declared_sockets_and_the_depth_limit():
    inner = {"nodes": [{"id": "in", "type": "SubgraphInput", "params": {"public_name": "text"}},
                       {"id": "tok", "type": "BPETokenizer"}],
             "edges": [{"source": "in", "target": "tok", "source_port": "value", "target_port": "text"}],
             "inputs": [{"name": "text", "type": "text"}],
             "outputs": [{"name": "ids", "type": "tensor", "source_node": "tok", "source_port": "tokens"}]}
    g = {"nodes": [{"id": "src", "type": "__Inputs__", "params": {"values": {"text": "abc"}}},
                   {"id": "sub", "type": "Subgraph", "title": "Tokenise", "subgraph": inner},
                   {"id": "insp", "type": "TokenBatchInspector"}],
         "edges": [{"source": "src", "target": "sub"},
                   {"source": "sub", "target": "insp", "source_port": "ids", "target_port": "tokens"}]}
    r = run_studio_graph(g)
    assert r["status"] == "success", r
    assert r["results"]["insp"]["output"]["ports"]["metrics"]["shape"] == [1, 3]
    with pytest.raises(StudioGraphError, match="no output port"):  # sockets of a subgraph are checked like catalogue ports
        parse_studio_graph({"nodes": g["nodes"], "edges": [g["edges"][0], {"source": "sub", "target": "insp", "source_port": "nope", "target_port": "tokens"}]})
    r = run_studio_graph({"nodes": [g["nodes"][1]], "edges": []})
    assert r["status"] == "failed" and "missing required input" in r["error"]
    nested = {"nodes": [], "edges": [], "inputs": [], "outputs": []}
    for _ in range(studio.MAX_SUBGRAPH_DEPTH + 1):
        nested = {"nodes": [{"id": "s", "type": "Subgraph", "subgraph": nested}], "edges": [], "inputs": [], "outputs": []}
    r = run_studio_graph({"nodes": nested["nodes"], "edges": []})
    assert r["status"] == "failed" and "depth" in r["error"]


# (display title in the canvas' palette, category the canvas stores in ``type``, node kind)
PALETTE = [
    ('Hugging Face Streamer', 'Data', 'HuggingFaceStreamer'),
    ('URL Dataset Streamer', 'Data', 'URLDatasetStreamer'),
    ('Local File Reader', 'Data', 'LocalFileReader'),
    ('BPE Tokenizer', 'Data', 'BPETokenizer'),
    ('Cycling DataLoader', 'Data', 'CyclingDataLoader'),
    ('Autograd Training Step', 'Evaluation', 'TrainingStep'),
    ('Triune MoE Transformer', 'Model', 'TriuneTransformer'),
    ('Vectorised GLA Attention', 'Model', 'VectorisedGLA'),
    ('Hybrid GLA + RoPE Attention', 'Model', 'HybridAttention'),
    ('Sparse MoE FFN Layer', 'Model', 'MoE_FFN'),
    ('Hierarchical Depth Router', 'Model', 'DepthRouter'),
    ('FP8 Scaled Linear', 'Model', 'FP8Linear'),
    ('NVFP4 Microscaling Linear', 'Model', 'FP4Linear'),
    ('Tensor Inspector', 'Analysis', 'TensorInspector'),
    ('Token Batch Inspector', 'Analysis', 'TokenBatchInspector'),
    ('Fast RMSNorm', 'Model', 'RMSNorm'),
    ('LoRA Adapter Layer', 'Model', 'LoRAAdapter'),
    ('CentroidSteer Optimizer', 'Optimizer', 'CentroidSteerOptimizer'),
    ('Muon Matrix Optimizer', 'Optimizer', 'MuonOptimizer'),
    ('AdamW Optimizer', 'Optimizer', 'AdamWOptimizer'),
    ('Cosine LR Scheduler', 'Optimizer', 'CosineLRScheduler'),
    ('Fast Cross-Entropy Loss', 'Loss', 'FastCrossEntropy'),
    ('Joint Exit Loss', 'Loss', 'JointExitLoss'),
    ('Router Stability Z-Loss', 'Loss', 'RouterZLoss'),
    ('Fast RoPE Kernel', 'Model', 'FastRoPE'),
    ('Fast RMSNorm Kernel', 'Model', 'FastRMSNorm'),
    ('Autoregressive Generator', 'Model', 'AutoregressiveGenerator'),
    ('BYOK Chat Router', 'Model', 'BYOKChatRouter'),
    ('Gradient Accumulator', 'Runtime', 'GradientAccumulator'),
    ('Checkpoint Manager', 'Runtime', 'CheckpointManager'),
    ('Dynamic Resource Manager', 'Runtime', 'DynamicResourceManager'),
    ('Layer Streaming Engine', 'Runtime', 'LayerStreamingEngine'),
    ('VRAM Profiler', 'Runtime', 'VRAMProfiler'),
    ('Restricted Python Runner', 'Runtime', 'PythonSandbox'),
    ('WandB Telemetry Logger', 'Runtime', 'WandbLogger'),
    ('Perplexity Evaluator', 'Evaluation', 'PerplexityEvaluator'),
    ('LoRA Fine-Tuner Engine', 'Evaluation', 'LoRAFineTuner'),
    ('SafeTensors Exporter', 'Export', 'SafeTensorsExport'),
    ('GGUF Export (Configuration Only)', 'Export', 'GGUFExport'),
    ('ONNX Graph Exporter', 'Export', 'ONNXExport'),
    ('Reroute Node', 'Reroute', 'RerouteNode'),
]


def test_nodes_are_identified_by_their_palette_title_before_their_category(tmp_path):
    """The canvas stores the palette title in ``title`` and only the broad category in ``type``; a saved graph must resolve
    to the specific node kinds, and a reroute junction passes values through."""
    from triune_b200.execution.studio import resolve_kind

    for title, category, kind in PALETTE:
        assert resolve_kind({"id": "n", "type": category, "title": title}) == kind, title
    assert resolve_kind({"id": "n", "type": "Data", "title": "My own reader"}) == "Data"  # an unknown title falls back to the category
    g = {"nodes": [{"id": "a", "type": "Data", "title": "Local File Reader", "details": f"file_path={_corpus(tmp_path)}"},
                   {"id": "r", "type": "Reroute", "title": "Reroute Node"}, {"id": "b", "type": "Data", "title": "BPE Tokenizer"}],
         "edges": [{"source": "a", "target": "r", "source_port": "text_sample", "target_port": "in"},
                   {"source": "r", "target": "b", "source_port": "out", "target_port": "text"}]}
    out = run_studio_graph(g)
    assert out["status"] == "success" and all(r["status"] == "completed" for r in out["results"].values())
    bad = {"nodes": [{"id": "s", "type": "Data", "title": "Hugging Face Streamer"}, {"id": "t", "type": "Evaluation", "title": "Autograd Training Step"}],
           "edges": [{"source": "s", "target": "t", "source_port": "dataset_stream", "target_port": "dataset_stream"}]}
    from triune_b200.execution.studio import parse_studio_graph

    assert parse_studio_graph(bad).order == ["s", "t"]
