"""Serving API on CPU through FastAPI's test client: chat (JSON and SSE), sessions, models, training, guards."""

import json

import pytest
import torch

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402

from triune_b200.serve import create_app, reset_state  # noqa: E402
from triune_b200.serve.server import check_bind_policy  # noqa: E402

TINY = dict(vocab_size=256, hidden_dim=64, num_layers=5, num_heads=2, head_dim=32, num_experts=4, reflex_exit_layer=2,
            limbic_exit_layer=3, router_prefix_layers=1)


@pytest.fixture()
def client():
    reset_state("cpu")
    return TestClient(create_app())


def test_health_models_and_guards(client, monkeypatch):
    assert client.get("/healthz").json()["status"] == "ok"
    ids = [m["id"] for m in client.get("/v1/models").json()["data"]]
    assert "triune-base" in ids and "triune-70b" in ids
    assert client.post("/v1/chat/completions", json={"prompt": "hi"}).status_code == 409
    monkeypatch.delenv("TRIUNE_API_TOKEN", raising=False)
    with pytest.raises(RuntimeError):
        check_bind_policy("0.0.0.0")
    assert check_bind_policy("127.0.0.1") == {"ssl_certfile": None, "ssl_keyfile": None}


def test_chat_sessions_and_streaming(client):
    torch.manual_seed(0)
    r = client.post("/v1/models/load", json={"model": "triune-nano", "overrides": TINY})
    assert r.status_code == 200 and r.json()["num_layers"] == 5
    sid = client.post("/v1/chat/sessions", json={}).json()["session_id"]
    body = {"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "temperature": 0.0, "session_id": sid}
    out = client.post("/v1/chat/completions", json=body).json()
    assert out["object"] == "chat.completion" and out["usage"]["completion_tokens"] <= 6
    first_prompt = out["usage"]["prompt_tokens"]
    out2 = client.post("/v1/chat/completions", json=body).json()  # resumes from the parked recurrent state
    assert out2["usage"]["prompt_tokens"] == first_prompt
    assert client.get("/v1/chat/sessions").json()["stats"]["active_sessions"] == 1
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True, "session_id": None}) as s:
        lines = [l for l in s.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]" and json.loads(lines[0][6:])["choices"][0]["delta"]["role"] == "assistant"
    assert client.delete(f"/v1/chat/sessions/{sid}").json()["deleted"]
    tok = client.post("/v1/tokenizer/tokenize", json={"text": "abc"}).json()
    assert tok["count"] == 3


def test_training_step_resources_and_sandbox(client):
    client.post("/v1/models/load", json={"model": "triune-nano", "overrides": TINY})
    s1 = client.post("/v1/training/step", json={"config": {"batch_size": 2, "seq_len": 32}}).json()
    s2 = client.post("/v1/training/step", json={"config": {}}).json()
    assert s2["step"] == s1["step"] + 1 and s2["loss"] > 0
    plan = client.post("/v1/resource/plan", json={"config": {**TINY, "batch_size": 4, "seq_len": 128}, "available_vram_gb": 180}).json()
    assert plan["fits"] and plan["recommended_mode"] == "resident"
    sb = client.post("/v1/sandbox/run", json={"code": "result = sum(range(5))"}).json()
    assert sb["success"] and sb["result"] == 10
    assert client.post("/v1/sandbox/run", json={"code": "import os"}).json()["success"] is False
    d = client.get("/v1/system/diagnostics").json()
    assert d["model"]["num_layers"] == 5
    snap = client.get("/v1/playground/neurons").json()
    assert "layer_bins" in snap


def test_shell_routes(client, tmp_path):
    """Product-shell endpoints: DAG execution and single nodes, node catalogue, plugins, system config, datasets,
    checkpoints (save, export, delete, path confinement), optimizer hyper-parameters, tuning knobs, provider keys."""
    cat = client.get("/v1/nodes/catalog").json()["nodes"]
    assert {"constant", "concat_text", "generate"} <= {n["type"] for n in cat}
    dag = {"nodes": [{"id": "a", "type": "text", "params": {"text": "foo"}}, {"id": "b", "type": "text", "params": {"text": "bar"}},
                     {"id": "c", "type": "concat_text", "params": {"separator": "-"}}],
           "edges": [{"from": "a.out", "to": "c.a"}, {"from": "b.out", "to": "c.b"}]}
    out = client.post("/v1/dag/execute", json={"dag": dag}).json()
    assert out["outputs"]["c.out"] == "foo-bar" and out["order"][-1] == "c"
    bad = client.post("/v1/dag/execute", json={"dag": {"nodes": [{"id": "x", "type": "no_such_node"}]}})
    assert bad.status_code == 422
    one = client.post("/v1/dag/execute_node", json={"type": "concat_text", "params": {"separator": "+"}, "inputs": {"a": "1", "b": "2"}})
    assert one.json()["outputs"] == {"out": "1+2"}

    assert client.get("/v1/plugins").json() == {"plugins": []} or isinstance(client.get("/v1/plugins").json()["plugins"], list)
    assert client.post("/v1/modules/scan_local", json={"directory": str(tmp_path / "none")}).status_code == 404
    found = client.get("/v1/modules/search").json()  # the modules that ship with the framework; remote catalogues are not asked
    assert {r["download_url"] for r in found["results"]} == {"builtin://custom_loss_nodes", "builtin://code_assistant_lora"} and found["github"] == []
    assert client.get("/v1/modules/search", params={"q": "zzz"}).json()["results"] == []

    cfg = client.post("/v1/system/config", json={"plugin_dir": str(tmp_path)}).json()["config"]
    assert cfg["plugin_dir"] == str(tmp_path)
    assert client.post("/v1/system/config", json={"nope": 1}).status_code == 400

    data = tmp_path / "corpus.txt"
    data.write_text("hello world\n" * 10)
    reg = client.post("/v1/datasets/local/register", json={"path": str(data), "name": "toy"}).json()
    assert reg["files"] == 1 and reg["bytes"] == data.stat().st_size
    assert client.post("/v1/datasets/select", json={"name": "toy"}).json()["train_config"]["dataset_path"] == str(data)
    assert client.get("/v1/datasets").json()["selected"] == "toy"
    assert client.post("/v1/datasets/select", json={"name": "other"}).status_code == 404

    assert client.post("/v1/training/optimizer", json={"lr": 1e-3}).status_code == 409
    assert client.post("/v1/checkpoints/export", json={"path": str(tmp_path / "m.safetensors")}).status_code == 409
    client.post("/v1/models/load", json={"model": "triune-nano", "overrides": TINY})
    client.post("/v1/training/step", json={"config": {"batch_size": 2, "seq_len": 32}})
    ch = client.post("/v1/training/optimizer", json={"lr": 5e-4}).json()
    assert ch["changed"] == {"lr": 5e-4}
    exp = client.post("/v1/checkpoints/export", json={"path": str(tmp_path / "m.safetensors"), "format": "safetensors"}).json()
    assert (tmp_path / "m.safetensors").stat().st_size > 1000 and exp["format"] == "safetensors"
    ck = tmp_path / "ck"
    client.post("/v1/checkpoints/save", json={"directory": str(ck), "name": "t1"})
    assert (ck / "t1.pt").is_file()
    assert client.post("/v1/checkpoints/delete", json={"directory": str(ck), "name": "../m.safetensors"}).status_code in (400, 404)
    assert (tmp_path / "m.safetensors").is_file()
    gone = client.post("/v1/checkpoints/delete", json={"directory": str(ck), "name": "t1.pt"}).json()
    assert not (ck / "t1.pt").exists() and gone["checkpoints"] == []

    import time as _time

    for n in ("a1", "a2", "a3"):
        client.post("/v1/checkpoints/save", json={"directory": str(ck), "name": n})
        _time.sleep(0.02)
        assert client.post("/v1/checkpoints/assign_project", json={"directory": str(ck), "name": f"{n}.pt", "project": "runA"}).status_code == 200
    client.post("/v1/checkpoints/save", json={"directory": str(ck), "name": "loose"})
    grouped = client.get("/v1/checkpoints/projects", params={"directory": str(ck)}).json()
    assert [c["name"] for c in grouped["projects"]["runA"]] == ["a1.pt", "a2.pt", "a3.pt"]
    assert [c["name"] for c in grouped["unassigned"]] == ["loose.pt"]
    pruned = client.post("/v1/checkpoints/prune_project", json={"directory": str(ck), "project": "runA", "keep": 1}).json()
    assert pruned["kept"] == ["a3.pt"] and sorted(pruned["deleted"]) == ["a1.pt", "a2.pt"] and (ck / "loose.pt").is_file()
    assert client.post("/v1/checkpoints/assign_project", json={"directory": str(ck), "name": "../x.pt", "project": "p"}).status_code in (400, 404)
    assert client.post("/v1/checkpoints/prune_project", json={"directory": str(ck), "project": "nope"}).status_code == 404

    knobs = client.post("/v1/hardware/tune", json={"knobs": {"TRIUNE_GEMM_PAIR_MIN_K": 1024}}).json()
    assert knobs["tuning"]["TRIUNE_GEMM_PAIR_MIN_K"] == "1024"
    client.post("/v1/hardware/tune", json={"knobs": {"TRIUNE_GEMM_PAIR_MIN_K": None}})
    assert client.get("/v1/system/config").json()["tuning"]["TRIUNE_GEMM_PAIR_MIN_K"] is None
    assert client.post("/v1/hardware/tune", json={"knobs": {"PATH": 1}}).status_code == 400
    saved = client.post("/v1/byok/save", json={"provider": "Example", "api_key": "sk-1234567890"}).json()
    assert saved["stored"] and "1234567" not in json.dumps(saved)
    assert client.post("/v1/byok/test", json={"provider": "example"}).json()["configured"]
    assert "gemm" in client.get("/v1/engine/benchmarks").json()["cases"]
    if not torch.cuda.is_available():  # the timed endpoints start child processes on a GPU; without one they say so
        assert client.post("/v1/engine/benchmarks", json={"case": "gemm"}).status_code == 409
        assert client.post("/v1/hardware/autotune", json={"m": 256, "n": 256, "k": 256}).status_code == 409
        from triune_b200.serve.routes_shell import _kernel_bench

        with pytest.raises(RuntimeError):  # the child runs, finds no GPU, exits non-zero: reported, not swallowed
            _kernel_bench("gemm", {"m": 256, "n": 256, "k": 256, "iters": 1}, {"TRIUNE_GEMM_PAIR": 0}, timeout=300)
    assert client.post("/v1/engine/benchmarks", json={"case": "nope"}).status_code == 404


def test_agents_and_turbo_mode(client, tmp_path):
    """Agent endpoints drive the loaded model; turbo mode answers greedy requests through the graph decoder's step
    function (eager on CPU) with the same tokens as the sampling path at temperature 0."""
    assert client.post("/v1/agents/run", json={"message": "hi"}).status_code == 409
    torch.manual_seed(0)
    client.post("/v1/models/load", json={"model": "triune-nano", "overrides": TINY})
    p = client.post("/v1/agents/persona", json={"name": "terse", "system_prompt": "Answer briefly.", "temperature": 0.0}).json()
    assert p["persona"]["name"] == "terse"
    mem = client.post("/v1/agents/memory", json={"set": {"colour": "green"}}).json()
    assert mem["items"] == {"colour": "green"}
    run = client.post("/v1/agents/run", json={"message": "hello", "max_tokens": 4}).json()
    assert run["persona"] == "terse" and isinstance(run["text"], str)
    team = client.post("/v1/agents/orchestrate", json={"task": "say hi", "max_tokens": 3}).json()
    assert [s["agent"] for s in team["steps"]] == ["planner", "worker"]
    st = client.get("/v1/agents/state").json()
    assert st["runs"] == 1 and st["memory_items"] == 1 and len(st["tools"]) > 0
    # the harness form: persona by the goal's words, workspace tools without the writing ones, a lesson kept on disk
    (tmp_path / "ws").mkdir()
    h = client.post("/v1/agents/run", json={"goal": "review the code for security risk", "workspace": str(tmp_path / "ws"), "max_tokens": 3,
                                            "store_dir": str(tmp_path / "store")}).json()
    assert h["persona"] == "sentinel" and "read_file" in h["tools_offered"] and "write_file" not in h["tools_offered"] and "shell" not in h["tools_offered"]
    assert (tmp_path / "store" / "memory.json").is_file()
    t = client.post("/v1/agents/run", json={"goal": "plan it", "team": ["architect", "engineer"], "max_tokens": 3, "store_dir": str(tmp_path / "store"),
                                            "workspace": str(tmp_path / "ws")}).json()
    assert [x["agent"] for x in t["steps"]] == ["architect", "engineer"]

    # pure greedy decoding of the same prompt, token by token through the ordinary model call
    from triune_b200.inference import generate_tokens
    from triune_b200.serve import get_state

    st = get_state()
    ids = torch.tensor([st.tokenizer.encode("User: abc\nAssistant:")])
    want, _, _ = generate_tokens(st.model, ids, 8, temperature=0.0, repetition_penalty=1.0, count_penalty=0.0)
    body = {"prompt": "abc", "max_tokens": 8, "temperature": 0.0, "repetition_penalty": 1.0}
    assert client.post("/v1/engine/turbo_mode", json={"enabled": True}).json()["turbo_mode"]
    out = st.generate("abc", max_new_tokens=8, temperature=0.0, repetition_penalty=1.0)
    assert out["telemetry"]["turbo"] and out["tokens"] == want
    turbo = client.post("/v1/chat/completions", json=body).json()
    assert turbo["usage"]["completion_tokens"] == len(want)
    sampled = st.generate("abc", max_new_tokens=4, temperature=0.7)  # anything but pure greedy keeps the sampling path
    assert "turbo" not in sampled["telemetry"]
    client.post("/v1/engine/turbo_mode", json={"enabled": False})
    assert "turbo" not in st.generate("abc", max_new_tokens=2, temperature=0.0, repetition_penalty=1.0)["telemetry"]


def test_adapter_export_and_upgrade_guards(client, tmp_path):
    """Adapter export re-writes saved LoRA weights; the upgrade endpoints refuse anything that is not a local model."""
    torch.save({"layers.0.lora_A": torch.randn(4, 8), "layers.0.lora_B": torch.zeros(8, 4)}, tmp_path / "adapter_model.pt")
    out = client.post("/v1/finetune/export", json={"adapter_path": str(tmp_path), "output_path": str(tmp_path / "a.safetensors")})
    assert out.status_code == 200 and (tmp_path / "a.safetensors").stat().st_size > 100
    assert client.post("/v1/finetune/export", json={"adapter_path": str(tmp_path / "missing")}).status_code == 404
    assert client.post("/v1/models/upgrade_to_triune", json={"source": "org/some-remote-model"}).status_code == 404
    assert client.post("/v1/models/distill", json={"source": str(tmp_path / "nothing-here")}).status_code == 404


def test_canvas_graphs_over_http(client, tmp_path):
    """The Studio canvas format on the DAG endpoints: execution with node events on the telemetry channel, the run queue,
    single nodes, the catalogue, and a graph compiled into the live engine's model and training settings."""
    from triune_b200.serve.engine_state import get_state

    cat = client.get("/v1/nodes/catalog").json()["studio_nodes"]
    assert len(cat) == 50 and {"TriuneTransformer", "TrainingStep", "Subgraph", "RerouteNode"} <= {n["name"] for n in cat}
    assert client.get("/v1/dag/queue").json() == {"active_run_id": None, "waiting": 0, "capacity": 1}
    corpus = tmp_path / "c.txt"
    corpus.write_text("a few words of text for the graph to read and tokenise\n")
    cfg = {"hidden_dim": 64, "num_layers": 4, "num_heads": 1, "num_experts": 4, "vocab_size": 256}
    g = {"run_id": "run-1", "nodes": [
        {"id": "d", "type": "Data", "title": "LocalFileReader", "params": {"file_path": str(corpus)}},
        {"id": "t", "type": "BPETokenizer"},
        {"id": "m", "type": "Model", "title": "TriuneTransformer", "params": {**cfg, "use_node_config": True}},
        {"id": "o", "type": "AdamWOptimizer", "params": {"lr": 2e-3, "weight_decay": 0.0}},
        {"id": "s", "type": "TrainingStep", "params": {"grad_accum_steps": 2, "max_grad_norm": 0.5}},
    ], "edges": [
        {"source": "d", "target": "t", "source_port": "text_sample", "target_port": "text"},
        {"source": "t", "target": "m", "source_port": "tokens", "target_port": "input_ids"},
        {"source": "m", "target": "o", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "m", "target": "s", "source_port": "model_handle", "target_port": "model_handle"},
        {"source": "o", "target": "s", "source_port": "optimizer_handle", "target_port": "optimizer_handle"},
        {"source": "t", "target": "s", "source_port": "tokens", "target_port": "tokens"},
    ]}
    events = []
    get_state().telemetry_listeners.append(events.append)
    out = client.post("/v1/dag/execute", json=g).json()
    assert out["status"] == "success" and out["run_id"] == "run-1", out
    assert out["results"]["s"]["output"]["ports"]["step_metrics"]["tokens"] > 0
    dag_events = [e["data"] for e in events if e.get("type") == "dag_event"]
    assert [e["event"] for e in dag_events].count("node_finished") == 5 and all(e["run_id"] == "run-1" for e in dag_events)
    bad = client.post("/v1/dag/execute", json={"nodes": [{"id": "a", "type": "BPETokenizer"}], "edges": [{"source": "a", "target": "b"}]})
    assert bad.status_code == 422
    one = client.post("/v1/dag/execute_node", json={"type": "RouterZLoss", "params": {"coeff": 1.0}, "inputs": {}})
    assert one.json()["status"] == "failed" and "router logits" in one.json()["error"]
    one = client.post("/v1/dag/execute_node", json={"node": {"type": "Runtime", "title": "Runtime"}})
    assert one.json()["status"] == "success"

    rec = client.post("/v1/dag/compile_to_training", json=g).json()
    assert rec["status"] == "compiled" and rec["applied"]["model_architecture"]["num_layers"] == 4
    assert rec["applied"]["training"] == {"optimizer": "adamw", "lr": 2e-3, "weight_decay": 0.0, "grad_accum_steps": 2, "grad_clip": 0.5}
    st = get_state()
    assert st.model is not None and st.model.num_layers == 4 and st.pending_training_config["optimizer"] == "adamw"
    step = client.post("/v1/training/step", json={"batch_size": 2, "seq_len": 16}).json()
    assert step["step"] == 1 and step["loss"] > 0
    assert type(st.trainer.optimizer).__name__ == "AdamW" and st.trainer.optimizer.param_groups[0]["lr"] > 0
    same = client.post("/v1/model/compile_dag", json={**g, "apply_model": False}).json()
    assert "model_architecture" not in same["applied"]


def test_module_lifecycle_dataset_stream_and_adapter_endpoints(client, tmp_path):
    """Install (copy or local git clone) / pull / uninstall of modules inside the plugin directory, a local dataset made the
    active stream, and a saved adapter attached to and detached from the live model. Remote sources are refused plainly."""
    import subprocess

    from triune_b200.plugins.registry import create_plugin
    from triune_b200.serve.engine_state import get_state

    plug_dir = tmp_path / "plugins"
    client.post("/v1/system/config", json={"plugin_dir": str(plug_dir)})
    src = create_plugin(tmp_path / "src", "echo_tools")
    r = client.post("/v1/modules/install", json={"path": str(src)})
    assert r.status_code == 200 and r.json()["status"] == "installed" and r.json()["plugins_found"] == ["echo_tools"], r.text
    assert (plug_dir / "echo_tools" / "plugin.json").is_file()
    assert client.post("/v1/modules/install", json={"path": str(src)}).status_code == 409
    assert client.post("/v1/modules/install", json={"url": "https://github.com/x/y"}).status_code == 501
    assert client.post("/v1/modules/install", json={"path": str(src), "name": "../escape"}).status_code == 403
    # a local git repository is cloned, and pulled after a new commit
    repo = tmp_path / "repo"
    repo.mkdir()
    git = ["git", "-C", str(repo), "-c", "user.email=a@b", "-c", "user.name=t"]
    subprocess.run(["git", "init", "-q", str(repo)], check=True)
    (repo / "README.md").write_text("one\n")
    subprocess.run(git + ["add", "-A"], check=True)
    subprocess.run(git + ["commit", "-qm", "one"], check=True)
    r = client.post("/v1/modules/clone", json={"url": "file://" + str(repo), "name": "cloned"})
    assert r.status_code == 200 and r.json()["is_git"], r.text
    (repo / "README.md").write_text("two\n")
    subprocess.run(git + ["commit", "-qam", "two"], check=True)
    r = client.post("/v1/modules/pull", json={"id": "cloned"})
    assert r.status_code == 200 and (plug_dir / "cloned" / "README.md").read_text() == "two\n", r.text
    assert client.post("/v1/modules/pull", json={"id": "echo_tools"}).status_code == 404
    assert client.post("/v1/modules/uninstall", json={"id": "cloned"}).json()["status"] == "uninstalled"
    assert not (plug_dir / "cloned").exists()
    assert client.post("/v1/modules/uninstall", json={"id": "cloned"}).status_code == 404

    assert client.get("/v1/datasets/stream/status").json()["is_streaming"] is False
    assert client.post("/v1/datasets/stream/connect", json={"dataset_name": "roneneldan/TinyStories"}).json()["status"] == "error"
    corpus = tmp_path / "c.jsonl"
    corpus.write_text(json.dumps({"text": "first document"}) + "\n" + json.dumps({"text": "second"}) + "\n")
    r = client.post("/v1/datasets/stream/connect", json={"dataset_name": "file://" + str(corpus)}).json()
    assert r["status"] == "connected" and r["buffered_chunks"] == 2 and r["sample_preview"] == "first document"
    assert client.get("/v1/datasets/stream/status").json()["path"] == str(corpus)

    assert client.post("/v1/finetune/adapter", json={"action": "attach", "path": str(tmp_path / "none")}).status_code == 409  # no model yet
    client.post("/v1/models/load", json={"model": "triune-nano", "overrides": TINY})
    assert client.post("/v1/finetune/adapter", json={"action": "attach", "path": str(tmp_path / "none")}).status_code == 404
    from triune_b200.trainer.finetune import LoRAConfig, TriuneFineTuner

    st = get_state()
    ft = TriuneFineTuner(st.model, LoRAConfig(rank=2, alpha=4.0))
    for p in ft.get_trainable_parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = torch.randint(0, 256, (1, 8))
    ft.save_adapter(tmp_path / "ad")
    ft.detach_lora()
    with torch.no_grad():
        y_base = st.model(x, force_depth=2)[0].clone()
    ft2 = TriuneFineTuner(st.model, LoRAConfig.from_pretrained(tmp_path / "ad"))
    ft2.load_adapter(tmp_path / "ad")  # what the saved adapter computes (rows a fused projection masks are not saved)
    with torch.no_grad():
        y_adapted = st.model(x, force_depth=2)[0].clone()
    ft2.detach_lora()
    assert not torch.allclose(y_adapted, y_base)
    r = client.post("/v1/finetune/adapter", json={"action": "attach", "path": str(tmp_path / "ad")}).json()
    assert r["action"] == "attached" and r["active_adapter"]["rank"] == 2
    with torch.no_grad():
        assert torch.allclose(st.model(x, force_depth=2)[0], y_adapted, atol=1e-5)
    client.post("/v1/finetune/adapter", json={"action": "attach", "path": str(tmp_path / "ad")})  # re-attach: no nesting
    with torch.no_grad():
        assert torch.allclose(st.model(x, force_depth=2)[0], y_adapted, atol=1e-5)
    assert client.post("/v1/finetune/adapter", json={"action": "detach"}).json()["action"] == "detached"
    with torch.no_grad():
        assert torch.allclose(st.model(x, force_depth=2)[0], y_base, atol=1e-6)


def test_studio_page_is_served_and_matches_the_api(client):
    """The packaged single-page Studio: served at / with its script and stylesheet; every API path the script calls is a
    route of this server, and every element id the script looks up exists in the page."""
    import re
    from pathlib import Path

    import triune_b200

    root = Path(triune_b200.__file__).parent / "studio"
    page = client.get("/")
    assert page.status_code == 200 and "Triune Studio" in page.text and page.headers["cache-control"].startswith("no-cache")
    js = client.get("/static/app.js")
    assert js.status_code == 200 and js.text == (root / "app.js").read_text()
    assert client.get("/static/style.css").status_code == 200
    assert "Triune Studio" in client.get("/some/client/side/route").text  # unknown paths fall back to the page
    routes = {getattr(r, "path", "") for r in client.app.routes}
    called = set(re.findall(r'"(/(?:v1|ws)/[A-Za-z0-9_/]+?)/?"', js.text))
    assert len(called) >= 25
    for path in called:
        assert path in routes or any(r.startswith(path + "/{") for r in routes), path
    ids = set(re.findall(r'\$\("#([A-Za-z0-9_-]+)"\)', js.text))  # ids completed at run time ("#node-" + id) are not literals
    html_ids = set(re.findall(r'id="([A-Za-z0-9_-]+)"', page.text))
    assert ids and ids <= html_ids, sorted(ids - html_ids)


def test_chat_through_a_local_ollama_daemon(client, monkeypatch):
    """``model: "ollama:<tag>"`` is answered by the daemon on the loopback address, with and without streaming; a daemon
    that does not answer is a 502."""
    from triune_b200.runtime import model_scanner as ms

    calls = []

    def fake(tag, msgs, base_url=ms.OLLAMA_URL, options=None, timeout=120.0):
        calls.append((tag, msgs, options))
        if tag == "down":
            raise ConnectionError("no Ollama daemon answers")
        yield from ("Hi", " there")

    monkeypatch.setattr(ms, "stream_ollama_chat", fake)
    body = {"model": "ollama:gemma3:4b", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 5, "temperature": 0.0}
    r = client.post("/v1/chat/completions", json=body)  # no local model is loaded: not needed for this backend
    assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] == "Hi there" and r.json()["model"] == "ollama:gemma3:4b"
    assert calls[0][0] == "gemma3:4b" and calls[0][1] == [{"role": "user", "content": "hello"}] and calls[0][2]["num_predict"] == 5
    with client.stream("POST", "/v1/chat/completions", json={**body, "stream": True}) as s:
        text = "".join(json.loads(l[6:])["choices"][0]["delta"].get("content", "") for l in s.iter_lines() if l.startswith("data: {"))
    assert text == "Hi there"
    assert client.post("/v1/chat/completions", json={**body, "model": "ollama:down"}).status_code == 502
