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
