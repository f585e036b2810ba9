"""HTTP / WebSocket routes of the serving API.

Parity with the serving surface of ``triune/api/routes.py``: OpenAI-style ``POST /v1/chat/completions`` (JSON or
server-sent events, per-session recurrent state, cancel), model listing / loading / presets, tokenizer, sessions,
device-memory statistics, resource planning, hardware profile, training control, checkpoints, fine-tuning, sandbox,
diagnostics, kernel inventory, neuron snapshots and the ``/ws/telemetry`` stream.
"""

from __future__ import annotations

import asyncio
import json
import queue as _queue
import re
import threading
import time
import uuid
from pathlib import Path
from typing import Any, Dict, List, Optional

from fastapi import APIRouter, HTTPException, WebSocket, WebSocketDisconnect
from fastapi.responses import JSONResponse, StreamingResponse
from pydantic import BaseModel, Field

from .engine_state import get_state

router = APIRouter()


# ---------------------------------------------------------------------------------------------------- schemas
HAS_TRIUNE_MODULES = True  # the graph engine, node registry and module manager are part of this package

# UTF-8 bytes that were read as Windows-1252 ("double decoding") turn up in scraped datasets and in the output of models
# trained on them: a lead character from U+00C2..U+00F4 followed by one to three characters that Windows-1252 maps to
# 0x80..0xBF. A run is repaired only when its bytes are valid UTF-8 again; typographic punctuation that results is
# written in ASCII, as the reference does (``triune/api/routes.py:146-172``).
_CP1252_TAIL = "\u0080-\u00bf\u0152\u0153\u0160\u0161\u0178\u017d\u017e\u0192\u02c6\u02dc\u2013\u2014\u2018-\u201e\u2020-\u2022\u2026\u2030\u2039\u203a\u20ac\u2122"
_MOJIBAKE_RUN = re.compile(f"[\u00c2-\u00f4][{_CP1252_TAIL}]{{1,3}}")
_ASCII_PUNCT = {"\u2018": "'", "\u2019": "'", "\u201c": '"', "\u201d": '"', "\u2013": "-", "\u2014": "--", "\u2026": "...", "\u00a0": " "}


def _repair_run(m) -> str:
    try:
        fixed = m.group(0).encode("cp1252").decode("utf-8")
    except (UnicodeEncodeError, UnicodeDecodeError):
        return m.group(0)
    return "".join(_ASCII_PUNCT.get(ch, ch) for ch in fixed)


def sanitize_text(text: str) -> str:
    """Repair double-decoded text and drop replacement characters; anything that is not a non-empty string gives ``""``."""
    if not text or not isinstance(text, str):
        return ""
    text = _MOJIBAKE_RUN.sub(_repair_run, text)
    text = text.replace("\u00e2\u20ac", '"')  # a closing quote whose last byte (0x9D) has no Windows-1252 character and was lost
    return text.replace("\ufffd", "")


class ChatMessage(BaseModel):
    role: str = "user"
    content: str = ""


class ChatRequest(BaseModel):
    model: Optional[str] = None
    messages: List[ChatMessage] = Field(default_factory=list)
    prompt: Optional[str] = None
    max_tokens: int = 256
    temperature: float = 0.7
    top_k: int = 50
    repetition_penalty: float = 1.1
    stream: bool = False
    stop: Optional[List[str]] = None
    session_id: Optional[str] = None
    decode_depth: Optional[int] = 2
    speculative: bool = False
    request_id: Optional[str] = None


class LoadRequest(BaseModel):
    model: str
    tokenizer_path: Optional[str] = None
    precision: Optional[str] = None
    overrides: Dict[str, Any] = Field(default_factory=dict)


class TrainRequest(BaseModel):
    config: Dict[str, Any] = Field(default_factory=dict)
    max_steps: Optional[int] = None


class FinetuneRequest(BaseModel):
    records: List[Any]
    rank: int = 16
    alpha: float = 32.0
    epochs: int = 1
    lr: float = 2e-4
    batch_size: int = 4
    max_seq_len: int = 512
    use_qlora: bool = False
    output_dir: str = "adapters/latest"
    max_steps: Optional[int] = None


def _prompt_of(req: ChatRequest) -> str:
    if req.prompt is not None:
        return req.prompt
    if not req.messages:
        raise HTTPException(400, "either 'messages' or 'prompt' is required")
    *history, last = req.messages
    if not history:
        return last.content
    lines = [f"{m.role.capitalize()}: {m.content}" for m in history if m.role != "assistant" or m.content]
    return "\n".join(lines + [last.content]) if req.session_id is None else last.content


def _completion(req_id: str, model_id: str, text: str, tele: Dict[str, Any], finish: str = "stop") -> Dict[str, Any]:
    return {"id": req_id, "object": "chat.completion", "created": int(time.time()), "model": model_id,
            "choices": [{"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": finish}],
            "usage": {"prompt_tokens": int(tele.get("prompt_tokens", 0)), "completion_tokens": int(tele.get("new_tokens", 0)),
                      "total_tokens": int(tele.get("prompt_tokens", 0)) + int(tele.get("new_tokens", 0))},
            "telemetry": {k: v for k, v in tele.items() if isinstance(v, (int, float, str))}}


# ---------------------------------------------------------------------------------------------------- chat
async def _ollama_completion(req: ChatRequest):
    """``model: "ollama:<tag>"``: the request is answered by the Ollama daemon on this machine's loopback address (the
    reference's Studio offers local Ollama models next to its own, ``triune/runtime/model_scanner.py:213-470``)."""
    from ..runtime.model_scanner import stream_ollama_chat

    tag = req.model.split(":", 1)[1]
    req_id = req.request_id or f"chatcmpl-{uuid.uuid4().hex[:24]}"
    msgs = [{"role": m.role, "content": m.content} for m in req.messages] or [{"role": "user", "content": req.prompt or ""}]
    opts = {"temperature": req.temperature, "top_k": req.top_k, "num_predict": req.max_tokens, "repeat_penalty": req.repetition_penalty}
    loop = asyncio.get_running_loop()
    if not req.stream:
        try:
            text = await loop.run_in_executor(None, lambda: "".join(stream_ollama_chat(tag, msgs, options=opts)))
        except ConnectionError as e:
            raise HTTPException(502, str(e))
        except Exception as e:
            raise HTTPException(500, f"{type(e).__name__}: {e}")
        return _completion(req_id, req.model, text, {"backend": "ollama"})
    pieces: "_queue.Queue[Optional[Dict[str, Any]]]" = _queue.Queue()

    def worker():
        try:
            for piece in stream_ollama_chat(tag, msgs, options=opts):
                pieces.put({"delta": piece})
        except Exception as e:
            pieces.put({"error": f"{type(e).__name__}: {e}"})
        finally:
            pieces.put(None)

    threading.Thread(target=worker, name=f"ollama-{req_id}", daemon=True).start()

    async def sse():
        head = {"id": req_id, "object": "chat.completion.chunk", "created": int(time.time()), "model": req.model}
        yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}) + "\n\n"
        while True:
            item = await loop.run_in_executor(None, pieces.get)
            if item is None:
                break
            if "error" in item:
                yield "data: " + json.dumps({**head, "error": item["error"]}) + "\n\n"
            else:
                yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"content": item["delta"]}, "finish_reason": None}]}) + "\n\n"
        yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {}, "finish_reason": "stop"}]}) + "\n\n"
        yield "data: [DONE]\n\n"

    return StreamingResponse(sse(), media_type="text/event-stream", headers={"Cache-Control": "no-cache", "X-Request-Id": req_id})


@router.post("/v1/chat/completions")
async def chat_completions(req: ChatRequest):
    st = get_state()
    if req.model and req.model.startswith("ollama:"):
        return await _ollama_completion(req)
    if st.model is None:
        raise HTTPException(409, "no model is loaded; POST /v1/models/load first")
    req_id = req.request_id or f"chatcmpl-{uuid.uuid4().hex[:24]}"
    prompt = _prompt_of(req)
    if not st.queue.acquire(timeout=30.0):
        raise HTTPException(429, "the serving queue is full")
    cancel = st.queue.register_request(req_id)
    kw = dict(session_id=req.session_id, max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k,
              repetition_penalty=req.repetition_penalty, decode_depth=req.decode_depth, stop=req.stop, cancel_event=cancel,
              speculative=req.speculative)

    def finish():
        st.queue.unregister_request(req_id)
        st.queue.release()

    if not req.stream:
        try:
            out = await asyncio.get_running_loop().run_in_executor(None, lambda: st.generate(prompt, **kw))
        except Exception as e:
            raise HTTPException(500, f"{type(e).__name__}: {e}")
        finally:
            finish()
        return _completion(req_id, st.model_id or "triune", out["text"], out["telemetry"], "cancelled" if cancel.is_set() else "stop")

    pieces: "_queue.Queue[Optional[Dict[str, Any]]]" = _queue.Queue()

    def worker():
        try:
            out = st.generate(prompt, stream_callback=lambda s: pieces.put({"delta": s}), **kw)
            pieces.put({"done": out["telemetry"]})
        except Exception as e:
            pieces.put({"error": f"{type(e).__name__}: {e}"})
        finally:
            finish()
            pieces.put(None)

    threading.Thread(target=worker, name=f"gen-{req_id}", daemon=True).start()

    async def sse():
        head = {"id": req_id, "object": "chat.completion.chunk", "created": int(time.time()), "model": st.model_id or "triune"}
        yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}) + "\n\n"
        loop = asyncio.get_running_loop()
        while True:
            item = await loop.run_in_executor(None, pieces.get)
            if item is None:
                break
            if "delta" in item:
                yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"content": item["delta"]}, "finish_reason": None}]}) + "\n\n"
            elif "error" in item:
                yield "data: " + json.dumps({**head, "error": item["error"]}) + "\n\n"
            else:
                yield "data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {}, "finish_reason": "cancelled" if cancel.is_set() else "stop"}],
                                             "telemetry": {k: v for k, v in item["done"].items() if isinstance(v, (int, float, str))}}) + "\n\n"
        yield "data: [DONE]\n\n"

    return StreamingResponse(sse(), media_type="text/event-stream", headers={"Cache-Control": "no-cache", "X-Request-Id": req_id})


@router.post("/v1/chat/cancel")
async def chat_cancel(body: Dict[str, Any]):
    return {"cancelled": get_state().queue.cancel_request(str(body.get("request_id", "")))}


@router.get("/v1/chat/sessions")
async def list_sessions():
    st = get_state()
    return {"sessions": list(st.sessions_meta.values()), "stats": st.srsm.stats()}


@router.post("/v1/chat/sessions")
async def create_session(body: Optional[Dict[str, Any]] = None):
    sid = (body or {}).get("session_id") or f"sess-{uuid.uuid4().hex[:16]}"
    get_state().sessions_meta.setdefault(sid, {"id": sid, "created": time.time(), "turns": 0, "title": (body or {}).get("title")})
    return {"session_id": sid}


@router.delete("/v1/chat/sessions/{session_id}")
async def delete_session(session_id: str):
    st = get_state()
    st.sessions_meta.pop(session_id, None)
    return {"deleted": st.srsm.clear_session(session_id)}


# ---------------------------------------------------------------------------------------------------- models
@router.get("/v1/models")
async def list_models():
    from ..models.zoo import CANONICAL_MODEL_SPECS, MODEL_REGISTRY

    st = get_state()
    data = [{"id": k, "object": "model", "owned_by": "triune", "params": v.params_label, "tier": v.tier,
             "layers": v.num_layers, "hidden_dim": v.hidden_dim, "experts": v.num_experts} for k, v in CANONICAL_MODEL_SPECS.items()]
    data += [{"id": k, "object": "model", "owned_by": "registry"} for k in MODEL_REGISTRY]
    return {"object": "list", "data": data, "active": st.model_id}


@router.get("/v1/models/active")
async def active_model():
    st = get_state()
    return {"loaded": st.model is not None, **(st.config if st.model is not None else {})}


@router.post("/v1/models/load")
async def load_model(req: LoadRequest):
    st = get_state()
    try:
        info = await asyncio.get_running_loop().run_in_executor(
            None, lambda: st.load_model(req.model, req.tokenizer_path, req.precision, **req.overrides))
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")
    return {"status": "loaded", **info}


@router.post("/v1/models/preset")
@router.post("/v1/model/set_preset")
async def set_preset(body: Dict[str, Any]):
    from ..models.zoo import get_model_spec

    spec = get_model_spec(body.get("preset_id") or body.get("preset"), **{k: v for k, v in body.items() if k not in ("preset_id", "preset", "load")})
    out = {"spec": spec.to_dict()}
    if body.get("load"):
        out["loaded"] = get_state().load_model(spec.model_id)
    return out


@router.post("/v1/models/export")
async def export_active(body: Dict[str, Any]):
    from ..export import export_model

    st = get_state()
    try:
        path = export_model(st.require_model(), body.get("output_path", "exports/model.safetensors"), body.get("format", "safetensors"))
    except NotImplementedError as e:
        raise HTTPException(501, str(e))
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")
    return {"path": str(path)}


@router.post("/v1/model/router/temperature")
async def router_temperature(body: Dict[str, Any]):
    st = get_state()
    st.config["router_temperature"] = float(body.get("temperature", 1.0))
    return {"temperature": st.config["router_temperature"]}


# ---------------------------------------------------------------------------------------------------- tokenizer
@router.post("/v1/tokenizer/tokenize")
async def tokenize(body: Dict[str, Any]):
    st = get_state()
    tok = st.tokenizer
    if tok is None:
        from .engine_state import ByteTokenizer

        tok = ByteTokenizer()
    ids = tok.encode(str(body.get("text", "")))
    return {"ids": ids, "count": len(ids), "pieces": [tok.decode([i], skip_special_tokens=False) for i in ids[:512]]}


# ---------------------------------------------------------------------------------------------------- memory / resources
@router.get("/v1/vram/stats")
async def vram_stats():
    from ..runtime.vram import VRAMProfiler

    st = get_state()
    return VRAMProfiler.get_vram_stats(st.device) if st.device.type == "cuda" else VRAMProfiler.get_vram_stats("cpu")


@router.post("/v1/vram/purge")
@router.post("/v1/vram/offload")
async def vram_purge():
    import gc

    import torch

    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return await vram_stats()


@router.post("/v1/resource/plan")
async def resource_plan(body: Dict[str, Any]):
    from ..runtime.memory_planner import MemoryPlanner

    return MemoryPlanner.estimate_vram(body.get("config", body), available_vram_gb=body.get("available_vram_gb")).to_dict()


@router.post("/v1/resource/estimate_hf")
async def resource_estimate_hf(body: Dict[str, Any]):
    from ..runtime.memory_planner import MemoryPlanner

    return MemoryPlanner.estimate_hf_model(body.get("config", body), int(body.get("batch_size", 1)), int(body.get("seq_len", 2048)),
                                           bool(body.get("training", False)), body.get("available_vram_gb"), body.get("quantization"))


@router.post("/v1/resource/assess")
async def resource_assess(body: Dict[str, Any]):
    from dataclasses import asdict

    from ..runtime.resource_manager import DynamicResourceManager

    a = DynamicResourceManager.assess_feasibility(body.get("config", body), device=get_state().device)
    return {**asdict(a), "report": DynamicResourceManager.format_assessment_report(a)}


@router.get("/v1/hardware/profile")
async def hardware_profile():
    from dataclasses import asdict

    from ..runtime.resource_manager import DynamicResourceManager

    return asdict(DynamicResourceManager.probe_hardware(get_state().device))


# ---------------------------------------------------------------------------------------------------- training
@router.get("/v1/training/status")
async def training_status():
    return get_state().train_status


@router.post("/v1/training/start")
async def training_start(req: TrainRequest):
    try:
        return get_state().start_training(req.config, req.max_steps)
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")


@router.post("/v1/training/pause")
async def training_pause():
    return await asyncio.get_running_loop().run_in_executor(None, get_state().stop_training)


@router.post("/v1/training/step")
async def training_step(req: Optional[TrainRequest] = None):
    st = get_state()
    try:
        return await asyncio.get_running_loop().run_in_executor(None, lambda: st.training_step(req.config if req else None))
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")


@router.post("/v1/training/config")
async def training_config(body: Dict[str, Any]):
    st = get_state()
    if st.trainer is not None:
        st.trainer.config.update(body)
        return {"config": {k: v for k, v in st.trainer.config.items() if isinstance(v, (int, float, str, bool, type(None)))}}
    return {"config": body, "note": "applied when training starts"}


@router.post("/v1/training/save_checkpoint")
@router.post("/v1/checkpoints/save")
async def checkpoint_save(body: Optional[Dict[str, Any]] = None):
    b = body or {}
    try:
        return {"path": get_state().save_checkpoint(b.get("directory", "checkpoints_full"), b.get("name", "latest"))}
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")


@router.get("/v1/checkpoints")
async def checkpoints(directory: str = "checkpoints_full"):
    return {"checkpoints": get_state().list_checkpoints(directory)}


@router.post("/v1/checkpoints/load")
async def checkpoint_load(body: Dict[str, Any]):
    try:
        return get_state().load_model(str(body["path"]), body.get("tokenizer_path"))
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")


# ---------------------------------------------------------------------------------------------------- fine-tuning
@router.post("/v1/finetune/start")
async def finetune_start(req: FinetuneRequest):
    try:
        return get_state().start_finetune(**req.model_dump())
    except Exception as e:
        raise HTTPException(400, f"{type(e).__name__}: {e}")


@router.get("/v1/finetune/status")
async def finetune_status():
    return get_state().finetune_status


@router.post("/v1/finetune/cancel")
async def finetune_cancel():
    get_state().cancel_finetune()
    return {"cancelling": True}


@router.get("/v1/finetune/adapters")
async def finetune_adapters():
    from ..trainer.finetune import list_adapters

    return {"adapters": list_adapters()}


@router.post("/v1/finetune/adapter")
async def finetune_adapter(body: Dict[str, Any]):
    """Attach a saved LoRA / QLoRA adapter to the live model (``action: attach``, ``path``; rank and alpha come from the
    adapter's own ``adapter_config.json`` when it has one) or take the attached one off (``action: detach``). An adapter
    that is already attached is detached first, so adapters never nest (``triune/api/routes.py:3950-4010``)."""
    from ..trainer.finetune import LoRAConfig, TriuneFineTuner

    st = get_state()
    action = str(body.get("action", "attach")).lower()
    with st.lock:
        prev = getattr(st, "_finetuner", None)
        if prev is not None:
            prev.detach_lora()
            st._finetuner = None
            st.active_adapter = None
        if action == "detach":
            return {"status": "success", "action": "detached", "active_adapter": None}
        if action != "attach":
            raise HTTPException(400, f"unknown action {action!r} (attach or detach)")
        if st.model is None:
            raise HTTPException(409, "no model is loaded; POST /v1/models/load first")
        model = st.model
        path = Path(str(body.get("path") or "checkpoints/lora_adapter"))
        if not (path.is_dir() and (path / "adapter_config.json").is_file()):
            raise HTTPException(404, f"no adapter at {path} (a directory with adapter_config.json)")
        try:
            cfg = LoRAConfig.from_pretrained(path)
            ft = TriuneFineTuner(model, cfg)
            ft.load_adapter(path)
        except Exception as e:
            raise HTTPException(400, f"{type(e).__name__}: {e}")
        st._finetuner = ft
        st.active_adapter = {"name": path.name, "path": str(path), "rank": cfg.rank, "alpha": cfg.alpha,
                             "trainable": ft.count_trainable_parameters()}
        st.srsm.clear_all()  # cached recurrent states were computed without the adapter
        return {"status": "success", "action": "attached", "active_adapter": st.active_adapter}


@router.post("/v1/finetune/merge")
async def finetune_merge():
    st = get_state()
    ft = getattr(st, "_finetuner", None)
    if ft is None:
        raise HTTPException(409, "no adapter is attached")
    ft.merge_and_unload()
    st._finetuner = None
    return {"merged": True}


# ---------------------------------------------------------------------------------------------------- misc
@router.post("/v1/sandbox/run")
async def sandbox_run(body: Dict[str, Any]):
    from ..runtime.sandbox import PythonSandbox

    sb = PythonSandbox(timeout=int(body.get("timeout", 10)), max_memory_mb=int(body.get("max_memory_mb", 256)))
    return await asyncio.get_running_loop().run_in_executor(None, lambda: sb.execute_code(str(body.get("code", "")), body.get("locals")))


@router.get("/v1/system/diagnostics")
async def diagnostics():
    return get_state().diagnostics()


@router.get("/v1/engine/kernels")
async def engine_kernels():
    from .. import _ext

    names = sorted(n for n in dir(_ext.ext()) if not n.startswith("_")) if _ext.ext_available() else []
    return {"extension_loaded": bool(names), "arch": "sm_100a", "entry_points": names}


@router.get("/v1/playground/neurons")
async def neurons():
    st = get_state()
    if st.model is not None and not st.scope.is_active:
        st.scope.attach(st.model)
    return st.scope.get_snapshot()


@router.websocket("/ws/telemetry")
async def ws_telemetry(ws: WebSocket):
    await ws.accept()
    st = get_state()
    q: "asyncio.Queue[Dict[str, Any]]" = asyncio.Queue(maxsize=256)
    loop = asyncio.get_running_loop()

    def listener(payload):
        try:
            loop.call_soon_threadsafe(lambda: q.full() or q.put_nowait(payload))
        except RuntimeError:
            pass

    st.telemetry_listeners.append(listener)
    try:
        await ws.send_json({"type": "hello", "training": st.train_status, "model": st.config if st.model is not None else None})
        while True:
            try:
                item = await asyncio.wait_for(q.get(), timeout=2.0)
            except asyncio.TimeoutError:
                item = {"type": "heartbeat", "time": time.time(), "training": st.train_status}
            await ws.send_json(item)
    except (WebSocketDisconnect, RuntimeError):
        pass
    finally:
        if listener in st.telemetry_listeners:
            st.telemetry_listeners.remove(listener)
