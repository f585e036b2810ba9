"""Process-wide serving / training state behind the HTTP API.

Parity: ``RealPyTorchEngineState`` (``triune/api/routes.py:752-3150``): owns the active model, tokenizer, optimizer,
a background training loop, generation, checkpoints and telemetry. This class is the thin stateful layer; every
operation delegates to the library (``inference``, ``Trainer``, ``TriuneFineTuner``, ``SessionRecurrentStateManager``).
"""

from __future__ import annotations

import os
import threading
import time
import uuid
from pathlib import Path
from typing import Any, Callable, Dict, Iterator, List, Optional

import torch

from ..callbacks import global_emitter
from ..runtime.neuron_scope import NeuronScope
from .srsm import ServingRequestQueue, SessionRecurrentStateManager


class ByteTokenizer:
    """Fallback tokenizer (UTF-8 bytes) so a freshly built model can be exercised without a vocabulary file."""

    pad_token_id, sep_token_id, eos_token_id = None, None, None

    def __init__(self, vocab_size: int = 256):
        self.vocab_size = vocab_size

    def encode(self, text: str) -> List[int]:
        return [b % self.vocab_size for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(int(i) % 256 for i in ids).decode("utf-8", errors="replace")

    def get_vocab_size(self) -> int:
        return self.vocab_size


class _TokAdapter:
    """Uniform ``encode -> list[int]`` / ``decode`` over ``tokenizers.Tokenizer``, the pure-Python BPE and HF tokenizers."""

    def __init__(self, tok):
        self.tok = tok
        for name in ("pad_token_id", "sep_token_id", "eos_token_id"):
            v = getattr(tok, name, None)
            if v is None and hasattr(tok, "token_to_id"):
                v = tok.token_to_id({"pad_token_id": "[PAD]", "sep_token_id": "[SEP]", "eos_token_id": "<|eot_id|>"}[name])
            setattr(self, name, v)

    def encode(self, text: str) -> List[int]:
        out = self.tok.encode(text)
        return list(getattr(out, "ids", out))

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        try:
            return self.tok.decode(list(ids), skip_special_tokens=skip_special_tokens)
        except TypeError:
            return self.tok.decode(list(ids))

    def get_vocab_size(self) -> int:
        t = self.tok
        return t.get_vocab_size() if hasattr(t, "get_vocab_size") else len(t)


class EngineState:
    def __init__(self, device: Optional[str] = None):
        self.device = torch.device(device or ("cuda:0" if torch.cuda.is_available() else "cpu"))
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = None
        self.tokenizer: Any = None
        self.model_id: Optional[str] = None
        self.config: Dict[str, Any] = {}
        self.srsm = SessionRecurrentStateManager()
        self.queue = ServingRequestQueue(16)
        self.scope = NeuronScope()
        self.trainer = None
        self._train_thread: Optional[threading.Thread] = None
        self._train_stop = threading.Event()
        self.train_status: Dict[str, Any] = {"running": False, "step": 0, "loss": None, "tok_s": 0.0, "error": None}
        self.finetune_status: Dict[str, Any] = {"running": False, "step": 0, "loss": None, "error": None, "adapter_dir": None}
        self._ft_cancel = threading.Event()
        self.lock = threading.RLock()
        self.telemetry_listeners: List[Callable[[Dict[str, Any]], None]] = []
        self.sessions_meta: Dict[str, Dict[str, Any]] = {}
        self.pending_training_config: Dict[str, Any] = {}  # settings compiled from a canvas graph, used by the next trainer
        self.turbo_mode = False          # greedy requests without a session decode through the graph-replayed decoder
        self._turbo_decoder = None       # (model object, depth) -> GraphedGreedyDecoder, rebuilt when either changes

    # ------------------------------------------------------------------ model lifecycle
    def load_model(self, spec: str, tokenizer_path: Optional[str] = None, precision: Optional[str] = None, **overrides) -> Dict[str, Any]:
        from ..data.tokenizer import load_tokenizer
        from ..inference import load_model_for_inference
        from ..models.zoo import load_model
        from ..utils import place_model

        with self.lock:
            self.stop_training()
            if os.path.exists(spec) and not spec.endswith(".json"):
                model = load_model_for_inference(spec, self.device, self.dtype)
            else:
                model = place_model(load_model(spec, **overrides), self.device, self.dtype).eval()
            if precision in ("fp8", "fp4", "nvfp4"):
                from ..recipes import apply_precision

                precision = apply_precision(model, precision, self.device)
            self.model, self.model_id = model, spec
            if tokenizer_path and os.path.exists(tokenizer_path):
                self.tokenizer = _TokAdapter(load_tokenizer(tokenizer_path))
            elif self.tokenizer is None or self.tokenizer.get_vocab_size() > int(getattr(model, "vocab_size", 1 << 30)):
                self.tokenizer = ByteTokenizer(min(256, int(getattr(model, "vocab_size", 256))))
            self.srsm.clear_all()
            self.scope.detach()
            self.trainer = None
            n = sum(p.numel() for p in model.parameters())
            self.config = {"model_id": spec, "params": n, "precision": precision or str(self.dtype).split(".")[-1],
                           "vocab_size": int(getattr(model, "vocab_size", 0)), "num_layers": int(getattr(model, "num_layers", 0)),
                           "hidden_dim": int(getattr(model, "hidden_dim", 0))}
            return dict(self.config)

    def require_model(self):
        if self.model is None:
            raise RuntimeError("no model is loaded; POST /v1/models/load first")
        return self.model

    # ------------------------------------------------------------------ generation
    def generate(self, prompt: str, *, session_id: Optional[str] = None, max_new_tokens: int = 256, temperature: float = 0.7,
                 top_k: int = 50, repetition_penalty: float = 1.1, decode_depth: Optional[int] = 2, stop=None, template: bool = True,
                 stream_callback: Optional[Callable[[str], None]] = None, cancel_event: Optional[threading.Event] = None,
                 speculative: bool = False) -> Dict[str, Any]:
        from ..inference import DEFAULT_STOPS, generate_response

        model = self.require_model()
        if (self.turbo_mode and temperature <= 0 and not session_id and stream_callback is None and not speculative
                and repetition_penalty == 1.0):
            return self._generate_turbo(model, prompt, max_new_tokens, decode_depth, stop, template)
        cache = None
        if session_id:
            hit = self.srsm.get_session_cache(session_id, self.device)
            if hit is not None:
                cache = hit[0]
        out = generate_response(model, self.tokenizer, prompt, max_new_tokens=max_new_tokens, temperature=temperature, top_k=top_k,
                                repetition_penalty=repetition_penalty, decode_depth=decode_depth,
                                stop=tuple(stop) if stop else DEFAULT_STOPS, stream_callback=stream_callback,
                                cancel_event=cancel_event, cache=cache, template=template, device=self.device,
                                speculative=speculative)
        if session_id and out.get("cache") is not None:
            self.srsm.update_session_cache(session_id, out["cache"], depth=decode_depth)
            meta = self.sessions_meta.setdefault(session_id, {"id": session_id, "created": time.time(), "turns": 0})
            meta["turns"] += 1
            meta["last_active"] = time.time()
        out.pop("cache", None)
        return out

    def _generate_turbo(self, model, prompt: str, max_new_tokens: int, decode_depth, stop, template: bool) -> Dict[str, Any]:
        """Pure greedy decoding with the per-token step replayed from one CUDA graph (eager on CPU): no sampling, no
        repetition penalty, no per-token callbacks, so the whole answer costs one host synchronisation."""
        from ..inference import DEFAULT_STOPS, GraphedGreedyDecoder, _cut_at_stop

        with self.lock:
            key = (id(model), decode_depth)
            if self._turbo_decoder is None or self._turbo_decoder[0] != key:
                self._turbo_decoder = (key, GraphedGreedyDecoder(model, 1, decode_depth))
            dec = self._turbo_decoder[1]
            text_in = f"User: {prompt}\nAssistant:" if template else prompt
            ids = torch.tensor([self.tokenizer.encode(text_in)], device=self.device, dtype=torch.long)
            n = max(1, min(int(max_new_tokens), 8192))
            t0 = time.perf_counter()
            dec.prefill(ids)
            t1 = time.perf_counter()
            toks = dec.decode(n)[0].tolist()
            t2 = time.perf_counter()
        eos = getattr(self.tokenizer, "sep_token_id", getattr(self.tokenizer, "eos_token_id", None))
        if eos is not None and eos in toks:
            toks = toks[: toks.index(eos)]
        text = self.tokenizer.decode(toks)
        tele = {"turbo": True, "prompt_tokens": int(ids.shape[1]), "ttft_s": t1 - t0, "new_tokens": len(toks),
                "decode_tok_s": n / max(1e-9, t2 - t1), "graph_replayed": self.device.type == "cuda"}
        return {"text": _cut_at_stop(text, tuple(stop) if stop else DEFAULT_STOPS), "tokens": toks, "telemetry": tele}

    # ------------------------------------------------------------------ training
    def _ensure_trainer(self, cfg: Dict[str, Any]):
        from ..data import SyntheticTokenSource
        from ..optim import CentroidSteerOptimizer
        from ..trainer import Trainer

        model = self.require_model()
        if self.trainer is None:
            run = {"lr": 3e-4, "min_lr": 3e-5, "warmup_steps": 10, "total_steps": 100000, "depth_mode": "cortex",
                   "grad_accum_steps": 1, "grad_clip": 1.0, "vocab_size": int(model.vocab_size), "batch_size": 4, "seq_len": 256}
            run.update(self.pending_training_config)
            run.update(cfg)
            if run.get("optimizer") or self.pending_training_config:
                from ..optim import build_optimizer

                opt = build_optimizer(model, {"optimizer": "centroid_steer", **run})
            else:
                opt = CentroidSteerOptimizer(model, lr=run["lr"], grad_clip=run["grad_clip"])
            src = SyntheticTokenSource(int(model.vocab_size), int(run["batch_size"]), int(run["seq_len"]), seed=0)
            self.trainer = Trainer(model, run, optimizer=opt, train_loader=src, device=self.device)
        else:
            self.trainer.config.update(cfg)
        return self.trainer

    def training_step(self, cfg: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        with self.lock:
            tr = self._ensure_trainer(cfg or {})
            t0 = time.perf_counter()
            out = tr.engine.step_once()
            loss = float(out["loss"])
            dt = time.perf_counter() - t0
            toks = int(tr.config.get("batch_size", 4)) * int(tr.config.get("seq_len", 256))
            self.train_status.update(step=tr.engine.step, loss=loss, tok_s=toks / max(dt, 1e-9))
            global_emitter.emit_loss_update(tr.engine.step, loss)
            self._broadcast({"type": "train", **{k: self.train_status[k] for k in ("step", "loss", "tok_s")}})
            return dict(self.train_status)

    def start_training(self, cfg: Optional[Dict[str, Any]] = None, max_steps: Optional[int] = None) -> Dict[str, Any]:
        if self._train_thread is not None and self._train_thread.is_alive():
            return dict(self.train_status)
        self._train_stop.clear()
        self.train_status.update(running=True, error=None)

        def loop():
            n = 0
            try:
                while not self._train_stop.is_set() and (max_steps is None or n < max_steps):
                    self.training_step(cfg if n == 0 else None)
                    n += 1
            except Exception as e:  # surfaced through /v1/training/status
                self.train_status["error"] = f"{type(e).__name__}: {e}"
            finally:
                self.train_status["running"] = False
                if self.model is not None:
                    self.model.eval()

        self._train_thread = threading.Thread(target=loop, name="triune-train", daemon=True)
        self._train_thread.start()
        return dict(self.train_status)

    def stop_training(self) -> Dict[str, Any]:
        self._train_stop.set()
        t = self._train_thread
        if t is not None and t.is_alive() and t is not threading.current_thread():
            t.join(timeout=60)
        self.train_status["running"] = False
        return dict(self.train_status)

    def save_checkpoint(self, directory: str = "checkpoints_full", name: str = "latest") -> str:
        from ..trainer import checkpoint as ckpt

        model = self.require_model()
        tr = self.trainer
        Path(directory).mkdir(parents=True, exist_ok=True)
        path = str(Path(directory) / f"{name}.pt")
        ckpt.save_checkpoint(path, model=model, optimizer=tr.optimizer if tr else None, step=tr.engine.step if tr else 0,
                             loss=float(self.train_status.get("loss") or 0.0), best_eval_loss=float("inf"), config=dict(self.config))
        return path

    def list_checkpoints(self, directory: str = "checkpoints_full") -> List[Dict[str, Any]]:
        d = Path(directory)
        if not d.is_dir():
            return []
        return [{"name": p.name, "path": str(p), "size_bytes": p.stat().st_size, "modified": p.stat().st_mtime}
                for p in sorted(d.glob("*.pt"), key=lambda p: -p.stat().st_mtime)]

    # ------------------------------------------------------------------ fine-tuning
    def start_finetune(self, records: List[Any], rank: int = 16, alpha: float = 32.0, epochs: int = 1, lr: float = 2e-4,
                       batch_size: int = 4, max_seq_len: int = 512, use_qlora: bool = False, output_dir: str = "adapters/latest",
                       max_steps: Optional[int] = None) -> Dict[str, Any]:
        from ..trainer.finetune import LoRAConfig, TriuneFineTuner

        model = self.require_model()
        if self.finetune_status["running"]:
            return dict(self.finetune_status)
        self._ft_cancel.clear()
        self.finetune_status.update(running=True, step=0, loss=None, error=None, adapter_dir=None)

        def run():
            try:
                ft = TriuneFineTuner(model, LoRAConfig(rank=rank, alpha=alpha, use_qlora=use_qlora, dropout=0.0), tokenizer=self.tokenizer)

                def cb(rec):
                    self.finetune_status.update(step=rec["step"], loss=rec["loss"])
                    self._broadcast({"type": "finetune", **rec})
                    if self._ft_cancel.is_set():
                        raise KeyboardInterrupt

                try:
                    ft.fit(records, epochs=epochs, batch_size=batch_size, lr=lr, max_seq_len=max_seq_len, max_steps=max_steps,
                           log_every=1, callback=cb)
                except KeyboardInterrupt:
                    pass
                self.finetune_status["adapter_dir"] = str(ft.save_adapter(output_dir))
                self._finetuner = ft
            except Exception as e:
                self.finetune_status["error"] = f"{type(e).__name__}: {e}"
            finally:
                self.finetune_status["running"] = False

        threading.Thread(target=run, name="triune-finetune", daemon=True).start()
        return dict(self.finetune_status)

    def cancel_finetune(self) -> None:
        self._ft_cancel.set()

    # ------------------------------------------------------------------ telemetry
    def _broadcast(self, payload: Dict[str, Any]) -> None:
        for fn in list(self.telemetry_listeners):
            try:
                fn(payload)
            except Exception:
                pass

    def diagnostics(self) -> Dict[str, Any]:
        from ..ops._c_bridge import get_native_c_info
        from ..runtime.capabilities import PrecisionCapabilities
        from ..runtime.vram import VRAMProfiler

        return {"device": str(self.device), "dtype": str(self.dtype), "model": dict(self.config) if self.model is not None else None,
                "capabilities": PrecisionCapabilities.detect(self.device).summary(), "native": get_native_c_info(),
                "vram": VRAMProfiler.get_vram_stats(self.device) if self.device.type == "cuda" else {"available": False},
                "sessions": self.srsm.stats(), "queue": self.queue.stats(), "training": dict(self.train_status)}


_STATE: Optional[EngineState] = None


def get_state() -> EngineState:
    global _STATE
    if _STATE is None:
        _STATE = EngineState()
    return _STATE


def reset_state(device: Optional[str] = None) -> EngineState:
    global _STATE
    _STATE = EngineState(device)
    return _STATE
