"""Checkpoint loading for inference and the text generation loop.

Parity: ``triune/inference.py:31-1051`` of the reference: ``load_checkpoint_model`` infers the architecture
from the state dict, ``load_model_for_inference`` resolves ``.pt`` checkpoints / presets, and
``generate_response`` does chunked prefill (1024 tokens) with the recurrent cache, top-k temperature sampling,
repetition (1.1) and count (0.35 per repeat) penalties, pad masking, stop strings, a streaming callback, a
cancel event, and time-to-first-token / decode-rate telemetry.

Differences: decoding keeps the GLA state on the device and advances it with the O(1) decode-step kernel; the
optional self-speculative path uses :class:`SelfSpeculativeGenerator`; sampling penalties are applied with
scatter ops (no per-token Python loops over the vocabulary).
"""

from __future__ import annotations

import re
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from .config import ModelConfig

DEFAULT_STOPS = ("\nUser:", "\nSystem:", "User:", "Assistant:")


def infer_config_from_state_dict(sd: Dict[str, torch.Tensor]) -> ModelConfig:
    """Recover the TriuneTransformer architecture from parameter shapes and key names."""
    sd = {k.replace("_orig_mod.", ""): v for k, v in sd.items()}
    V, d = sd["final_head.weight"].shape
    layers = 1 + max(int(m.group(1)) for k in sd for m in [re.match(r"layers\.(\d+)\.", k)] if m)
    exits = sorted({int(m.group(1)) for k in sd for m in [re.match(r"layers\.(\d+)\.exit_head\.weight", k)] if m})
    moe_layers = sorted({int(m.group(1)) for k in sd for m in [re.match(r"layers\.(\d+)\.ffn\.router\.weight", k)] if m})
    first_moe = moe_layers[0] if moe_layers else layers
    E = sd[f"layers.{first_moe}.ffn.router.weight"].shape[0] if moe_layers else 1
    expert_hidden = sd[f"layers.{first_moe}.ffn.experts.0.0.weight"].shape[0] if moe_layers else None
    dense_hidden = sd["layers.0.ffn.0.weight"].shape[0] if "layers.0.ffn.0.weight" in sd else None
    hd_total = sd["layers.0.attn.gla.q_proj.weight"].shape[0]
    head_dim = 64 if hd_total % 64 == 0 and (hd_total // 64) * 64 == d and d <= 2048 else 128
    if hd_total % head_dim != 0:
        head_dim = 64
    while hd_total % head_dim != 0 and head_dim > 1:  # narrow test models: the largest power of two that divides
        head_dim //= 2
    reflex = exits[0] if exits else max(1, first_moe - 1)
    limbic = exits[1] if len(exits) > 1 else min(layers - 2, reflex + 1)
    return ModelConfig(vocab_size=V, hidden_dim=d, num_layers=layers, num_heads=hd_total // head_dim, head_dim=head_dim,
                       num_experts=E, top_k=1, router_prefix_layers=max(1, min(3, reflex - 1)) if reflex > 1 else 1,
                       reflex_exit_layer=reflex, limbic_exit_layer=limbic, expert_hidden=expert_hidden,
                       dense_hidden=dense_hidden, shared_expert=f"layers.{first_moe}.ffn.shared.0.weight" in sd)


def load_checkpoint_model(path: str, device="cpu", dtype: Optional[torch.dtype] = None):
    """Load a ``.pt`` checkpoint (ours or the reference's) into a freshly built model. Returns (model, checkpoint)."""
    from .models.transformer import TriuneTransformer
    from .utils import place_model

    from .trainer.checkpoint import safe_torch_load

    ck = safe_torch_load(path)
    sd = ck.get("model_state", ck.get("model", ck)) if isinstance(ck, dict) else ck
    sd = {k.replace("_orig_mod.", ""): v for k, v in sd.items()}
    cfg_dict = ck.get("config") if isinstance(ck, dict) else None
    if isinstance(ck, dict) and ck.get("architecture") and not (cfg_dict and "hidden_dim" in cfg_dict):
        cfg_dict = {**ck["architecture"], **(cfg_dict or {})}
    cfg = None
    if cfg_dict and all(k in cfg_dict for k in ("hidden_dim", "num_layers", "num_heads")):
        try:
            cfg = ModelConfig.from_dict(cfg_dict).validate()
        except Exception:
            cfg = None
    if cfg is None:
        cfg = infer_config_from_state_dict(sd)
    if cfg_dict and "top_k" in cfg_dict:
        cfg.top_k = int(cfg_dict["top_k"])
    model = TriuneTransformer.from_config(cfg)
    model.load_state_dict(sd, strict=False)
    place_model(model, device, dtype)
    model.eval()
    return model, (ck if isinstance(ck, dict) else {})


def load_model_for_inference(spec: str, device="cpu", dtype: Optional[torch.dtype] = None):
    """``spec`` is a checkpoint path or a preset name (random-initialised)."""
    import os

    from .models.factory import build_model
    from .utils import place_model

    if os.path.exists(spec):
        return load_checkpoint_model(spec, device, dtype)[0]
    model = build_model(spec)
    place_model(model, device, dtype)
    return model.eval()


def _apply_penalties(logits: torch.Tensor, history: torch.Tensor, repetition_penalty: float, count_penalty: float):
    """logits [V]; history 1-D token ids. Repetition penalty divides positive / multiplies negative logits of seen
    tokens; the count penalty subtracts ``count_penalty * (count - 1)`` for tokens seen more than once."""
    if history.numel() == 0:
        return logits
    counts = torch.zeros_like(logits).scatter_add_(0, history, torch.ones_like(history, dtype=logits.dtype))
    seen = counts > 0
    if repetition_penalty and repetition_penalty != 1.0:
        pen = torch.where(logits > 0, logits / repetition_penalty, logits * repetition_penalty)
        logits = torch.where(seen, pen, logits)
    if count_penalty:
        logits = logits - count_penalty * (counts - 1).clamp_min(0)
    return logits


@torch.no_grad()
def generate_tokens(model, input_ids: torch.Tensor, max_new_tokens: int = 64, temperature: float = 0.7, top_k: int = 50,
                    repetition_penalty: float = 1.1, count_penalty: float = 0.35, eos_token_id: Optional[int] = None,
                    pad_token_id: Optional[int] = None, decode_depth: Optional[int] = 2, prefill_chunk: int = 1024,
                    cache: Optional[List[Any]] = None, on_token: Optional[Callable[[int], bool]] = None,
                    cancel_event: Optional[threading.Event] = None, generator: Optional[torch.Generator] = None
                    ) -> Tuple[List[int], List[Any], Dict[str, float]]:
    """Autoregressive generation for one sequence. Returns (new token ids, cache, telemetry)."""
    was = model.training
    model.eval()
    dev = input_ids.device
    t0 = time.perf_counter()
    if cache is None:
        cache = model.init_cache(1)
    logits = None
    for s in range(0, input_ids.shape[1], prefill_chunk):
        logits, cache = model(input_ids[:, s : s + prefill_chunk], force_depth=decode_depth, cache=cache,
                              last_token_only=True)
    ttft = None
    history = input_ids[0]
    out: List[int] = []
    t_dec = time.perf_counter()
    for _ in range(max_new_tokens):
        if cancel_event is not None and cancel_event.is_set():
            break
        lg = logits[0, -1].float()
        if pad_token_id is not None and 0 <= pad_token_id < lg.numel():
            lg[pad_token_id] = float("-inf")
        lg = _apply_penalties(lg, history, repetition_penalty, count_penalty)
        if temperature and temperature > 0:
            if top_k and top_k > 0:
                kth = torch.topk(lg, min(top_k, lg.numel())).values[-1]
                lg = lg.masked_fill(lg < kth, float("-inf"))
            tok = int(torch.multinomial(F.softmax(lg / temperature, -1), 1, generator=generator))
        else:
            tok = int(lg.argmax())
        if ttft is None:
            ttft = time.perf_counter() - t0
        out.append(tok)
        history = torch.cat((history, torch.tensor([tok], device=dev)))
        if on_token is not None and on_token(tok) is False:
            break
        if eos_token_id is not None and tok == eos_token_id:
            break
        logits, cache = model(torch.tensor([[tok]], device=dev), force_depth=decode_depth, cache=cache,
                              last_token_only=True)
    dt = max(1e-9, time.perf_counter() - t_dec)
    model.train(was)
    tele = {"ttft_s": ttft or 0.0, "decode_tok_s": len(out) / dt, "new_tokens": len(out),
            "prompt_tokens": int(input_ids.shape[1])}
    return out, cache, tele


class StreamingDecoder:
    """Incremental detokeniser that only emits text once it is stable (no partial multi-byte pieces)."""

    def __init__(self, tokenizer):
        self.tok = tokenizer
        self.ids: List[int] = []
        self.emitted = ""

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        text = self.tok.decode(self.ids)
        if text.endswith("�"):
            return ""
        delta = text[len(self.emitted):]
        self.emitted = text
        return delta


class IncrementalStreamingDecoder:
    """Detokeniser for streamed generation with the reference's interface (``triune/inference.py:714-745``): ``step``
    returns (text so far, newly stable text); pieces that end inside a multi-byte character are held back; the window of
    ids decoded together restarts at white space or after 16 ids so a long reply costs linear, not quadratic, time."""

    def __init__(self, tokenizer, skip_special_tokens: bool = True):
        self.tokenizer, self.skip_special_tokens = tokenizer, skip_special_tokens
        self.token_cache: List[int] = []
        self.print_len = 0
        self.cumulative_text = ""

    def _decode(self) -> str:
        try:
            return self.tokenizer.decode(self.token_cache, skip_special_tokens=self.skip_special_tokens)
        except TypeError:  # tokenizers of this framework take ids only
            return self.tokenizer.decode(self.token_cache)

    def step(self, token_id: int) -> Tuple[str, str]:
        self.token_cache.append(int(token_id))
        text = self._decode()
        if text.endswith("\ufffd"):
            return self.cumulative_text, ""
        delta = text[self.print_len:]
        self.cumulative_text += delta
        if text.endswith((" ", "\n")) or len(self.token_cache) >= 16:
            self.token_cache, self.print_len = [], 0
        else:
            self.print_len = len(text)
        return self.cumulative_text, delta

    def flush(self) -> Tuple[str, str]:
        delta = ""
        if self.token_cache:
            text = self._decode()
            delta = text[self.print_len:]
            self.cumulative_text += delta
            self.token_cache, self.print_len = [], 0
        return self.cumulative_text, delta


def optimize_hf_model_for_inference(model: torch.nn.Module) -> torch.nn.Module:
    """Route the RMSNorm modules of a Hugging Face model through this framework's fused kernel while no gradient is being
    recorded and the module is in eval mode; training keeps the model's own forward. Gemma-family norms, whose weight is
    an offset from one, are handled. Models under layer streaming are left alone (their weights move between calls).
    Reference: ``triune/inference.py:31-110``."""
    from . import ops

    if getattr(model, "_streaming_engine", None) is not None or getattr(model, "_layer_streaming_active", False):
        return model
    for mod in model.modules():
        name = type(mod).__name__.lower()
        w = getattr(mod, "weight", None)
        if getattr(mod, "_triune_rms_fused", False) or "rmsnorm" not in name or not isinstance(w, torch.Tensor):
            continue
        if w.dim() != 1 or w.numel() == 0 or w.device.type == "meta":
            continue
        eps = float(getattr(mod, "eps", getattr(mod, "variance_epsilon", 1e-6)))
        offset = 1.0 if "gemma" in name else 0.0

        def fused(x, _m=mod, _orig=mod.forward, _eps=eps, _off=offset):
            if torch.is_grad_enabled() or _m.training:
                return _orig(x)
            wt = _m.weight if _off == 0.0 else (_off + _m.weight.float())
            return ops.rmsnorm(x, wt.to(device=x.device, dtype=x.dtype), _eps)

        mod.forward = fused
        mod._triune_rms_fused = True
    return model


def release_cuda_graph_runner(model) -> None:
    """Drop the captured decode graph (and its static cache) that a graphed decoder left on ``model``
    (``triune/inference.py:304-317`` of the reference)."""
    if model is None:
        return
    for attr in ("_triune_cg_runner", "_graphed_decoder"):
        runner = getattr(model, attr, None)
        if runner is None:
            continue
        for meth in ("release", "reset"):
            fn = getattr(runner, meth, None)
            if callable(fn):
                try:
                    fn()
                except Exception:
                    pass
                break
        try:
            delattr(model, attr)
        except AttributeError:
            setattr(model, attr, None)


def generate_response(model, tokenizer, prompt: str, max_new_tokens: int = 256, temperature: float = 0.7, top_k: int = 50,
                      repetition_penalty: float = 1.1, decode_depth: Optional[int] = 2, stop: Tuple[str, ...] = DEFAULT_STOPS,
                      stream_callback: Optional[Callable[[str], None]] = None, cancel_event: Optional[threading.Event] = None,
                      cache: Optional[List[Any]] = None, template: bool = True, device=None, speculative: bool = False,
                      k_draft: int = 3, eos_token_id: Optional[int] = None, pad_token_id: Optional[int] = None) -> Dict[str, Any]:
    """Chat-style generation. Returns {"text", "tokens", "telemetry", "cache"}. ``eos_token_id`` / ``pad_token_id`` override
    what the tokenizer names."""
    dev = torch.device(device) if device is not None else next(model.parameters()).device
    text_in = f"User: {prompt}\nAssistant:" if template else prompt
    ids = torch.tensor([tokenizer.encode(text_in)], device=dev, dtype=torch.long)
    max_new_tokens = min(int(max_new_tokens), 8192)
    eos = eos_token_id if eos_token_id is not None else getattr(tokenizer, "sep_token_id", getattr(tokenizer, "eos_token_id", None))
    pad = pad_token_id if pad_token_id is not None else getattr(tokenizer, "pad_token_id", None)
    if speculative and temperature <= 0:
        from .models.speculative import SelfSpeculativeGenerator

        gen = SelfSpeculativeGenerator(model, tokenizer, k_draft=k_draft, eos_token_id=eos, pad_token_id=pad)
        t0 = time.perf_counter()
        full = gen.generate(ids, max_new_tokens, temperature=0.0)
        toks = full[0, ids.shape[1]:].tolist()
        text = tokenizer.decode(toks)
        tele = dict(gen.telemetry, decode_tok_s=len(toks) / max(1e-9, time.perf_counter() - t0),
                    acceptance_rate=gen.acceptance_rate)
        return {"text": _cut_at_stop(text, stop), "tokens": toks, "telemetry": tele, "cache": None}
    decoder = StreamingDecoder(tokenizer)
    state = {"text": "", "stopped": False}

    def on_token(tok: int) -> bool:
        delta = decoder.push(tok)
        state["text"] += delta
        for s in stop:
            if s and s in state["text"]:
                state["stopped"] = True
                return False
        if delta and stream_callback is not None:
            stream_callback(delta)
        return True

    toks, cache, tele = generate_tokens(model, ids, max_new_tokens, temperature, top_k, repetition_penalty, 0.35, eos, pad,
                                        decode_depth, 1024, cache, on_token, cancel_event)
    return {"text": _cut_at_stop(state["text"], stop), "tokens": toks, "telemetry": tele, "cache": cache}


def _cut_at_stop(text: str, stop: Tuple[str, ...]) -> str:
    cut = len(text)
    for s in stop:
        if s:
            i = text.find(s)
            if i >= 0:
                cut = min(cut, i)
    return text[:cut].strip()


class GraphedGreedyDecoder:
    """Greedy decoding with the whole per-token step (all layers, exit head, arg-max, state update) captured in ONE
    CUDA graph and replayed once per token, with no host synchronisation until the requested tokens are done.

    A decode step of a small model is a few hundred kernel launches of a few microseconds each: run eagerly it is bound
    by launch latency and Python, not by the GPU. Everything that changes between steps lives in device memory: the
    current token, the position (RoPE rows are gathered by a device index), the recurrent states (updated in place) and
    the output buffer. On a CPU device the same step function runs eagerly, which is what the tests compare against.
    """

    def __init__(self, model, batch_size: int = 1, decode_depth: Optional[int] = 2, max_positions: int = 32768):
        self.model, self.B, self.depth = model, batch_size, decode_depth
        self.device = next(model.parameters()).device
        self.max_positions = max_positions
        self.graph = None
        self.states: List[Optional[torch.Tensor]] = []
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)
        self.step_idx = torch.zeros(1, dtype=torch.long, device=self.device)
        self.token = torch.zeros(batch_size, 1, dtype=torch.long, device=self.device)
        self.out: Optional[torch.Tensor] = None

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, prefill_chunk: int = 4096) -> torch.Tensor:
        """Runs the prompt, loads the static state buffers, returns the first generated token [B, 1]."""
        m = self.model
        m.eval()
        cache = m.init_cache(self.B)
        logits = None
        for s in range(0, input_ids.shape[1], prefill_chunk):
            logits, cache = m(input_ids[:, s : s + prefill_chunk], force_depth=self.depth, cache=cache, last_token_only=True)
        # make sure every rotary table covers the positions the graph will index
        for mod in m.modules():
            if hasattr(mod, "_build") and hasattr(mod, "head_dim") and hasattr(mod, "_cos"):
                mod(1, self.device, offset=min(self.max_positions, max(mod.max_seq_len, input_ids.shape[1] + 1)) - 1)
        new_states = [c[0] if isinstance(c, tuple) else None for c in cache]
        if len(self.states) == len(new_states) and all((a is None) == (b is None) for a, b in zip(self.states, new_states)):
            for a, b in zip(self.states, new_states):
                if a is not None:
                    a.copy_(b)
        else:
            self.states = [None if s is None else s.clone() for s in new_states]
            self.graph = None
        self.pos.fill_(input_ids.shape[1])
        self.token.copy_(logits[:, -1].argmax(-1, keepdim=True))
        return self.token.clone()

    def _step(self):
        cache = [(s, self.pos) if s is not None else (None, self.pos) for s in self.states]
        logits, new_cache = self.model(self.token, force_depth=self.depth, cache=cache, last_token_only=True)
        for s, c in zip(self.states, new_cache):
            if s is not None and isinstance(c, tuple) and c[0] is not None:
                s.copy_(c[0])
        self.out.index_copy_(1, self.step_idx, self.token)
        self.token.copy_(logits[:, -1].argmax(-1, keepdim=True))
        self.pos.add_(1)
        self.step_idx.add_(1)

    @torch.no_grad()
    def decode(self, max_new_tokens: int) -> torch.Tensor:
        """-> [B, max_new_tokens] token ids (the first one is the token ``prefill`` returned)."""
        if self.out is None or self.out.shape[1] < max_new_tokens:
            self.out = torch.zeros(self.B, max_new_tokens, dtype=torch.long, device=self.device)
            self.graph = None
        self.step_idx.zero_()
        if self.device.type != "cuda":
            for _ in range(max_new_tokens):
                self._step()
            return self.out[:, :max_new_tokens].clone()
        if self.graph is None:
            # snapshot, warm up on a side stream (allocator and autotune effects must not land in the capture), restore
            snap = ([None if s is None else s.clone() for s in self.states], self.pos.clone(), self.token.clone())
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step()
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step()
            self.graph = g
            for s, b in zip(self.states, snap[0]):
                if s is not None:
                    s.copy_(b)
            self.pos.copy_(snap[1])
            self.token.copy_(snap[2])
            self.step_idx.zero_()
        for _ in range(max_new_tokens):
            self.graph.replay()
        return self.out[:, :max_new_tokens].clone()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        self.prefill(input_ids)
        return torch.cat((input_ids, self.decode(max_new_tokens)), dim=1)


class GraphedSpeculativeDecoder:
    """Greedy self-speculative decoding with one whole ROUND captured in a CUDA graph: the Reflex exit drafts ``k``
    tokens (k single-token steps through the first layers), the full depth verifies all of them plus the current token in
    ONE batched pass, and the longest agreeing prefix plus one corrected token are committed, all without a host
    synchronisation. The output equals plain greedy decoding at full depth token for token.

    Parity: ``SelfSpeculativeGenerator`` (``triune/model/speculative.py:45-280`` of the reference), which runs the same
    scheme from Python with cloned caches. What differs here: the acceptance count stays on the device (an index into
    the per-token states the mixers return, see ``VectorisedGLA.forward_token_states``), every candidate token of a round
    is written to the output buffer and the write position advances by the accepted count, so a round has the same
    launches whatever it accepts and can be replayed. Batch size 1, recurrent (GLA / Gated DeltaNet) mixers.
    """

    def __init__(self, model, k_draft: int = 3, max_positions: int = 32768):
        self.model, self.k = model, int(k_draft)
        self.device = next(model.parameters()).device
        self.max_positions = max_positions
        self.draft_depth = 0
        self.n_draft_layers = model.exit_layers[0] + 1
        self.n_layers = model.exit_layers[2] + 1
        for blk in model.layers[: self.n_layers]:
            if getattr(blk.attn, "gla", None) is None:
                raise NotImplementedError("graphed speculative decoding covers the recurrent mixers")
        dev = self.device
        self.states: List[torch.Tensor] = []
        self.draft_states: List[torch.Tensor] = []
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.draft_pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.token = torch.zeros(1, 1, dtype=torch.long, device=dev)
        self.step_idx = torch.zeros(1, dtype=torch.long, device=dev)
        self.cand = torch.zeros(1, self.k + 1, dtype=torch.long, device=dev)   # [current token, drafts]
        self.accepted = torch.zeros(1, dtype=torch.long, device=dev)           # drafted tokens accepted, all rounds
        self.rounds = torch.zeros(1, dtype=torch.long, device=dev)
        self.out: Optional[torch.Tensor] = None
        self.graph = None
        self._ar = torch.arange(self.k + 1, device=dev)

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, prefill_chunk: int = 4096) -> torch.Tensor:
        m = self.model
        m.eval()
        assert input_ids.shape[0] == 1, "speculative decoding runs one sequence"
        cache = m.init_cache(1)
        logits = None
        for s in range(0, input_ids.shape[1], prefill_chunk):
            logits, cache = m(input_ids[:, s : s + prefill_chunk], force_depth=2, cache=cache, last_token_only=True)
        for mod in m.modules():
            if hasattr(mod, "_build") and hasattr(mod, "head_dim") and hasattr(mod, "_cos"):
                mod(1, self.device, offset=min(self.max_positions, max(mod.max_seq_len, input_ids.shape[1] + 1)) - 1)
        new_states = [c[0] for c in cache[: self.n_layers]]
        if len(self.states) == len(new_states):
            for a, b in zip(self.states, new_states):
                a.copy_(b)
        else:
            self.states = [s.clone() for s in new_states]
            self.draft_states = [s.clone() for s in new_states[: self.n_draft_layers]]
            self.graph = None
        self.pos.fill_(input_ids.shape[1])
        self.token.copy_(logits[:, -1].argmax(-1, keepdim=True))
        self.accepted.zero_()
        self.rounds.zero_()
        return self.token.clone()

    # ------------------------------------------------------------------ one round
    def _draft(self):
        m = self.model
        for a, b in zip(self.draft_states, self.states):
            a.copy_(b)
        self.draft_pos.copy_(self.pos)
        self.cand[:, 0:1].copy_(self.token)
        for i in range(self.k):
            cache = [(s, self.draft_pos) for s in self.draft_states] + [(None, self.draft_pos)] * (len(m.layers) - self.n_draft_layers)
            logits, new_cache = m(self.cand[:, i : i + 1], force_depth=self.draft_depth, cache=cache, last_token_only=True)
            for s, c in zip(self.draft_states, new_cache):
                s.copy_(c[0])
            self.cand[:, i + 1 : i + 2].copy_(logits[:, -1].argmax(-1, keepdim=True))
            self.draft_pos.add_(1)

    def _verify(self):
        """All k + 1 candidate tokens through the full depth in one pass -> (greedy targets [1, k+1], per-layer states
        after each token)."""
        from . import ops

        m = self.model
        x = ops.embedding(self.cand, m.token_embed.weight)
        per_layer = []
        for i in range(self.n_layers):
            blk = m.layers[i]
            y, sts = blk.attn.gla.forward_token_states(blk.norm1(x), self.states[i], self.pos)
            n2, x = blk.norm2.forward_add(y, x)
            x = x + blk._ffn(n2, False)
            per_layer.append(sts)
        logits = m._head(x, 2, False)
        return logits.argmax(-1), per_layer

    def _round(self):
        self._draft()
        targets, per_layer = self._verify()                       # targets[:, i] follows cand[:, i]
        k = self.k
        agree = (self.cand[:, 1:] == targets[:, :k]).to(torch.long)
        n = torch.cumprod(agree, dim=1).sum(dim=1)                # [1]: drafted tokens accepted
        # every candidate output of the round goes to the buffer; only n + 1 of them are kept by the index advance
        idx = (self.step_idx + self._ar).clamp_(max=self.out.shape[1] - 1)
        self.out.index_copy_(1, idx, targets)
        for s, sts in zip(self.states, per_layer):
            s.copy_(sts.index_select(0, n).squeeze(0))             # state after the last accepted token
        self.token.copy_(targets.gather(1, n.view(1, 1)))
        self.pos.add_(n + 1)
        self.step_idx.add_(n + 1)
        self.accepted.add_(n)
        self.rounds.add_(1)

    # ------------------------------------------------------------------ decoding
    @torch.no_grad()
    def decode(self, max_new_tokens: int, rounds_per_check: int = 8) -> torch.Tensor:
        """-> [1, max_new_tokens]; the first token is the one ``prefill`` returned."""
        need = max_new_tokens + self.k + 2
        if self.out is None or self.out.shape[1] < need:
            self.out = torch.zeros(1, need, dtype=torch.long, device=self.device)
            self.graph = None
        self.step_idx.fill_(1)
        self.out[:, 0:1].copy_(self.token)
        cuda = self.device.type == "cuda"
        if cuda and self.graph is None:
            snap = ([s.clone() for s in self.states], self.pos.clone(), self.token.clone(), self.out.clone())
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._round()
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._round()
            self.graph = g
            for s, b in zip(self.states, snap[0]):
                s.copy_(b)
            self.pos.copy_(snap[1])
            self.token.copy_(snap[2])
            self.out.copy_(snap[3])
            self.step_idx.fill_(1)
            self.accepted.zero_()
            self.rounds.zero_()
        while True:
            for _ in range(rounds_per_check):
                if cuda:
                    self.graph.replay()
                else:
                    self._round()
            if int(self.step_idx.item()) >= max_new_tokens:  # one host read per `rounds_per_check` rounds
                break
        return self.out[:, :max_new_tokens].clone()

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int) -> torch.Tensor:
        self.prefill(input_ids)
        return torch.cat((input_ids, self.decode(max_new_tokens)), dim=1)

    @property
    def acceptance_rate(self) -> float:
        r = int(self.rounds.item())
        return float(self.accepted.item()) / max(1, r * self.k)
