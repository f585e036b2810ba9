"""Hugging Face -> Triune conversion.

Parity (``triune/model/transmuter.py:86-675``):
  * ``transmute_hf_to_triune``           keep the HF network, attach the three-tier exits (``attach_early_exits``);
  * ``transfer_weights_to_native_triune`` build a native ``TriuneTransformer`` and initialise it from the teacher:
    embeddings / untied head, final norm, per-layer norms, Q/K/V/O (GQA key/value heads expanded to the query head
    count, the decay-gate projection seeded from 0.1 * K), dense FFN and MoE experts upcycled from the teacher MLP
    (SwiGLU teachers: mean of gate and up), each expert perturbed by a 1e-3 factor so the router can break symmetry;
    matrices of a different shape are cropped / zero-padded;
  * ``distill_native_triune_step``       KL distillation of all three exits against the teacher;
  * ``ollama_to_hf_candidate``           Ollama tag -> HF repo id.

Here the student stores Q,K,V,G as one fused ``[4*H*D, d]`` parameter and experts as stacked ``[E, h, d]`` tensors, so the
surgery writes into slices of those parameters.
"""

from __future__ import annotations

import re
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig
from .adapters import attach_early_exits

_OLLAMA_HF = {
    "gemma3:1b": "google/gemma-3-1b-it", "gemma3:4b": "google/gemma-3-4b-it", "gemma3:12b": "google/gemma-3-12b-it",
    "gemma2:2b": "google/gemma-2-2b-it", "gemma2:9b": "google/gemma-2-9b-it",
    "llama3.2:1b": "meta-llama/Llama-3.2-1B-Instruct", "llama3.2:3b": "meta-llama/Llama-3.2-3B-Instruct",
    "llama3.1:8b": "meta-llama/Llama-3.1-8B-Instruct", "llama3:8b": "meta-llama/Meta-Llama-3-8B-Instruct",
    "qwen2.5:0.5b": "Qwen/Qwen2.5-0.5B-Instruct", "qwen2.5:1.5b": "Qwen/Qwen2.5-1.5B-Instruct",
    "qwen2.5:3b": "Qwen/Qwen2.5-3B-Instruct", "qwen2.5:7b": "Qwen/Qwen2.5-7B-Instruct",
    "qwen3:0.6b": "Qwen/Qwen3-0.6B", "qwen3:1.7b": "Qwen/Qwen3-1.7B", "qwen3:4b": "Qwen/Qwen3-4B", "qwen3:8b": "Qwen/Qwen3-8B",
    "mistral:7b": "mistralai/Mistral-7B-Instruct-v0.3", "phi3:mini": "microsoft/Phi-3-mini-4k-instruct",
    "phi4-mini:3.8b": "microsoft/Phi-4-mini-instruct", "smollm2:1.7b": "HuggingFaceTB/SmolLM2-1.7B-Instruct",
    "tinyllama:1.1b": "TinyLlama/TinyLlama-1.1B-Chat-v1.0",
}


def ollama_to_hf_candidate(name: str) -> Optional[str]:
    if not name:
        return None
    s = str(name).strip()
    if s.lower().startswith("ollama:"):
        s = s[7:].strip()
    if "/" in s and ":" not in s:
        return s  # already an org/repo id or a path
    key = s.lower()
    if key in _OLLAMA_HF:
        return _OLLAMA_HF[key]
    base, _, tag = key.partition(":")
    m = re.match(r"^([0-9]+(?:\.[0-9]+)?[bm])", tag or "")
    if base and m and f"{base}:{m.group(1)}" in _OLLAMA_HF:  # "gemma3:4b-instruct-q4_K_M" -> "gemma3:4b"
        return _OLLAMA_HF[f"{base}:{m.group(1)}"]
    if not tag or tag == "latest":
        for t in ("4b", "7b", "8b", "3b", "1.7b", "mini"):
            if f"{base}:{t}" in _OLLAMA_HF:
                return _OLLAMA_HF[f"{base}:{t}"]
    return None


def resolve_hf_backbone(hf_model: nn.Module):
    """(embed_tokens, lm_head, layers, final_norm, text_config, attach_target) for Llama/Qwen/Mistral/Gemma/GPT-2/
    GPT-NeoX layouts and multimodal wrappers that nest the text model under ``language_model``."""
    cfg = getattr(hf_model, "config", None)
    text_cfg = getattr(cfg, "text_config", cfg)
    head = getattr(hf_model, "lm_head", None) or getattr(hf_model, "embed_out", None)
    inner = getattr(hf_model, "model", None) or getattr(hf_model, "transformer", None) or getattr(hf_model, "gpt_neox", None)
    target = hf_model
    lang = getattr(hf_model, "language_model", None)
    if lang is not None and not hasattr(inner, "layers"):
        target, inner = lang, getattr(lang, "model", lang)
        head = head or getattr(lang, "lm_head", None)
    inner = inner if inner is not None else hf_model
    emb = next((getattr(inner, n) for n in ("embed_tokens", "wte", "embed_in") if getattr(inner, n, None) is not None), None)
    if emb is None and hasattr(hf_model, "get_input_embeddings"):
        emb = hf_model.get_input_embeddings()
    if head is None and hasattr(hf_model, "get_output_embeddings"):
        head = hf_model.get_output_embeddings()
    layers = next((getattr(inner, n) for n in ("layers", "h", "blocks") if getattr(inner, n, None) is not None), None)
    norm = next((getattr(inner, n) for n in ("norm", "ln_f", "final_layer_norm") if getattr(inner, n, None) is not None), None)
    return emb, head, layers, norm, text_cfg, target


def compute_tier_indices(num_layers: int, reflex_ratio: float = 0.25) -> Tuple[int, int]:
    n = max(3, int(num_layers))
    reflex = max(1, min(n - 2, int(round(n * max(0.15, min(0.45, float(reflex_ratio)))))))
    limbic = max(reflex + 1, min(n - 1, int(round(n * 0.60))))
    return reflex, limbic


def transmute_hf_to_triune(model_or_source, *, reflex_ratio: float = 0.25, rank: int = 64, use_jev: bool = True,
                           jev_threshold: float = 0.85, device=None, local_files_only: bool = True):
    """Attach reflex/limbic exits to an HF causal LM (an instance, or a path / repo id to load). Returns
    ``(model, metadata)``."""
    if isinstance(model_or_source, nn.Module):
        model = model_or_source
    else:
        from transformers import AutoModelForCausalLM

        src = ollama_to_hf_candidate(str(model_or_source)) or str(model_or_source)
        model = AutoModelForCausalLM.from_pretrained(src, local_files_only=local_files_only)
    if device is not None:
        model = model.to(device)
    _, head, layers, _, text_cfg, target = resolve_hf_backbone(model)
    n = len(layers) if layers is not None else int(getattr(text_cfg, "num_hidden_layers", 12))
    r_idx, l_idx = compute_tier_indices(n, reflex_ratio)
    if isinstance(getattr(target, "lm_head", None), nn.Linear) or isinstance(getattr(target, "final_head", None), nn.Linear):
        attach_early_exits(target, reflex_layer=r_idx, limbic_layer=l_idx, rank=rank, use_jev=use_jev, jev_threshold=jev_threshold)
    else:
        raise ValueError("the model exposes no linear LM head to tie the exit projections to")
    if target is not model:
        for a in ("reflex_head", "limbic_head", "reflex_layer_idx", "limbic_layer_idx", "_exit_manager", "reflex_jev_router",
                  "limbic_jev_router", "use_jev", "generate_adaptive"):
            if hasattr(target, a):
                setattr(model, a, getattr(target, a))
    model._is_triune_transmuted, model._exits_calibrated = True, False
    model.reflex_exit_layer, model.limbic_exit_layer = r_idx, l_idx
    meta = {"weights_transferred": True, "transmute_mode": "early_exit", "reflex_exit_layer": r_idx,
            "limbic_exit_layer": l_idx, "num_layers": n, "use_jev": bool(use_jev)}
    return model, meta


# ------------------------------------------------------------------------------------------------ weight surgery
def _copy_fit(dst: torch.Tensor, src: torch.Tensor) -> int:
    """Copy ``src`` into ``dst``; different shapes are cropped / zero-padded. Returns the number of elements copied."""
    with torch.no_grad():
        s = src.detach().to(device=dst.device, dtype=dst.dtype)
        if s.shape == dst.shape:
            dst.copy_(s)
            return dst.numel()
        dst.zero_()
        if s.ndim == 1:
            n = min(dst.shape[0], s.shape[0])
            dst[:n].copy_(s[:n])
            return n
        r, c = min(dst.shape[0], s.shape[0]), min(dst.shape[1], s.shape[1])
        dst[:r, :c].copy_(s[:r, :c])
        return r * c


def expand_gqa_weight(w: torch.Tensor, q_heads: int, kv_heads: int) -> torch.Tensor:
    """[kv_heads*hd, d] -> [q_heads*hd, d] by repeating each key/value head for its query group."""
    if kv_heads <= 0 or q_heads <= 0 or kv_heads == q_heads or q_heads % kv_heads or w.shape[0] % kv_heads:
        return w
    hd = w.shape[0] // kv_heads
    return w.view(kv_heads, hd, w.shape[1]).repeat_interleave(q_heads // kv_heads, dim=0).reshape(q_heads * hd, w.shape[1])


def _w(mod) -> Optional[torch.Tensor]:
    w = getattr(mod, "weight", None) if mod is not None else None
    if w is None or w.device.type == "meta" or not w.dtype.is_floating_point:
        return None  # missing, not materialised, or packed integer storage
    return w


def _first(obj, *names):
    for n in names:
        v = getattr(obj, n, None) if obj is not None else None
        if v is not None:
            return v
    return None


def _teacher_parts(layer):
    attn = _first(layer, "self_attn", "attention", "attn")
    mlp = _first(layer, "mlp", "feed_forward")
    return dict(norm1=_first(layer, "input_layernorm", "ln_1"), norm2=_first(layer, "post_attention_layernorm", "ln_2"),
                q=_first(attn, "q_proj"), k=_first(attn, "k_proj"), v=_first(attn, "v_proj"), o=_first(attn, "o_proj", "out_proj"),
                gate=_first(mlp, "gate_proj"), up=_first(mlp, "up_proj", "c_fc", "fc_in", "dense_h_to_4h"),
                down=_first(mlp, "down_proj", "c_proj", "fc_out", "dense_4h_to_h"))


def transfer_weights_to_native_triune(hf_model: nn.Module, tokenizer: Any = None, *, reflex_ratio: float = 0.25,
                                      num_experts: int = 8, top_k: int = 2, shared_expert: bool = True,
                                      target_dim: Optional[int] = None, target_layers: Optional[int] = None):
    """Returns ``(student TriuneTransformer, report)``."""
    from .transformer import TriuneTransformer

    emb, head, t_layers, t_norm, tcfg, _ = resolve_hf_backbone(hf_model)
    if t_layers is None or len(t_layers) == 0:
        raise ValueError("the source model exposes no transformer layers")
    t_dim = int(getattr(tcfg, "hidden_size", emb.weight.shape[1] if emb is not None else 768))
    t_vocab = int(getattr(tcfg, "vocab_size", emb.weight.shape[0] if emb is not None else 32000))
    t_heads = int(getattr(tcfg, "num_attention_heads", 0) or max(1, t_dim // 64))
    t_kv = int(getattr(tcfg, "num_key_value_heads", 0) or t_heads)
    s_dim = int(target_dim or t_dim)
    hd = next((c for c in (64, 128, 32, 16) if s_dim % c == 0), max(16, s_dim // max(1, t_heads)))
    heads = max(1, s_dim // hd)
    s_dim = heads * hd
    L = max(4, int(target_layers or len(t_layers)))
    reflex, limbic = compute_tier_indices(L, reflex_ratio)
    reflex = max(reflex, 2)
    limbic = max(limbic, reflex + 1)
    if limbic >= L:
        limbic, reflex = L - 1, min(reflex, L - 2)
    cfg = ModelConfig(vocab_size=t_vocab, hidden_dim=s_dim, num_layers=L, num_heads=heads, head_dim=hd,
                      num_experts=max(1, int(num_experts)), top_k=max(1, min(int(top_k), int(num_experts))),
                      shared_expert=bool(shared_expert), router_prefix_layers=1, reflex_exit_layer=reflex,
                      limbic_exit_layer=limbic)
    student = TriuneTransformer.from_config(cfg)
    ref = next((p for p in hf_model.parameters() if p.device.type != "meta" and p.dtype.is_floating_point), None)
    if ref is not None:
        student = student.to(device=ref.device, dtype=ref.dtype)
    stats = {"tensors": 0, "params": 0}

    def rec(n: int):
        if n > 0:
            stats["tensors"] += 1
            stats["params"] += int(n)

    emb_w, head_w = _w(emb), _w(head)
    if emb_w is not None:
        rec(_copy_fit(student.token_embed.weight, emb_w))
    head_bias = getattr(head, "bias", None) if head is not None else None
    untied = False
    if head_w is not None:
        tied = emb_w is not None and head_bias is None and (head_w.data_ptr() == emb_w.data_ptr() or (
            head_w.shape == emb_w.shape and torch.allclose(head_w.float(), emb_w.float(), atol=1e-6, rtol=1e-5)))
        if not tied:
            new_head = nn.Linear(s_dim, t_vocab, bias=head_bias is not None, device=student.token_embed.weight.device,
                                 dtype=student.token_embed.weight.dtype)
            rec(_copy_fit(new_head.weight, head_w))
            if head_bias is not None:
                rec(_copy_fit(new_head.bias, head_bias))
            student.final_head = new_head
            untied = True
    norm_w = _w(t_norm)
    if norm_w is not None:
        rec(_copy_fit(student.final_norm.weight, norm_w))
    HD = heads * hd
    for si, blk in enumerate(student.layers):
        ti = min(len(t_layers) - 1, int(round(si * (len(t_layers) - 1) / max(1, L - 1))))
        t = _teacher_parts(t_layers[ti])
        for dst, src in ((blk.norm1, t["norm1"]), (blk.norm2, t["norm2"])):
            if _w(src) is not None:
                rec(_copy_fit(dst.weight, _w(src)))
        gla = blk.attn.gla
        if gla is not None:
            fused = gla.qkvg_weight.data  # rows: [q | k | v | g], each H*D
            if _w(t["q"]) is not None:
                rec(_copy_fit(fused[0:HD], _w(t["q"])))
            if _w(t["k"]) is not None:
                k = expand_gqa_weight(_w(t["k"]), t_heads, t_kv)
                rec(_copy_fit(fused[HD : 2 * HD], k))
                rec(_copy_fit(fused[3 * HD : 4 * HD], k * 0.1))  # mild, input-dependent decay to start from
            if _w(t["v"]) is not None:
                rec(_copy_fit(fused[2 * HD : 3 * HD], expand_gqa_weight(_w(t["v"]), t_heads, t_kv)))
            if _w(t["o"]) is not None:
                rec(_copy_fit(gla.out_proj.weight, _w(t["o"])))
        gate, up, down = _w(t["gate"]), _w(t["up"]), _w(t["down"])
        if up is not None and getattr(t["up"], "__class__", None).__name__ == "Conv1D":
            up, down = up.t(), (down.t() if down is not None else None)  # GPT-2 stores [in, out]
        fc1 = 0.5 * (gate + up) if gate is not None and up is not None and gate.shape == up.shape else up
        ffn = blk.ffn
        if hasattr(ffn, "w1"):  # stacked MoE experts
            if ffn.shared is not None:
                if fc1 is not None:
                    rec(_copy_fit(ffn.shared[0].weight, fc1))
                if down is not None:
                    rec(_copy_fit(ffn.shared[2].weight, down))
            E = ffn.num_experts
            for e in range(E):
                f = 1.0 + (e - (E - 1) / 2.0) * 1e-3
                if fc1 is not None:
                    rec(_copy_fit(ffn.w1.data[e], fc1 * f))
                if down is not None:
                    rec(_copy_fit(ffn.w2.data[e], down / f))
        else:
            if fc1 is not None:
                rec(_copy_fit(ffn[0].weight, fc1))
            if down is not None:
                rec(_copy_fit(ffn[2].weight, down))
        if blk.exit_norm is not None and norm_w is not None:
            rec(_copy_fit(blk.exit_norm.weight, norm_w))
    if tokenizer is not None:
        student.tokenizer = tokenizer
    student._exits_calibrated = False
    total = sum(p.numel() for p in student.parameters())
    report = {"weights_transferred": stats["tensors"] > 0, "transmute_mode": "native_distill",
              "transferred_tensors": stats["tensors"], "transferred_params": stats["params"], "total_student_params": total,
              "coverage_ratio": round(min(1.0, stats["params"] / max(1, total)), 4), "lm_head_transferred": head_w is not None,
              "lm_head_untied": untied, "exits_calibrated": False, "teacher_layers": len(t_layers), "student_layers": L,
              "teacher_dim": t_dim, "student_dim": s_dim, "reflex_exit_layer": reflex, "limbic_exit_layer": limbic,
              "needs_distillation": True}
    return student, report


def distill_native_triune_step(student, teacher: nn.Module, input_ids: torch.Tensor, optimizer, *, temperature: float = 2.0,
                               ce_weight: float = 0.1, reflex_weight: float = 0.25, limbic_weight: float = 0.35
                               ) -> Dict[str, float]:
    """One KL step aligning the three exits with the teacher's next-token distribution (+ a small CE term)."""
    student.train()
    teacher.eval()
    temp = max(0.1, float(temperature))
    with torch.no_grad():
        try:
            out = teacher(input_ids=input_ids, use_cache=False)
        except TypeError:
            out = teacher(input_ids)
        t_logits = out.logits if hasattr(out, "logits") else (out[0] if isinstance(out, tuple) else out)
        target = F.softmax(t_logits.float() / temp, dim=-1)
    optimizer.zero_grad(set_to_none=True)
    reflex, limbic, cortex, _ = student.forward_all_exits(input_ids)  # one pass through the trunk for all three exits

    def kl(s_logits):
        v = min(s_logits.size(-1), target.size(-1))
        q = target[..., :v].reshape(-1, v)
        if v < target.size(-1):
            q = q / q.sum(-1, keepdim=True).clamp_min(1e-12)
        return F.kl_div(F.log_softmax(s_logits[..., :v].float() / temp, -1).reshape(-1, v), q, reduction="batchmean") * temp * temp

    losses = {"cortex_kl": kl(cortex), "limbic_kl": kl(limbic), "reflex_kl": kl(reflex)}
    total = losses["cortex_kl"] + limbic_weight * losses["limbic_kl"] + reflex_weight * losses["reflex_kl"]
    if ce_weight > 0 and input_ids.size(1) > 1:
        losses["ce"] = F.cross_entropy(cortex[:, :-1].reshape(-1, cortex.size(-1)).float(), input_ids[:, 1:].reshape(-1))
        total = total + ce_weight * losses["ce"]
    total.backward()
    torch.nn.utils.clip_grad_norm_([p for p in student.parameters() if p.grad is not None], 1.0)
    optimizer.step()
    losses["loss"] = total
    vals = torch.stack([v.detach().float() for v in losses.values()]).tolist()  # one host read
    return dict(zip(losses.keys(), vals))
