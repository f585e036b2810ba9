"""Analytic device-memory model and execution-mode recommendation.

Parity (``triune/runtime/memory_planner.py:28-254``): ``MemoryPlanner.estimate_vram(config)`` returns a breakdown
(parameters / optimizer / activations / overhead), whether the run fits, and recommended batch / precision / streaming
settings; ``estimate_hf_model`` does the same from a Hugging Face config. The accounting follows THIS framework's
training state: bf16 parameters + fp32 master + fp32 gradient arena (10 B / param), AdamW moments for the AdamW tier,
one momentum buffer for the Muon tier, subspace state for the expert tier, and activations of the fused kernels (the
GLA scan keeps chunk states, not T x T scores; the loss never materialises the logits).
"""

from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Optional

import torch

from ..config import ModelConfig, model_config_from_flat

GB = 2.0**30
B200_HBM_GB = 180.0


@dataclass
class MemoryEstimate:
    total_params: int
    active_params: int
    param_memory_gb: float
    optimizer_memory_gb: float
    gradient_memory_gb: float
    activation_memory_gb: float
    overhead_gb: float
    total_gb: float
    available_gb: float
    fits: bool
    recommended_batch_size: int
    recommended_mode: str           # "resident" | "resident+checkpointing" | "layer_streaming" | "disk_streaming"
    recommended_precision: str
    notes: list = field(default_factory=list)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


class MemoryPlanner:
    @staticmethod
    def _cfg(config) -> ModelConfig:
        return config if isinstance(config, ModelConfig) else model_config_from_flat(dict(config))

    @staticmethod
    def activation_bytes_per_token(cfg: ModelConfig, checkpointing: bool) -> float:
        d, L = cfg.hidden_dim, cfg.num_layers
        hd = cfg.num_heads * cfg.head_dim
        if checkpointing:
            return 2.0 * d * L + 2.0 * (8 * d + 4 * hd + cfg.resolved_expert_hidden() * max(1, cfg.top_k))  # inputs + one live layer
        dense = 2.0 * (6 * d + 5 * hd + 2 * cfg.resolved_dense_hidden())
        moe = 2.0 * (6 * d + 5 * hd + (cfg.top_k + (1 if cfg.shared_expert else 0)) * (2 * cfg.resolved_expert_hidden() + 2 * d))
        n_dense = min(L, cfg.reflex_exit_layer + 1) if cfg.family == "triune" else L
        chunk_states = 4.0 * cfg.num_heads * cfg.head_dim * cfg.head_dim / 64.0  # one fp32 state per 64-token chunk
        return n_dense * dense + (L - n_dense) * moe + L * chunk_states

    @classmethod
    def estimate_vram(cls, config, target_vram_gb: float = B200_HBM_GB, available_vram_gb: Optional[float] = None,
                      training: bool = True) -> MemoryEstimate:
        raw = config if isinstance(config, dict) else config.to_dict()
        cfg = cls._cfg(config)
        if available_vram_gb is None and torch.cuda.is_available():
            available_vram_gb = torch.cuda.get_device_properties(0).total_memory / GB
        avail = float(available_vram_gb or target_vram_gb)
        total, active = cfg.param_count()
        wbytes = 0.5625 if raw.get("use_fp4") else (1.0 if raw.get("use_fp8") else 2.0)
        batch, seq = int(raw.get("batch_size", 16)), int(raw.get("seq_len", 2048))
        ckpt = bool(raw.get("gradient_checkpointing", False))
        param_gb = total * wbytes / GB
        if training:
            master_gb = total * 4.0 / GB
            grad_gb = total * 4.0 / GB
            emb = 2 * cfg.vocab_size * cfg.hidden_dim + cfg.vocab_size
            expert = max(0, total - active) + 0  # routed experts dominate the steer tier
            muon = max(0, total - emb - expert)
            opt_gb = master_gb + (emb * 8.0 + muon * 4.0 + expert * 0.5) / GB
        else:
            grad_gb = opt_gb = 0.0
        act_tok = cls.activation_bytes_per_token(cfg, ckpt) if training else 2.0 * (4 * cfg.hidden_dim)
        act_gb = act_tok * batch * seq / GB
        if not training:  # recurrent state per sequence instead of activations per token
            act_gb += batch * cfg.num_layers * cfg.num_heads * cfg.head_dim * cfg.head_dim * 4.0 / GB
        overhead = 1.5 + 0.02 * (param_gb + opt_gb)  # context, workspace, allocator slack
        need = param_gb + opt_gb + grad_gb + act_gb + overhead
        notes = []
        mode, rec_batch = "resident", batch
        if need > avail:
            fixed = param_gb + opt_gb + grad_gb + overhead
            if fixed < avail * 0.9:
                if not ckpt and training:
                    act_ck = cls.activation_bytes_per_token(cfg, True) * batch * seq / GB
                    if fixed + act_ck <= avail:
                        mode = "resident+checkpointing"
                        notes.append("activation checkpointing makes the requested batch fit")
                if mode == "resident":
                    per_seq = act_gb / max(1, batch)
                    rec_batch = max(1, int((avail * 0.9 - fixed) / max(per_seq, 1e-9)))
                    notes.append(f"batch reduced from {batch} to {rec_batch}")
            elif param_gb / max(1, cfg.num_layers) * 3 + overhead < avail:
                mode, rec_batch = "layer_streaming", max(1, batch // 2)
                notes.append("training state exceeds device memory: stream layers from pinned host memory")
            else:
                mode, rec_batch = "disk_streaming", 1
                notes.append("a single layer's training state does not fit: stream NVFP4 weights from disk (QLoRA)")
        prec = "fp4" if raw.get("use_fp4") else ("fp8" if raw.get("use_fp8") else "bf16")
        return MemoryEstimate(total, active, param_gb, opt_gb, grad_gb, act_gb, overhead, need, avail, need <= avail,
                              rec_batch, mode, prec, notes)

    @classmethod
    def estimate_hf_model(cls, hf_config: Any, batch_size: int = 1, seq_len: int = 2048, training: bool = False,
                          available_vram_gb: Optional[float] = None, quantization: Optional[str] = None) -> Dict[str, Any]:
        g = (lambda k, d=None: hf_config.get(k, d)) if isinstance(hf_config, dict) else (lambda k, d=None: getattr(hf_config, k, d))
        d, L = int(g("hidden_size", 4096)), int(g("num_hidden_layers", 32))
        V, ff = int(g("vocab_size", 32000)), int(g("intermediate_size", 4 * d))
        heads = int(g("num_attention_heads", max(1, d // 128)))
        kv = int(g("num_key_value_heads", heads) or heads)
        hd = int(g("head_dim", d // heads) or d // heads)
        E = int(g("num_local_experts", g("num_experts", 1)) or 1)
        attn = d * heads * hd * 2 + d * kv * hd * 2
        mlp = 3 * d * ff * E + (d * E if E > 1 else 0)
        total = V * d * (1 if g("tie_word_embeddings", False) else 2) + L * (attn + mlp + 2 * d) + d
        q = (quantization or "").lower()
        wbytes = 0.5625 if ("4" in q) else (1.0 if "8" in q else 2.0)
        param_gb = total * wbytes / GB
        kv_gb = 2.0 * L * kv * hd * 2.0 * batch_size * seq_len / GB
        train_gb = total * 12.0 / GB if training else 0.0
        act_gb = (2.0 * batch_size * seq_len * (d * (34 if training else 4) + (5 * heads * 0))) * (L if training else 1) / GB
        if available_vram_gb is None and torch.cuda.is_available():
            available_vram_gb = torch.cuda.get_device_properties(0).total_memory / GB
        avail = float(available_vram_gb or B200_HBM_GB)
        need = param_gb + kv_gb + train_gb + act_gb + 1.5
        if need <= avail:
            mode = "resident"
        elif param_gb / max(1, L) * 3 + kv_gb + 2 < avail:
            mode = "layer_streaming"
        else:
            mode = "disk_streaming"
        return {"total_params": int(total), "param_memory_gb": param_gb, "kv_cache_gb": kv_gb, "training_state_gb": train_gb,
                "activation_gb": act_gb, "total_gb": need, "available_gb": avail, "fits": need <= avail,
                "recommended_mode": mode, "recommended_quantization": None if need <= avail else ("nvfp4" if wbytes > 0.6 else q)}
