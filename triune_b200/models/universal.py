"""Dense and MoE "universal" transformers and the small engine around them.

Parity: ``triune/universal.py:147-666`` of the reference (``UniversalDenseTransformer``,
``UniversalMoETransformer``, ``TriuneUniversalEngine``, ``upgrade_model``). The dense model takes a
``mixer`` in {``sdpa``, ``gla``, ``gated_deltanet``} and a ``ffn`` in {``swiglu``, ``gelu``}; residual adds are
fused with the following RMSNorm; the gate and up projections of SwiGLU are ONE weight so the FFN is two GEMMs.
``UniversalTransformer`` is an alias of the dense class.
"""

from __future__ import annotations

from typing import Any, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from .attention import SoftmaxAttention, VectorisedGLA
from .block import DenseFFN
from .norms import RMSNorm


class SwiGLUFFN(nn.Module):
    """down( silu(gate(x)) * up(x) ) with gate and up stored as one [2*hidden, dim] weight."""

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.dim, self.hidden = dim, hidden
        self.gate_up = nn.Parameter(torch.empty(2 * hidden, dim))
        self.down = nn.Linear(hidden, dim, bias=False)
        nn.init.normal_(self.gate_up, std=0.02)
        self._register_state_dict_hook(self._split)
        self._register_load_state_dict_pre_hook(self._fuse)

    @staticmethod
    def _split(module, sd, prefix, meta):
        w = sd.pop(prefix + "gate_up")
        sd[prefix + "gate_proj.weight"], sd[prefix + "up_proj.weight"] = w[: module.hidden], w[module.hidden:]
        sd[prefix + "down_proj.weight"] = sd.pop(prefix + "down.weight")
        return sd

    def _fuse(self, sd, prefix, *a):
        g, u = prefix + "gate_proj.weight", prefix + "up_proj.weight"
        if g in sd and u in sd:
            sd[prefix + "gate_up"] = torch.cat((sd.pop(g), sd.pop(u)), dim=0)
        if prefix + "down_proj.weight" in sd:
            sd[prefix + "down.weight"] = sd.pop(prefix + "down_proj.weight")

    def forward(self, x):
        return ops.swiglu_mlp(x, self.gate_up, self.down.weight)


class DenseAttention(nn.Module):
    """A stand-alone attention layer with the reference's constructor (``triune/universal.py:147-268``): grouped-query
    softmax attention, or gated linear attention when ``use_gla``. ``forward(x, state) -> (out, new_state)`` where the
    state is the key/value cache or the GLA recurrent state."""

    def __init__(self, dim: int, num_heads: int, head_dim: Optional[int] = None, num_kv_heads: Optional[int] = None,
                 use_gla: bool = False):
        super().__init__()
        self.dim, self.num_heads, self.use_gla = dim, num_heads, use_gla
        self.head_dim = head_dim or dim // num_heads
        self.num_kv_heads = num_kv_heads or num_heads
        self.mixer = (VectorisedGLA(dim, num_heads, self.head_dim) if use_gla
                      else SoftmaxAttention(dim, num_heads, self.head_dim, self.num_kv_heads))

    def forward(self, x, state=None):
        return self.mixer(x, cache=state)


class DenseMLP(nn.Module):
    """A stand-alone feed-forward layer (``triune/universal.py:270-315``): SwiGLU (two GEMMs, gate and up as one weight)
    or GELU. ``hidden_dim`` defaults to four times ``dim``."""

    def __init__(self, dim: int, hidden_dim: Optional[int] = None, act_type: str = "swiglu"):
        super().__init__()
        self.act_type = act_type.lower()
        hidden = hidden_dim or 4 * dim
        self.ffn = SwiGLUFFN(dim, hidden) if self.act_type == "swiglu" else DenseFFN(dim, hidden)

    def forward(self, x):
        return self.ffn(x)


class DenseTransformerBlock(nn.Module):
    """Pre-norm block of ``DenseAttention`` and ``DenseMLP`` (``triune/universal.py:317-345``); the residual add and the
    second norm are one kernel. ``forward(x, state) -> (x, new_state)``."""

    def __init__(self, dim: int, num_heads: int, hidden_dim: Optional[int] = None, num_kv_heads: Optional[int] = None,
                 use_gla: bool = False):
        super().__init__()
        self.norm1 = RMSNorm(dim)
        self.attn = DenseAttention(dim, num_heads, num_kv_heads=num_kv_heads, use_gla=use_gla)
        self.norm2 = RMSNorm(dim)
        self.mlp = DenseMLP(dim, hidden_dim=hidden_dim)

    def forward(self, x, state=None):
        a, new_state = self.attn(self.norm1(x), state=state)
        n, x = self.norm2.forward_add(a, x)
        return x + self.mlp(n), new_state


class UniversalBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int):
        super().__init__()
        d, H, D = cfg.hidden_dim, cfg.num_heads, cfg.head_dim
        if cfg.mixer == "sdpa":
            self.attn = SoftmaxAttention(d, H, D, cfg.num_kv_heads, cfg.rope_base, cfg.rope_max_seq_len)
        else:
            self.attn = VectorisedGLA(d, H, D, use_delta_rule=(cfg.mixer == "gated_deltanet"), use_rope=cfg.use_rope,
                                      rope_base=cfg.rope_base, rope_max_seq_len=cfg.rope_max_seq_len,
                                      learn_beta=(cfg.mixer == "gated_deltanet"))
        hidden = cfg.resolved_dense_hidden()
        self.mlp = SwiGLUFFN(d, hidden) if cfg.ffn == "swiglu" else DenseFFN(d, hidden)
        self.input_norm = RMSNorm(d)
        self.post_attn_norm = RMSNorm(d)
        self.layer_idx = layer_idx
        self._use_gradient_checkpointing = False

    def _body(self, x, cache):
        a, new_cache = self.attn(self.input_norm(x), cache=cache)
        n, x = self.post_attn_norm.forward_add(a, x)
        return x + self.mlp(n), new_cache

    def forward(self, x, cache=None):
        if self._use_gradient_checkpointing and self.training and torch.is_grad_enabled() and cache is None:
            return torch.utils.checkpoint.checkpoint(lambda t: self._body(t, None), x, use_reentrant=False)
        return self._body(x, cache)


class UniversalDenseTransformer(nn.Module):
    def __init__(self, cfg: Optional[ModelConfig] = None, **kw):
        super().__init__()
        if cfg is None:
            cfg = ModelConfig(family="universal", **kw)
        self.cfg = cfg
        self.vocab_size, self.hidden_dim, self.num_layers = cfg.vocab_size, cfg.hidden_dim, cfg.num_layers
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_dim)
        self.layers = nn.ModuleList([UniversalBlock(cfg, i) for i in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_dim)
        self.lm_head = nn.Linear(cfg.hidden_dim, cfg.vocab_size, bias=False)
        self.apply(self._init)
        if cfg.tie_embeddings:
            self.embed_tokens.weight = self.lm_head.weight

    @classmethod
    def from_config(cls, cfg: ModelConfig):
        model = cls(cfg)
        if getattr(cfg, "gla_scale", "none") not in (None, "none"):
            from .attention import set_gla_scale

            set_gla_scale(model, cfg.gla_scale)
        return model

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def init_cache(self, batch_size: int = 1) -> List[Any]:
        return [(None, 0) for _ in range(self.num_layers)]

    def enable_gradient_checkpointing(self, flag: bool = True):
        for l in self.layers:
            l._use_gradient_checkpointing = flag

    def hidden_states(self, input_ids=None, cache=None, inputs_embeds=None):
        x = inputs_embeds if inputs_embeds is not None else ops.embedding(input_ids, self.embed_tokens.weight)
        new_cache = list(cache) if cache is not None else None
        for i, layer in enumerate(self.layers):
            lc = None
            if cache is not None:
                lc = cache[i] if cache[i] is not None else (None, 0)
            x, nc = layer(x, cache=lc)
            if new_cache is not None:
                new_cache[i] = nc
        return self.norm(x), new_cache

    def forward(self, input_ids=None, cache=None, last_token_only: bool = False, inputs_embeds=None, force_depth=None,
                **_):
        h, new_cache = self.hidden_states(input_ids, cache, inputs_embeds)
        if last_token_only:
            h = h[:, -1:, :]
        logits = ops.linear(h, self.lm_head.weight)
        if cache is not None:
            return logits, new_cache
        return logits, None

    def forward_loss(self, input_ids, labels, force_depth: int = 2, ignore_index: int = -100, n_valid=None):
        h, _ = self.hidden_states(input_ids)
        return ops.linear_cross_entropy(h, self.lm_head.weight, labels, ignore_index=ignore_index, n_valid=n_valid)

    def num_parameters(self) -> int:
        return sum(p.numel() for p in {id(p): p for p in self.parameters()}.values())


UniversalTransformer = UniversalDenseTransformer


class UniversalMoETransformer(nn.Module):
    """Thin wrapper that presents a TriuneTransformer under the universal interface."""

    def __init__(self, cfg: Optional[ModelConfig] = None, **kw):
        super().__init__()
        from .transformer import TriuneTransformer

        cfg = cfg or ModelConfig(**kw)
        self.cfg = cfg
        self.model = TriuneTransformer.from_config(cfg)

    def forward(self, input_ids, **kw):
        kw.setdefault("force_depth", 2)
        return self.model(input_ids, **kw)

    def forward_loss(self, input_ids, labels, **kw):
        return self.model.forward_loss(input_ids, labels, **kw)

    def init_cache(self, batch_size: int = 1):
        return self.model.init_cache(batch_size)


class TriuneUniversalEngine:
    """Train-step / generate convenience around any model of this package (reference: ``universal.py:447-560``)."""

    def __init__(self, model: nn.Module, optimizer=None, lr: float = 1e-4, device=None):
        from ..optim.factory import build_optimizer

        self.model = model
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.optimizer = optimizer or build_optimizer(model, {"lr": lr})

    def train_step(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> float:
        self.model.train()
        if labels is None:
            input_ids, labels = input_ids[:, :-1], input_ids[:, 1:]
        loss = self.model.forward_loss(input_ids.to(self.device), labels.to(self.device))
        loss.backward()
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        return float(loss.detach())

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 32, temperature: float = 0.0, top_k: int = 0):
        self.model.eval()
        ids = input_ids.to(self.device)
        cache = self.model.init_cache(ids.shape[0])
        logits, cache = self.model(ids, cache=cache, last_token_only=True, force_depth=2)
        out = [ids]
        for _ in range(max_new_tokens):
            lg = logits[:, -1].float()
            if temperature > 0:
                if top_k > 0:
                    kth = torch.topk(lg, top_k).values[:, -1:]
                    lg = lg.masked_fill(lg < kth, float("-inf"))
                nxt = torch.multinomial(F.softmax(lg / temperature, -1), 1)
            else:
                nxt = lg.argmax(-1, keepdim=True)
            out.append(nxt)
            logits, cache = self.model(nxt, cache=cache, last_token_only=True, force_depth=2)
        return torch.cat(out, dim=1)


def _is_silu(act) -> bool:
    """True when a gated MLP's activation is SiLU (or unnamed, as in this framework's own blocks): only then is the MLP a
    SwiGLU; GELU-gated MLPs (Gemma) keep their own forward."""
    if act is None:
        return True
    if act is F.silu or isinstance(act, nn.SiLU):
        return True
    return type(act).__name__.lower() in ("silu", "siluactivation", "swish")


def upgrade_model(model: nn.Module, lora_rank: int = 0, streaming_device=None, attach_optimizer: bool = False, lr: float = 1e-4):
    """Patch a third-party (e.g. Hugging Face) causal LM in place: RMSNorm modules call the fused kernel, SwiGLU
    MLPs call the fused activation, and optionally LoRA adapters / layer streaming / a tiered optimizer are attached.
    Reference: ``triune/universal.py:562-666``."""
    patched = {"rmsnorm": 0, "swiglu": 0, "lora": 0}
    for mod in model.modules():
        name = mod.__class__.__name__.lower()
        if "rmsnorm" in name and isinstance(getattr(mod, "weight", None), torch.Tensor) and mod.weight.dim() == 1 \
                and not isinstance(mod, RMSNorm):
            eps = float(getattr(mod, "variance_epsilon", getattr(mod, "eps", 1e-6)))
            if "gemma" in name:  # the Gemma family stores the scale as an offset from one
                mod.forward = (lambda m, e: (lambda x: ops.rmsnorm(x, (1.0 + m.weight.float()).to(x.dtype), e)))(mod, eps)
            else:
                mod.forward = (lambda m, e: (lambda x: ops.rmsnorm(x, m.weight, e)))(mod, eps)
            patched["rmsnorm"] += 1
        elif all(hasattr(mod, a) for a in ("gate_proj", "up_proj", "down_proj")) and _is_silu(getattr(mod, "act_fn", None)):
            mod.forward = (lambda m: (lambda x: m.down_proj(ops.swiglu(m.gate_proj(x), m.up_proj(x)))))(mod)
            patched["swiglu"] += 1
    if lora_rank > 0:
        from ..trainer.finetune import LoRAConfig, apply_lora

        patched["lora"] = apply_lora(model, LoRAConfig(rank=lora_rank))
    if streaming_device is not None:
        from ..runtime.streaming import enable_layer_streaming

        enable_layer_streaming(model, streaming_device)
    if attach_optimizer:
        from ..optim.factory import build_optimizer

        model._triune_optimizer = build_optimizer(model, {"lr": lr, "optimizer": "adamw" if lora_rank > 0 else "centroid_steer"})
    model._triune_upgrade = patched
    return model
