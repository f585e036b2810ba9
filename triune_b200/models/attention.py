"""Sequence mixers: gated linear attention, Gated DeltaNet and softmax attention.

Parity: ``VectorisedGLA`` / ``HybridAttention`` of the reference (``triune/model/attention.py:296-653``):
bias-free q/k/v/g/out projections, q,k = normalize(elu+1) then RoPE, g = logsigmoid, O(1) recurrent
cache ``(state, offset)``. Design differences: the four input projections are ONE parameter
(``qkvg_weight`` [4*H*D, dim]) so the fused GEMM needs no concatenation, and it is split back into
``{q,k,v,g}_proj.weight`` only when a state dict is written or read.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import gla_cuda
from ..config import GLA_HEAD_DIM, ROPE_BASE, ROPE_MAX_SEQ_LEN
from .rotary import RotaryEmbedding


def parse_cache(cache: Any) -> Tuple[Optional[torch.Tensor], int, str]:
    """Accept the three cache formats of the reference: tuple (state, offset), dict, bare tensor."""
    def _off(o):  # a device tensor offset (position kept on the GPU for graph-replayed decoding) passes through
        return o if torch.is_tensor(o) else int(o)

    if isinstance(cache, dict):
        return cache.get("state"), _off(cache.get("offset", 0)), "dict"
    if isinstance(cache, tuple):
        return cache[0], _off(cache[1]), "tuple"
    if torch.is_tensor(cache):
        return cache, 0, "tensor"
    return None, 0, "none"


def format_cache(state, cache, fmt: str, offset: int, seq_len: int):
    if fmt == "dict":
        return {"state": state, "offset": offset + seq_len}
    if fmt == "tuple":
        return (state, offset + seq_len)
    if fmt == "tensor":
        return state
    return (state, offset + seq_len) if cache is not None else None


class _ProjView:
    """Read-only stand-in for ``nn.Linear`` exposing a slice of the fused projection weight."""

    def __init__(self, owner: "VectorisedGLA", index: int):
        self._owner, self._index = owner, index

    @property
    def weight(self) -> torch.Tensor:
        hd = self._owner.hidden_dim
        return self._owner.qkvg_weight[self._index * hd : (self._index + 1) * hd]

    bias = None

    def __call__(self, x):
        return F.linear(x, self.weight)


def _project(mod: nn.Module, x: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
    """Plain ``nn.Linear`` goes straight to the GEMM (``alpha`` rides in its epilogue); wrapped / quantised
    replacements (LoRA, FP8, NVFP4) run their own forward."""
    if type(mod) is nn.Linear:
        return ops.linear(x, mod.weight, mod.bias, alpha)
    return mod(x if alpha == 1.0 else x * alpha)


def set_gla_scale(model: nn.Module, mode) -> int:
    """Output scale of every (non-delta-rule) GLA mixer of ``model``: ``"none"`` / ``None`` = 1, ``"fla"`` =
    head_dim ** -0.5, or a number. Returns the number of mixers set.

    The reference multiplies nothing on its PyTorch path, but where the flash-linear-attention package is installed
    its CUDA path calls ``chunk_gla(..., scale=None)`` (``triune/model/attention.py:536-566``), whose default is
    head_dim ** -0.5 on the queries. A checkpoint trained there carries that factor in its weights, so the choice is
    part of the model's configuration here (``ModelConfig.gla_scale``) instead of depending on what is installed.
    GLA is linear in the queries, so the factor is applied to the mixer output, inside the output projection's GEMM."""
    n = 0
    for m in model.modules():
        if isinstance(m, VectorisedGLA) and not m.use_delta_rule:
            if mode in (None, "none", "", 1, 1.0):
                m.out_scale = 1.0
            elif mode == "fla":
                m.out_scale = float(m.head_dim) ** -0.5
            else:
                m.out_scale = float(mode)
            n += 1
    return n


class VectorisedGLA(nn.Module):
    """Multi-head GLA (or Gated DeltaNet when ``use_delta_rule``) with fused QKVG projection."""

    _SPLIT = ("q_proj", "k_proj", "v_proj", "g_proj")

    def __init__(self, dim: int, heads: int, head_dim: int = GLA_HEAD_DIM, use_delta_rule: bool = False,
                 use_rope: bool = True, rope_base: float = ROPE_BASE, rope_max_seq_len: int = ROPE_MAX_SEQ_LEN,
                 learn_beta: bool = False):
        super().__init__()
        self.dim, self.heads, self.head_dim = dim, heads, head_dim
        self.hidden_dim = heads * head_dim
        self.use_delta_rule = use_delta_rule
        self.use_rope = use_rope
        self.out_scale = 1.0  # see set_gla_scale
        self.qkvg_weight = nn.Parameter(torch.empty(4 * self.hidden_dim, dim))
        self.out_proj = nn.Linear(self.hidden_dim, dim, bias=False)
        self.beta_proj = nn.Linear(dim, heads, bias=False) if (use_delta_rule and learn_beta) else None
        nn.init.normal_(self.qkvg_weight, mean=0.0, std=0.02)
        if use_rope:
            self.rope = RotaryEmbedding(head_dim, max_seq_len=rope_max_seq_len, base=rope_base)
        self._register_state_dict_hook(self._split_on_save)
        self._register_load_state_dict_pre_hook(self._fuse_on_load)

    # --- reference-compatible checkpoint keys -----------------------------------------------
    @staticmethod
    def _split_on_save(module, state_dict, prefix, local_metadata):
        w = state_dict.pop(prefix + "qkvg_weight")
        hd = module.hidden_dim
        for i, name in enumerate(VectorisedGLA._SPLIT):
            state_dict[f"{prefix}{name}.weight"] = w[i * hd : (i + 1) * hd]
        return state_dict

    def _fuse_on_load(self, state_dict, prefix, *args):
        keys = [f"{prefix}{n}.weight" for n in self._SPLIT]
        if all(k in state_dict for k in keys):
            state_dict[prefix + "qkvg_weight"] = torch.cat([state_dict.pop(k) for k in keys], dim=0)

    @property
    def q_proj(self):
        return _ProjView(self, 0)

    @property
    def k_proj(self):
        return _ProjView(self, 1)

    @property
    def v_proj(self):
        return _ProjView(self, 2)

    @property
    def g_proj(self):
        return _ProjView(self, 3)

    def forward(self, x: torch.Tensor, cache=None):
        B, T, _ = x.shape
        H, D = self.heads, self.head_dim
        state, offset, fmt = parse_cache(cache)
        lora = getattr(self, "qkvg_lora", None)  # set by the fine-tuner (FusedProjectionLoRA)
        x2 = x.reshape(B * T, self.dim)
        qkvg = lora(x2) if lora is not None else ops.linear(x2, self.qkvg_weight)
        cos = sin = None
        if self.use_rope:
            cos, sin = self.rope(T, x.device, offset=offset)
        if not self.use_delta_rule and gla_cuda.core_supported(qkvg, T, D):
            out, new_state = gla_cuda.gla_attention_core(qkvg, cos, sin, state, B, T, H)
            y = _project(self.out_proj, out.view(B, T, self.hidden_dim), self.out_scale)
            return y, format_cache(new_state if cache is not None else None, cache, fmt, offset, T)
        q, k, v, g = ops.qk_feature_map(qkvg, cos, sin, B, T, H, D)
        if self.use_delta_rule:
            beta = torch.sigmoid(self.beta_proj(x)).view(B, T, H) if self.beta_proj is not None else None
            out, new_state = ops.gated_deltanet(q, k, v, g, beta=beta, initial_state=state, gate_logits=True)
        else:
            out, new_state = ops.gla(q, k, v, g, initial_state=state, gate_logits=True)
        out = out.reshape(B, T, self.hidden_dim).to(x.dtype)
        y = _project(self.out_proj, out, 1.0 if self.use_delta_rule else self.out_scale)
        return y, format_cache(new_state if cache is not None else None, cache, fmt, offset, T)


    def forward_token_states(self, x: torch.Tensor, state, offset):
        """``x`` [B, T, dim] with T small -> (y [B, T, dim], states [T, B, H, D, D]): the mixer output of every token and
        the recurrent state AFTER every token. Speculative verification runs all drafted tokens in one batched pass
        (one projection GEMM in, one out) and then keeps the state of the last ACCEPTED token; a recurrent state cannot
        be rolled back, so the per-token states are what replaces truncating a KV cache."""
        B, T, _ = x.shape
        H, D = self.heads, self.head_dim
        x2 = x.reshape(B * T, self.dim)
        qkvg = ops.linear(x2, self.qkvg_weight)
        cos = sin = None
        if self.use_rope:
            cos, sin = self.rope(T, x.device, offset=offset)
        q, k, v, g = ops.qk_feature_map(qkvg, cos, sin, B, T, H, D)
        beta = None
        if self.use_delta_rule and self.beta_proj is not None:
            beta = torch.sigmoid(self.beta_proj(x)).view(B, T, H)
        outs, states, s = [], [], state
        for j in range(T):
            sl = slice(j, j + 1)
            if self.use_delta_rule:
                o, s = ops.gated_deltanet(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta=None if beta is None else beta[:, sl],
                                          initial_state=s, gate_logits=True)
            else:
                o, s = ops.gla(q[:, sl], k[:, sl], v[:, sl], g[:, sl], initial_state=s, gate_logits=True)
            outs.append(o)
            states.append(s)
        out = torch.cat(outs, dim=1).reshape(B, T, self.hidden_dim).to(x.dtype)
        y = _project(self.out_proj, out, 1.0 if self.use_delta_rule else self.out_scale)
        return y, torch.stack(states)


class SoftmaxAttention(nn.Module):
    """Causal softmax attention with RoPE, GQA and a KV cache (library SDPA; not on a named hot path).

    Reference: the ``use_sdpa`` branch of ``HybridAttention`` (``triune/model/attention.py:606-653``) and the
    dense model's attention (``triune/universal.py:200-266``).
    """

    def __init__(self, dim: int, heads: int, head_dim: Optional[int] = None, num_kv_heads: Optional[int] = None,
                 rope_base: float = ROPE_BASE, rope_max_seq_len: int = ROPE_MAX_SEQ_LEN):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.head_dim = head_dim or dim // heads
        self.kv_heads = num_kv_heads or heads
        self.q_proj = nn.Linear(dim, heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(dim, self.kv_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(dim, self.kv_heads * self.head_dim, bias=False)
        self.out_proj = nn.Linear(heads * self.head_dim, dim, bias=False)
        self.rope = RotaryEmbedding(self.head_dim, max_seq_len=rope_max_seq_len, base=rope_base)

    def forward(self, x, cache=None):
        B, T, _ = x.shape
        past, offset, fmt = parse_cache(cache)
        q = ops.linear(x, self.q_proj.weight).view(B, T, self.heads, self.head_dim)
        k = ops.linear(x, self.k_proj.weight).view(B, T, self.kv_heads, self.head_dim)
        v = ops.linear(x, self.v_proj.weight).view(B, T, self.kv_heads, self.head_dim)
        cos, sin = self.rope(T, x.device, offset=offset)
        q, k = ops.apply_rope(q, cos, sin), ops.apply_rope(k, cos, sin)
        if past is not None:
            k = torch.cat((past[0], k), dim=1)
            v = torch.cat((past[1], v), dim=1)
        new_state = (k, v) if cache is not None else None
        kk, vv = k, v
        if self.kv_heads != self.heads:
            rep = self.heads // self.kv_heads
            kk, vv = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        if past is None or T == 1:
            mask, causal = None, (past is None and T > 1)
        else:  # a multi-token chunk after a prefix: query i sees the whole prefix and chunk positions <= i
            P = kk.shape[1] - T
            mask = torch.ones(T, P + T, dtype=torch.bool, device=x.device).tril(diagonal=P)
            causal = False
        o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), attn_mask=mask,
                                           is_causal=causal)
        o = o.transpose(1, 2).reshape(B, T, self.heads * self.head_dim)
        return _project(self.out_proj, o), format_cache(new_state, cache, fmt, offset, T)


class HybridAttention(nn.Module):
    """Attention slot of a block: GLA by default, softmax attention when ``use_sdpa``."""

    def __init__(self, dim: int, heads: int, use_fp4: bool = False, use_fp8: bool = False, use_delta_rule: bool = False,
                 use_sdpa: bool = False, layer_idx: int = 0, reflex_exit_layer: Optional[int] = None,
                 head_dim: Optional[int] = None, **kwargs):
        super().__init__()
        self.dim, self.heads = dim, heads
        self.use_sdpa = use_sdpa
        self.layer_idx = layer_idx
        self.head_dim = head_dim or (dim // heads if heads > 0 and dim % heads == 0 else GLA_HEAD_DIM)
        if use_sdpa:
            self.sdpa = SoftmaxAttention(dim, heads, self.head_dim, **{k: v for k, v in kwargs.items() if k in ("num_kv_heads",)})
            self.gla = None
        else:
            self.gla = VectorisedGLA(dim, heads, self.head_dim, use_delta_rule=use_delta_rule,
                                     **{k: v for k, v in kwargs.items() if k in ("use_rope", "rope_base", "rope_max_seq_len", "learn_beta")})
            self.sdpa = None

    def forward(self, x, cache=None):
        return (self.sdpa if self.use_sdpa else self.gla)(x, cache=cache)
