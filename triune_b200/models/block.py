"""Pre-norm transformer block: mixer, dense or MoE FFN, optional early-exit head.

Parity: ``TransformerBlock`` (``triune/model/block.py:20-120``): ``x += attn(norm1 x)``, ``x += ffn(norm2 x)``,
exit head = ``Linear(d, V)`` WITH bias after its own RMSNorm, per-sub-block activation checkpointing, and
token-compacted FFN under an ``active_mask``. Here the residual add after the mixer is fused with the second
norm (one pass over the stream), and the dense FFN is a single fused op (GEMM + bias + GELU epilogue).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn
import torch.utils.checkpoint

from .. import ops
from ..config import NUM_EXPERTS, TOP_K_EXPERTS, checkpoint_bwd_ctx
from .attention import HybridAttention
from .moe import MoE_FFN
from .norms import RMSNorm


class DenseFFN(nn.Sequential):
    """Linear -> GELU(tanh) -> Linear, state-dict keys ``0.*`` / ``2.*`` like ``nn.Sequential``."""

    def __init__(self, dim: int, hidden: int):
        super().__init__(nn.Linear(dim, hidden), nn.GELU(approximate="tanh"), nn.Linear(hidden, dim))

    def forward(self, x):
        if type(self[0]) is nn.Linear and type(self[2]) is nn.Linear:
            return ops.mlp_gelu(x, self[0].weight, self[0].bias, self[2].weight, self[2].bias)
        if getattr(self[0], "fused_gelu", False):  # quantised projections take the activation into their GEMM epilogue
            return self[2](self[0](x, gelu=True))
        return self[2](ops.gelu_tanh(self[0](x)))  # wrapped projections run their own forward


class TransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, layer_idx: int, vocab_size: int, exit_layers, num_experts: int = NUM_EXPERTS,
                 use_moe: bool = True, use_fp4: bool = False, use_fp8: bool = False, use_sdpa: bool = False,
                 top_k: int = TOP_K_EXPERTS, expert_hidden: Optional[int] = None, dense_hidden: Optional[int] = None,
                 shared_expert: bool = True, head_dim: Optional[int] = None, use_delta_rule: bool = False,
                 capacity_multiplier: float = 1.5, **attn_kwargs):
        super().__init__()
        self.attn = HybridAttention(dim, heads, use_fp4=use_fp4, use_fp8=use_fp8, use_sdpa=use_sdpa, layer_idx=layer_idx,
                                    reflex_exit_layer=min(exit_layers) if exit_layers else None, head_dim=head_dim,
                                    use_delta_rule=use_delta_rule, **attn_kwargs)
        if use_moe:
            self.ffn = MoE_FFN(dim, num_experts=num_experts, top_k=top_k, use_fp4=use_fp4, use_fp8=use_fp8,
                               shared_expert=shared_expert, expert_hidden=expert_hidden,
                               capacity_multiplier=capacity_multiplier)
        else:
            self.ffn = DenseFFN(dim, dense_hidden or dim * 4)
        self.norm1 = RMSNorm(dim)
        self.norm2 = RMSNorm(dim)
        self.layer_idx = layer_idx
        if layer_idx in exit_layers:
            self.exit_norm = RMSNorm(dim)
            self.exit_head = nn.Linear(dim, vocab_size)
        else:
            self.exit_norm = None
            self.exit_head = None
        self.use_moe = use_moe
        self._use_gradient_checkpointing = False

    def _ffn(self, n, update_stats):
        return self.ffn(n, update_stats=update_stats) if isinstance(self.ffn, MoE_FFN) else self.ffn(n)

    def _body(self, x, cache, update_stats):
        attn_out, new_cache = self.attn(self.norm1(x), cache=cache)
        n2, x = self.norm2.forward_add(attn_out, x)
        return x + self._ffn(n2, update_stats), new_cache

    def exit_logits(self, x, last_token_only: bool = False):
        xe = x[:, -1:, :] if last_token_only else x
        return ops.linear(self.exit_norm(xe), self.exit_head.weight, self.exit_head.bias)

    def forward(self, x: torch.Tensor, return_exit: bool = False, cache=None, update_stats: bool = True,
                exit_decider: Optional[Callable[[torch.Tensor], bool]] = None, exit_last_token_only: bool = False,
                active_mask: Optional[torch.Tensor] = None):
        compact = active_mask is not None and active_mask.shape == x.shape[:2] and not bool(active_mask.all())
        if compact:
            attn_out, new_cache = self.attn(self.norm1(x), cache=cache)
            x = x + attn_out
            xa = x[active_mask]
            if xa.numel() > 0:
                fa = self._ffn(self.norm2(xa.unsqueeze(0)), update_stats).squeeze(0)
                x = x.clone()
                x[active_mask] = xa + fa.to(x.dtype)
        elif self._use_gradient_checkpointing and self.training and torch.is_grad_enabled() and cache is None:
            # the MoE statistics update must run exactly once: on the first pass, not on the recomputation
            calls = {"n": 0}

            def run(t):
                first = calls["n"] == 0
                calls["n"] += 1
                if first:
                    return self._body(t, None, update_stats)
                with checkpoint_bwd_ctx():  # user modules inside the block can ask is_checkpoint_recomputing()
                    return self._body(t, None, False)

            x, new_cache = torch.utils.checkpoint.checkpoint(run, x, use_reentrant=False)
        else:
            x, new_cache = self._body(x, cache, update_stats)
        if self.exit_head is not None and (return_exit or (exit_decider is not None and exit_decider(x))):
            return x, self.exit_logits(x, exit_last_token_only), new_cache
        return x, None, new_cache
