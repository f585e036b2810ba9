"""TriuneTransformer: multi-exit (Reflex / Limbic / Cortex) MoE language model over GLA mixers.

Parity: ``triune/model/transformer.py:28-904`` of the reference. Same constructor arguments (plus
``top_k`` / ``expert_hidden`` / ``dense_hidden`` / ``shared_expert``), same state-dict keys, same forward
contract:

* ``forward(input_ids, force_depth, cache, temperature, return_balance_loss, last_token_only, exit_policy,
  confidence_threshold, inputs_embeds, tokenizer)`` returns ``(logits, route_logits[, balance_loss])`` or
  ``(logits, new_cache)`` when a cache is passed;
* layers ``0..reflex`` use a dense FFN, later layers the MoE FFN; exits sit on ``reflex_exit_layer`` and
  ``limbic_exit_layer``; the final head is tied to the embedding;
* ``exit_policy``: ``gumbel`` (depth router per sequence), ``calm`` / ``confidence`` (top-2 probability margin,
  Limbic threshold 0.85x, unsettled rows continue and settled tokens skip later FFNs), ``jev``.

The depth logic is organised around one primitive, :meth:`_advance` (run layers ``[a, b)`` on a residual
stream), instead of the reference's three unrolled branches. ``forward_loss`` adds a training entry point
that feeds the exit/LM heads into the fused head-GEMM + cross-entropy op so full logits never exist.
"""

from __future__ import annotations

import contextlib
import math
from typing import Any, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..config import (
    DEPTH_BALANCE_COEF,
    GLA_HEAD_DIM,
    HIDDEN_DIM,
    LIMBIC_EXIT_LAYER,
    NUM_EXPERTS,
    NUM_HEADS,
    NUM_LAYERS,
    REFLEX_EXIT_LAYER,
    ROUTER_PREFIX_LAYERS,
    TARGET_DEPTH_DIST,
    TOP_K_EXPERTS,
    VOCAB_SIZE,
    ModelConfig,
)
from .block import TransformerBlock
from .norms import RMSNorm
from .router import GumbelSoftmaxRouter


class TriuneTransformer(nn.Module):
    def __init__(
        self,
        vocab_size: int = VOCAB_SIZE,
        hidden_dim: int = HIDDEN_DIM,
        num_layers: int = NUM_LAYERS,
        num_heads: int = NUM_HEADS,
        head_dim: int = GLA_HEAD_DIM,
        num_experts: int = NUM_EXPERTS,
        router_prefix_layers: int = ROUTER_PREFIX_LAYERS,
        reflex_exit_layer: int = REFLEX_EXIT_LAYER,
        limbic_exit_layer: int = LIMBIC_EXIT_LAYER,
        target_depth_dist=TARGET_DEPTH_DIST,
        balance_coef: float = DEPTH_BALANCE_COEF,
        use_fp4: bool = False,
        use_fp8: bool = False,
        streaming_fp8_weights: bool = False,
        scale_residual_projections: bool = False,
        use_reflex_sdpa: bool = False,
        top_k: int = TOP_K_EXPERTS,
        expert_hidden: Optional[int] = None,
        dense_hidden: Optional[int] = None,
        shared_expert: bool = True,
        capacity_multiplier: float = 1.5,
    ):
        super().__init__()
        if not (0 < router_prefix_layers < reflex_exit_layer < limbic_exit_layer < num_layers):
            raise ValueError(
                f"Layer hierarchy violation: expected 0 < router_prefix_layers ({router_prefix_layers}) < "
                f"reflex_exit_layer ({reflex_exit_layer}) < limbic_exit_layer ({limbic_exit_layer}) < "
                f"num_layers ({num_layers})"
            )
        if num_experts < 1:
            raise ValueError(f"num_experts must be >= 1; got {num_experts}")
        if vocab_size < 1:
            raise ValueError(f"vocab_size must be >= 1; got {vocab_size}")
        if num_heads < 1 or head_dim < 1:
            raise ValueError(f"num_heads ({num_heads}) and head_dim ({head_dim}) must be >= 1")
        if not math.isfinite(balance_coef) or balance_coef < 0:
            raise ValueError(f"balance_coef must be a finite non-negative float; got {balance_coef}")
        if any(not math.isfinite(d) or d < 0 for d in target_depth_dist):
            raise ValueError(f"target_depth_dist elements must be finite non-negative floats; got {target_depth_dist}")
        if abs(sum(target_depth_dist) - 1.0) > 1e-4:
            raise ValueError(f"target_depth_dist must sum to 1.0; got {target_depth_dist}")
        if hidden_dim != num_heads * head_dim:
            raise ValueError(f"hidden_dim ({hidden_dim}) must equal num_heads * head_dim ({num_heads * head_dim})")
        self.num_layers, self.hidden_dim, self.num_heads, self.head_dim = num_layers, hidden_dim, num_heads, head_dim
        self.vocab_size, self.num_experts, self.top_k = vocab_size, num_experts, top_k
        self.router_prefix_layers = router_prefix_layers
        self.reflex_exit_layer, self.limbic_exit_layer = reflex_exit_layer, limbic_exit_layer
        self.use_fp4, self.use_fp8 = use_fp4, use_fp8
        self.last_route_logits = self.last_depth_choice = self.last_balance_loss = None
        self.last_calm_exit_depths = None
        self.last_calm_compaction_stats = None
        self._composite_id_map: dict[int, int] = {}
        self._base_vocab_size = vocab_size
        self.compressed_embed_mode = "mean_pool"

        self.token_embed = nn.Embedding(vocab_size, hidden_dim)
        exits = [reflex_exit_layer, limbic_exit_layer]
        self.layers = nn.ModuleList(
            [
                TransformerBlock(
                    hidden_dim, num_heads, i, vocab_size, exits, num_experts=num_experts,
                    use_moe=(i > reflex_exit_layer), use_fp4=use_fp4, use_fp8=use_fp8,
                    use_sdpa=use_reflex_sdpa and (i <= reflex_exit_layer), top_k=top_k, expert_hidden=expert_hidden,
                    dense_hidden=dense_hidden, shared_expert=shared_expert, head_dim=head_dim,
                    capacity_multiplier=capacity_multiplier,
                )
                for i in range(num_layers)
            ]
        )
        self.router = GumbelSoftmaxRouter(hidden_dim, target_depth_dist=target_depth_dist, balance_coef=balance_coef)
        self.jev_router = None
        self.final_norm = RMSNorm(hidden_dim)
        self.final_head = nn.Linear(hidden_dim, vocab_size, bias=False)
        self.apply(self._init_weights)
        self.token_embed.weight = self.final_head.weight
        if scale_residual_projections and num_layers > 0:
            std = 0.02 / math.sqrt(2 * num_layers)
            for name, p in self.named_parameters():
                if "out_proj" in name or name.endswith(".2.weight") or name.endswith(".w2"):
                    nn.init.normal_(p, mean=0.0, std=std)

    @classmethod
    def from_config(cls, cfg: ModelConfig) -> "TriuneTransformer":
        cfg.validate()
        model = cls._from_validated(cfg)
        model.model_config = cfg  # plain attribute: checkpoints record the architecture from here
        if getattr(cfg, "gla_scale", "none") not in (None, "none"):
            from .attention import set_gla_scale

            set_gla_scale(model, cfg.gla_scale)
        return model

    @classmethod
    def _from_validated(cls, cfg: ModelConfig) -> "TriuneTransformer":
        return cls(
            vocab_size=cfg.vocab_size, hidden_dim=cfg.hidden_dim, num_layers=cfg.num_layers, num_heads=cfg.num_heads,
            head_dim=cfg.head_dim, num_experts=cfg.num_experts, router_prefix_layers=cfg.router_prefix_layers,
            reflex_exit_layer=cfg.reflex_exit_layer, limbic_exit_layer=cfg.limbic_exit_layer,
            target_depth_dist=cfg.target_depth_dist, balance_coef=cfg.balance_coef, use_fp4=cfg.use_fp4,
            use_fp8=cfg.use_fp8, scale_residual_projections=cfg.scale_residual_projections, top_k=cfg.top_k,
            expert_hidden=cfg.expert_hidden, dense_hidden=cfg.dense_hidden, shared_expert=cfg.shared_expert,
            capacity_multiplier=cfg.capacity_multiplier,
        )

    @staticmethod
    def _init_weights(module):
        if isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=0.02)

    # ------------------------------------------------------------------ small utilities
    @property
    def exit_layers(self):
        return (self.reflex_exit_layer, self.limbic_exit_layer, self.num_layers - 1)

    def init_cache(self, batch_size: int = 1) -> list[Any]:
        return [(None, 0) for _ in range(self.num_layers)]

    def enable_gradient_checkpointing(self, flag: bool = True):
        for layer in self.layers:
            layer._use_gradient_checkpointing = flag

    def enable_jev_routing(self, threshold: float = 0.85, distance_metric: str = "geodesic"):
        from .jev import JEVExitRouter

        self.jev_router = JEVExitRouter(self.hidden_dim, threshold=threshold, distance_metric=distance_metric)
        p = next(self.parameters())
        self.jev_router.to(device=p.device, dtype=p.dtype)
        return self.jev_router

    def enable_layer_streaming(self, device, chunk_size: int = 1, pin_memory=None, async_prefetch: bool = True,
                               fp8_weights: bool = False, grad_clip: float = 1.0, instant_optimizer: bool = True,
                               resident_gpu_layers: int = 0, activation_checkpointing: bool = True):
        from ..runtime.streaming import LayerStreamingEngine, StreamingConfig

        cfg = StreamingConfig(enabled=True, chunk_size=chunk_size, pin_memory=pin_memory, async_prefetch=async_prefetch,
                              fp8_weights=fp8_weights, grad_clip=grad_clip, instant_optimizer=instant_optimizer,
                              resident_gpu_layers=resident_gpu_layers, activation_checkpointing=activation_checkpointing)
        engine = LayerStreamingEngine(self, device=device, config=cfg)
        engine.attach()
        self._streaming_engine = engine
        return engine

    @staticmethod
    def _slice_cache(cache, idx):
        if cache is None:
            return None
        out = []
        for entry in cache:
            if isinstance(entry, tuple) and entry[0] is not None:
                out.append((entry[0].index_select(0, idx), entry[1]))
            else:
                out.append(entry)
        return out

    @staticmethod
    def _scatter_cache(dst, src, idx, batch_size, device):
        if dst is None or src is None:
            return dst
        for i, entry in enumerate(src):
            if isinstance(entry, tuple) and entry[0] is not None:
                s, off = entry
                if isinstance(dst[i], tuple) and dst[i][0] is not None:
                    dst[i] = (dst[i][0].index_copy(0, idx, s.to(dst[i][0].dtype)), off)
                else:
                    full = torch.zeros(batch_size, *s.shape[1:], device=device, dtype=s.dtype)
                    dst[i] = (full.index_copy(0, idx, s), off)
        return dst

    # ------------------------------------------------------------------ embeddings
    def embed_compressed(self, input_ids: torch.Tensor, tokenizer) -> torch.Tensor:
        """Embed ids that include composite (n-gram) tokens >= base vocab by pooling constituent embeddings."""
        base_v = self._base_vocab_size
        flat = input_ids.reshape(-1)
        emb = self.token_embed(flat.clamp(max=self.token_embed.num_embeddings - 1))
        high = (flat >= base_v).nonzero(as_tuple=True)[0]
        if high.numel():
            rows = []
            for pos in high.tolist():
                parts = tokenizer.decompress_tokens([int(flat[pos])]) if hasattr(tokenizer, "decompress_tokens") else []
                parts = [p for p in parts if 0 <= p < base_v] or [0]
                e = self.token_embed(torch.tensor(parts, device=flat.device))
                if self.compressed_embed_mode == "order_pool":
                    wts = torch.linspace(1.0, 0.5, len(parts), device=flat.device, dtype=e.dtype).unsqueeze(1)
                    rows.append((e * wts).sum(0) / wts.sum())
                else:
                    rows.append(e.mean(0))
            emb = emb.clone()
            emb[high] = torch.stack(rows).to(emb.dtype)
        return emb.view(*input_ids.shape, -1)

    def extend_vocabulary_for_tokenizer(self, tokenizer) -> int:
        """Grow the tied embedding/head so composite ids get their own rows, initialised by pooling."""
        new_ids = sorted(getattr(tokenizer, "decomp_rules", {}).keys()) if hasattr(tokenizer, "decomp_rules") else []
        new_ids = [i for i in new_ids if i not in self._composite_id_map]
        if not new_ids:
            return 0
        old = self.final_head.weight.data
        start = old.shape[0]
        rows = []
        for cid in new_ids:
            parts = [p for p in tokenizer.decompress_tokens([cid]) if 0 <= p < self._base_vocab_size] or [0]
            rows.append(old[torch.tensor(parts, device=old.device)].mean(0))
        w = torch.cat((old, torch.stack(rows)), dim=0)
        self.final_head = nn.Linear(self.hidden_dim, w.shape[0], bias=False).to(device=old.device, dtype=old.dtype)
        self.final_head.weight.data.copy_(w)
        self.token_embed = nn.Embedding(w.shape[0], self.hidden_dim).to(device=old.device, dtype=old.dtype)
        self.token_embed.weight = self.final_head.weight
        for j, cid in enumerate(new_ids):
            self._composite_id_map[int(cid)] = start + j
        self.vocab_size = w.shape[0]
        for idx in (self.reflex_exit_layer, self.limbic_exit_layer):
            blk = self.layers[idx]
            oh = blk.exit_head
            nh = nn.Linear(self.hidden_dim, w.shape[0]).to(device=old.device, dtype=old.dtype)
            nh.weight.data[: oh.weight.shape[0]].copy_(oh.weight.data)
            nh.weight.data[oh.weight.shape[0]:].copy_(w[start:])
            nh.bias.data.zero_()
            nh.bias.data[: oh.bias.shape[0]].copy_(oh.bias.data)
            blk.exit_head = nh
        return len(new_ids)

    def _embed(self, input_ids, inputs_embeds, tokenizer):
        if (input_ids is None) == (inputs_embeds is None):
            raise ValueError("Provide exactly one of input_ids or inputs_embeds")
        if inputs_embeds is not None:
            return inputs_embeds
        tok = tokenizer if tokenizer is not None else getattr(self, "tokenizer", None)
        if self._composite_id_map or tok is not None:
            if input_ids.numel() > 0 and int(input_ids.max().item()) >= self._base_vocab_size:
                cmap = self._composite_id_map
                high = input_ids[input_ids >= self._base_vocab_size].unique().tolist()
                if cmap and all(int(t) in cmap for t in high):
                    remapped = input_ids.clone()
                    for t in high:
                        remapped[input_ids == int(t)] = cmap[int(t)]
                    return self.token_embed(remapped)
                if tok is not None:
                    return self.embed_compressed(input_ids, tok)
        return ops.embedding(input_ids, self.token_embed.weight)

    # ------------------------------------------------------------------ layer execution
    def _forward_block(self, layer, x, return_exit, cache=None, update_stats=True, exit_decider=None,
                       exit_last_token_only=False, active_mask=None):
        return layer(x, return_exit, cache, update_stats=update_stats, exit_decider=exit_decider,
                     exit_last_token_only=exit_last_token_only, active_mask=active_mask)

    def _run_layers(self, x, start_layer, end_layer, cache=None, update_stats=True, active_mask=None):
        new_cache = list(cache) if cache is not None else None
        for i in range(start_layer, end_layer):
            lc = None
            if cache is not None:
                lc = cache[i] if i < len(cache) and cache[i] is not None else (None, 0)
            x, _, nc = self._forward_block(self.layers[i], x, False, cache=lc, update_stats=update_stats,
                                           active_mask=active_mask)
            if new_cache is not None:
                new_cache[i] = nc
        return x, new_cache

    def _advance(self, x, start, depth, cache, last_token_only, update_stats=True, active_mask=None,
                 want_logits=True):
        """Run layers ``[start, exit_layer(depth)]`` and return (hidden, logits, cache)."""
        end = self.exit_layers[depth]
        x, cache = self._run_layers(x, start, end + 1, cache=cache, update_stats=update_stats, active_mask=active_mask)
        logits = None
        if want_logits:
            logits = self._head(x, depth, last_token_only)
        return x, logits, cache

    def _head_modules(self, depth: int):
        if depth == 2:
            return self.final_norm, self.final_head
        blk = self.layers[self.exit_layers[depth]]
        return blk.exit_norm, blk.exit_head

    def _head(self, x, depth: int, last_token_only: bool = False):
        norm, head = self._head_modules(depth)
        xe = x[:, -1:, :] if last_token_only else x
        return ops.linear(norm(xe), head.weight, head.bias)

    def _route(self, x, force_depth, B, device, temperature=1.0):
        logits, y, bal = self.router(x, temperature=temperature, force_depth=force_depth)
        if force_depth is None:
            choice = y.argmax(dim=-1)
        else:
            choice = torch.full((B,), force_depth, device=device, dtype=torch.long)
        return logits, y, choice, bal

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: Optional[torch.Tensor], force_depth: Optional[int] = None, cache: Optional[List[Any]] = None,
                temperature: float = 1.0, return_balance_loss: bool = False, last_token_only: bool = False,
                exit_policy: str = "gumbel", confidence_threshold: float = 0.8,
                inputs_embeds: Optional[torch.Tensor] = None, tokenizer: Optional[Any] = None):
        if force_depth is not None and force_depth not in (0, 1, 2):
            raise ValueError(f"force_depth must be 0, 1, or 2; got {force_depth}")
        x = self._embed(input_ids, inputs_embeds, tokenizer)
        B, T = x.shape[:2]
        device = x.device
        P = self.router_prefix_layers
        x_prefix, new_cache = self._run_layers(x, 0, P, cache=cache)
        route_logits, _, depth_choice, balance_loss = self._route(x_prefix, force_depth, B, device, temperature)
        self.last_route_logits = route_logits.detach()
        self.last_depth_choice = depth_choice.detach()
        self.last_balance_loss = balance_loss

        def finish(logits, nc):
            if cache is not None:
                return logits, nc
            if return_balance_loss:
                return logits, route_logits, balance_loss
            return logits, route_logits

        if force_depth is not None:
            _, logits, new_cache = self._advance(x_prefix, P, force_depth, new_cache, last_token_only)
            return finish(logits, new_cache)

        if exit_policy in ("calm", "confidence"):
            logits, new_cache = self._forward_calm(x_prefix, new_cache, cache is not None, last_token_only,
                                                   confidence_threshold)
            return finish(logits, new_cache)

        if exit_policy == "jev" and self.jev_router is not None:
            xr, jc = self._run_layers(x_prefix, P, self.reflex_exit_layer + 1, cache=new_cache)
            res = self.jev_router(xr)
            if float(res.should_exit.float().mean()) >= 0.5:
                return finish(self._head(xr, 0, last_token_only), jc)
            xc, jc = self._run_layers(xr, self.reflex_exit_layer + 1, self.num_layers, cache=jc)
            return finish(self._head(xc, 2, last_token_only), jc)

        # per-sequence depth chosen by the router
        final_logits = None
        for d in (0, 1, 2):
            idx = (depth_choice == d).nonzero(as_tuple=True)[0]
            if idx.numel() == 0:
                continue
            whole = idx.numel() == B
            x_d = x_prefix if whole else x_prefix.index_select(0, idx)
            d_cache = new_cache if whole else (self._slice_cache(new_cache, idx) if cache is not None else None)
            _, logits_d, d_cache = self._advance(x_d, P, d, d_cache, last_token_only)
            if whole:
                final_logits, new_cache = logits_d, d_cache
                break
            if final_logits is None:
                final_logits = torch.empty(B, logits_d.shape[1], logits_d.shape[2], device=device, dtype=logits_d.dtype)
            final_logits = final_logits.index_copy(0, idx, logits_d)
            if cache is not None:
                new_cache = self._scatter_cache(new_cache, d_cache, idx, B, device)
        if final_logits is None:
            final_logits = torch.empty(B, T, self.final_head.out_features, device=device, dtype=x_prefix.dtype)
        return finish(final_logits, new_cache)

    @staticmethod
    def _margin(logits):
        top2 = torch.topk(F.softmax(logits.float(), dim=-1), 2, dim=-1).values
        return top2[..., 0] - top2[..., 1]

    def _forward_calm(self, x_prefix, cache, use_cache, last_token_only, tau):
        """Confidence-based exits. Rows with any unsettled token continue; settled tokens skip later FFNs."""
        B = x_prefix.shape[0]
        device = x_prefix.device
        P = self.router_prefix_layers
        cache = cache if use_cache else None
        x, logits, cache = self._advance(x_prefix, P, 0, cache, last_token_only)
        out = logits.clone()
        settled = self._margin(logits) >= tau
        depths = torch.where(settled, 0, 2)
        stats = {"total_tokens": int(settled.numel()), "reflex_tokens": int(settled.sum()), "limbic_tokens": 0,
                 "cortex_tokens": 0, "limbic_rows": 0, "cortex_rows": 0, "limbic_seq_len": 0, "cortex_seq_len": 0}
        rows = torch.arange(B, device=device)
        start = self.reflex_exit_layer + 1
        for depth, thr, tag in ((1, tau * 0.85, "limbic"), (2, None, "cortex")):
            need = (~settled.index_select(0, rows)).any(dim=1).nonzero(as_tuple=True)[0] if rows.numel() else rows
            if need.numel() == 0:
                break
            rows = rows.index_select(0, need)
            x = x.index_select(0, need)
            uns = ~settled.index_select(0, rows)  # [rows, T_out]
            sub_cache = self._slice_cache(cache, rows) if use_cache else None
            T_cur = x.shape[1]
            if not last_token_only and not use_cache:
                cols = uns.any(dim=0).nonzero(as_tuple=True)[0]
                T_cur = int(cols[-1]) + 1
                x, uns = x[:, :T_cur], uns[:, :T_cur]
            mask = uns if (not last_token_only or x.shape[1] == 1) else None
            x, _, sub_cache = self._advance(x, start, depth, sub_cache, False, active_mask=mask, want_logits=False)
            if use_cache:
                cache = self._scatter_cache(cache, sub_cache, rows, B, device)
            stats[f"{tag}_rows"], stats[f"{tag}_seq_len"] = int(rows.numel()), T_cur
            if last_token_only:
                lg = self._head(x, depth, True)  # [rows, 1, V]
                r_idx = torch.arange(rows.numel(), device=device)
                t_idx = torch.zeros_like(r_idx)
                flat = lg[:, 0]
                sel = uns[:, -1] if uns.shape[1] == lg.shape[1] else uns[:, 0]
                r_idx, flat = r_idx[sel], flat[sel]
                t_idx = t_idx[sel]
            else:
                r_idx, t_idx = uns.nonzero(as_tuple=True)
                norm, head = self._head_modules(depth)
                flat = ops.linear(norm(x[r_idx, t_idx].unsqueeze(0)), head.weight, head.bias).squeeze(0)
            abs_rows = rows.index_select(0, r_idx)
            out = out.index_put((abs_rows, t_idx), flat.to(out.dtype))
            stats[f"{tag}_tokens"] = int(r_idx.numel())
            if thr is not None:
                ok = self._margin(flat) >= thr
                depths = depths.index_put((abs_rows, t_idx), torch.where(ok, 1, 2))
                settled = settled.index_put((abs_rows, t_idx), ok)
            else:
                settled = settled.index_put((abs_rows, t_idx), torch.ones_like(r_idx, dtype=torch.bool))
            start = self.exit_layers[depth] + 1
        self.last_calm_exit_depths = depths.detach()
        self.last_depth_choice = depths[:, -1].detach()
        self.last_calm_compaction_stats = stats
        return out, cache

    # ------------------------------------------------------------------ multi-exit helpers
    def forward_hidden_all_exits(self, input_ids, update_stats=False):
        """Hidden states at the three exits (before the exit norms) plus router outputs."""
        B = input_ids.shape[0]
        x = ops.embedding(input_ids, self.token_embed.weight)
        P = self.router_prefix_layers
        x_prefix, _ = self._run_layers(x, 0, P, update_stats=update_stats)
        route_logits, _, choice, bal = self._route(x_prefix, None, B, x.device)
        self.last_route_logits, self.last_depth_choice, self.last_balance_loss = route_logits.detach(), choice.detach(), bal
        xr, _ = self._run_layers(x_prefix, P, self.reflex_exit_layer + 1, update_stats=update_stats)
        xl, _ = self._run_layers(xr, self.reflex_exit_layer + 1, self.limbic_exit_layer + 1, update_stats=update_stats)
        xc, _ = self._run_layers(xl, self.limbic_exit_layer + 1, self.num_layers, update_stats=update_stats)
        return xr, xl, xc, route_logits

    def forward_all_exits(self, input_ids, update_stats=False):
        xr, xl, xc, route_logits = self.forward_hidden_all_exits(input_ids, update_stats)
        return self._head(xr, 0), self._head(xl, 1), self._head(xc, 2), route_logits

    def forward_loss(self, input_ids, labels, force_depth: int = 2, ignore_index: int = -100,
                     n_valid: Optional[int] = None, return_route: bool = False):
        """Mean next-token CE at one exit through the fused head + CE op (labels already shifted).

        With ``return_route`` the depth router is evaluated on the prefix output of the same pass and
        ``(loss, route_logits, balance_loss)`` is returned; the route logits keep their graph, so a router loss
        added by the caller trains the router and the prefix layers (the ``dynamic`` training mode)."""
        x = ops.embedding(input_ids, self.token_embed.weight)
        end = self.exit_layers[force_depth] + 1
        route_logits = bal = None
        if return_route:
            P = min(self.router_prefix_layers, end)
            xp, _ = self._run_layers(x, 0, P)
            route_logits, _, choice, bal = self._route(xp, None, x.shape[0], x.device)
            self.last_route_logits, self.last_depth_choice, self.last_balance_loss = (
                route_logits.detach(), choice.detach(), bal)
            h, _ = self._run_layers(xp, P, end)
        else:
            h, _ = self._run_layers(x, 0, end)
        norm, head = self._head_modules(force_depth)
        loss = ops.linear_cross_entropy(norm(h), head.weight, labels, bias=head.bias, ignore_index=ignore_index,
                                        n_valid=n_valid)
        if return_route:
            return loss, route_logits, bal
        return loss

    def exit_losses(self, input_ids, labels, ignore_index: int = -100, n_valid: Optional[int] = None,
                    update_stats: bool = True):
        """CE at all three exits (joint training mode) without materialising any [N, V] logits."""
        xr, xl, xc, route_logits = self.forward_hidden_all_exits(input_ids, update_stats)
        losses = []
        for d, h in enumerate((xr, xl, xc)):
            norm, head = self._head_modules(d)
            losses.append(ops.linear_cross_entropy(norm(h), head.weight, labels, bias=head.bias,
                                                   ignore_index=ignore_index, n_valid=n_valid))
        return losses, route_logits

    def distill_exit_heads(self, calibration_ids: torch.Tensor, steps: int = 50, lr: float = 3e-3, batch_size: int = 7,
                           weight_decay: float = 0.01) -> dict:
        """KL self-distillation of the Reflex/Limbic exit norms+heads toward the frozen Cortex predictions."""
        was_training = self.training
        flags = [(p, p.requires_grad) for p in self.parameters()]
        exit_params = []
        for idx in (self.reflex_exit_layer, self.limbic_exit_layer):
            blk = self.layers[idx]
            exit_params += list(blk.exit_norm.parameters()) + list(blk.exit_head.parameters())
        if not exit_params or steps <= 0 or calibration_ids.numel() == 0:
            return {"steps": 0, "initial_kl_loss": 0.0, "final_kl_loss": 0.0}
        try:
            for p in self.parameters():
                p.requires_grad_(False)
            for p in exit_params:
                p.requires_grad_(True)
            dev = next(self.parameters()).device
            batches = list(calibration_ids.to(dev).split(max(1, int(batch_size))))
            self.eval()
            torch.manual_seed(42)
            opt = torch.optim.AdamW(exit_params, lr=lr, weight_decay=weight_decay)
            init = None
            final = 0.0
            for _ in range(steps):
                tot = 0.0
                for b in batches:
                    opt.zero_grad()
                    with torch.no_grad():
                        xr, xl, xc, _ = self.forward_hidden_all_exits(b, update_stats=False)
                        pc = F.softmax(self._head(xc, 2).float().reshape(-1, self.final_head.out_features), dim=-1)
                    loss = 0.0
                    for d, h in ((0, xr), (1, xl)):
                        norm, head = self._head_modules(d)
                        lg = F.linear(norm(h.detach()).float(), head.weight.float(), head.bias.float())
                        loss = loss + F.kl_div(F.log_softmax(lg.reshape(-1, lg.shape[-1]), dim=-1), pc, reduction="batchmean")
                    loss.backward()
                    opt.step()
                    tot += float(loss.detach())
                avg = tot / max(1, len(batches))
                init = avg if init is None else init
                final = avg
            return {"steps": int(steps), "initial_kl_loss": round(init or 0.0, 4), "final_kl_loss": round(final, 4)}
        finally:
            for p, f in flags:
                p.requires_grad_(f)
            self.train(was_training)

    def num_parameters(self) -> int:
        seen, n = set(), 0
        for p in self.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += p.numel()
        return n
