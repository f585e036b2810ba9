"""Tensor parallelism for the dense model family (``UniversalDenseTransformer``) with sequence-parallel activations.

Layout (the Megatron sequence-parallel scheme, with the collectives fused into the GEMMs of
:mod:`triune_b200.parallel.tensor_parallel`):

* between blocks every rank holds a contiguous slice of the ``B*T`` token rows, ``[M / tp, d]``: norms, residual
  adds, the final norm and the LM head + cross entropy run on the local rows only;
* the fused q/k/v/gate (and beta) projection and the FFN gate/up projection are column parallel: the all-gather of
  the row shards happens inside the GEMM (``ag_gemm``), each rank gets all ``M`` rows of ITS heads / hidden slice,
  which is exactly what the linear-attention scan needs (whole sequences, a subset of heads);
* the attention output projection and the FFN down projection are row parallel: the partial sums are
  reduce-scattered back to row shards inside the GEMM epilogue (``gemm_rs``).

Embeddings, norm weights and the LM head are replicated; their gradients are partial (each rank saw its rows) and are
summed over the group by :meth:`TensorParallelDense.allreduce_replicated_grads`. The reference has no tensor
parallelism (its ``UniversalDenseTransformer``, ``triune/universal.py:200-420``, runs replicated under DDP).
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .. import _ext, ops
from ..models.attention import VectorisedGLA
from ..models.universal import SwiGLUFFN, UniversalBlock, UniversalDenseTransformer
from ..ops import gla_cuda
from .tensor_parallel import TPContext, _ColumnParallelFn, _RowParallelFn


def _own(t: torch.Tensor, tp: TPContext) -> nn.Parameter:
    return nn.Parameter(t.detach().clone().contiguous().to(tp.device))


class TPBlock(nn.Module):
    """One ``UniversalBlock`` with its projections sharded over the tensor-parallel group."""

    def __init__(self, block: UniversalBlock, tp: TPContext):
        super().__init__()
        attn = block.attn
        if not isinstance(attn, VectorisedGLA):
            raise NotImplementedError("tensor parallelism covers the GLA / Gated DeltaNet mixers")
        w, r = tp.world, tp.rank
        H, D, d = attn.heads, attn.head_dim, attn.dim
        if H % w != 0:
            raise ValueError(f"{H} heads cannot be split over {w} ranks")
        self.tp, self.heads_local, self.head_dim, self.dim = tp, H // w, D, d
        self.use_delta_rule, self.use_rope = attn.use_delta_rule, attn.use_rope
        self.rope = attn.rope if attn.use_rope else None
        h0, h1 = r * self.heads_local, (r + 1) * self.heads_local
        qkvg = attn.qkvg_weight.detach().view(4, H, D, d)[:, h0:h1].reshape(4 * self.heads_local * D, d)
        self.has_beta = attn.beta_proj is not None
        if self.has_beta:  # per-head write strengths ride along as extra output columns of the same GEMM
            qkvg = torch.cat((qkvg, attn.beta_proj.weight.detach()[h0:h1]), dim=0)
        self.pad_cols = (-qkvg.shape[0]) % 8  # the GEMM kernels want output widths that are multiples of 8
        if self.pad_cols:
            qkvg = torch.cat((qkvg, qkvg.new_zeros(self.pad_cols, d)), dim=0)
        self.qkvg_weight = _own(qkvg, tp)
        self.out_weight = _own(attn.out_proj.weight.detach().view(d, H, D)[:, h0:h1].reshape(d, self.heads_local * D), tp)
        mlp = block.mlp
        self.swiglu = isinstance(mlp, SwiGLUFFN)
        if self.swiglu:
            hid = mlp.hidden
            if hid % w != 0:
                raise ValueError(f"FFN width {hid} cannot be split over {w} ranks")
            self.hidden_local = hid // w
            s0, s1 = r * self.hidden_local, (r + 1) * self.hidden_local
            self.up_weight = _own(mlp.gate_up.detach().view(2, hid, d)[:, s0:s1].reshape(2 * self.hidden_local, d), tp)
            self.down_weight = _own(mlp.down.weight.detach()[:, s0:s1], tp)
            self.up_bias = self.down_bias = None
        else:  # Linear -> GELU -> Linear
            hid = mlp[0].out_features
            if hid % w != 0:
                raise ValueError(f"FFN width {hid} cannot be split over {w} ranks")
            self.hidden_local = hid // w
            s0, s1 = r * self.hidden_local, (r + 1) * self.hidden_local
            self.up_weight = _own(mlp[0].weight.detach()[s0:s1], tp)
            self.up_bias = _own(mlp[0].bias.detach()[s0:s1], tp)
            self.down_weight = _own(mlp[2].weight.detach()[:, s0:s1], tp)
            self.down_bias = _own(mlp[2].bias.detach(), tp)  # replicated: added once, on the reduced rows
        self.input_norm, self.post_attn_norm = block.input_norm, block.post_attn_norm

    # ------------------------------------------------------------------ rank-local checkpoints
    def checkpoint_pieces(self, prefix: str):
        """This rank's slices under the unsharded model's state-dict keys, as views of the live parameters:
        ``(key, dim, start, stop, full, tensor)`` (``trainer/sharded_checkpoint.py``)."""
        w, r = self.tp.world, self.tp.rank
        Hl, D = self.heads_local, self.head_dim
        H = Hl * w
        hd = Hl * D
        for j, name in enumerate(("q_proj", "k_proj", "v_proj", "g_proj")):
            yield (f"{prefix}attn.{name}.weight", 0, r * hd, (r + 1) * hd, H * D, self.qkvg_weight[j * hd : (j + 1) * hd])
        if self.has_beta:
            yield (f"{prefix}attn.beta_proj.weight", 0, r * Hl, (r + 1) * Hl, H, self.qkvg_weight[4 * hd : 4 * hd + Hl])
        yield (f"{prefix}attn.out_proj.weight", 1, r * hd, (r + 1) * hd, H * D, self.out_weight)
        hl = self.hidden_local
        s0, s1, hid = r * hl, (r + 1) * hl, hl * w
        if self.swiglu:
            yield (f"{prefix}mlp.gate_proj.weight", 0, s0, s1, hid, self.up_weight[:hl])
            yield (f"{prefix}mlp.up_proj.weight", 0, s0, s1, hid, self.up_weight[hl:])
            yield (f"{prefix}mlp.down_proj.weight", 1, s0, s1, hid, self.down_weight)
        else:
            yield (f"{prefix}mlp.0.weight", 0, s0, s1, hid, self.up_weight)
            yield (f"{prefix}mlp.0.bias", 0, s0, s1, hid, self.up_bias)
            yield (f"{prefix}mlp.2.weight", 1, s0, s1, hid, self.down_weight)

    def checkpoint_replicated(self, prefix: str):
        out = {}
        for name in ("input_norm", "post_attn_norm"):
            for k, v in getattr(self, name).state_dict().items():
                out[f"{prefix}{name}.{k}"] = v
        if not self.swiglu:
            out[f"{prefix}mlp.2.bias"] = self.down_bias
        return out

    def _mix(self, proj: torch.Tensor, B: int, T: int) -> torch.Tensor:
        """Linear-attention scan over whole sequences for this rank's heads. proj: [B*T, 4*Hl*D (+Hl)(+pad)]."""
        Hl, D = self.heads_local, self.head_dim
        width = 4 * Hl * D
        qkvg = proj if proj.shape[1] == width else proj[:, :width].contiguous()
        cos = sin = None
        if self.use_rope:
            cos, sin = self.rope(T, proj.device, offset=0)
        if not self.use_delta_rule and gla_cuda.core_supported(qkvg, T, D):
            out, _ = gla_cuda.gla_attention_core(qkvg, cos, sin, None, B, T, Hl)
            return out
        q, k, v, g = ops.qk_feature_map(qkvg, cos, sin, B, T, Hl, D)
        if self.use_delta_rule:
            beta = torch.sigmoid(proj[:, width : width + Hl].float()).view(B, T, Hl) if self.has_beta else None
            out, _ = ops.gated_deltanet(q, k, v, g, beta=beta, gate_logits=True)
        else:
            out, _ = ops.gla(q, k, v, g, gate_logits=True)
        return out.reshape(B * T, Hl * D).to(proj.dtype)

    def forward(self, x_s: torch.Tensor, B: int, T: int) -> torch.Tensor:
        tp = self.tp
        proj = _ColumnParallelFn.apply(self.input_norm(x_s), self.qkvg_weight, tp)       # all-gather -> GEMM
        a_s = _RowParallelFn.apply(self._mix(proj, B, T), self.out_weight, tp)            # GEMM -> reduce-scatter
        n, x_s = self.post_attn_norm.forward_add(a_s, x_s)
        up = _ColumnParallelFn.apply(n, self.up_weight, tp)
        if self.swiglu:
            h = ops.swiglu(up[:, : self.hidden_local], up[:, self.hidden_local :])
        else:
            h = ops.gelu_tanh(up + self.up_bias)
        m_s = _RowParallelFn.apply(h.contiguous(), self.down_weight, tp)
        if self.down_bias is not None:
            m_s = m_s + self.down_bias
        return x_s + m_s


class TensorParallelDense(nn.Module):
    """A ``UniversalDenseTransformer`` whose blocks are sharded over ``tp``; every rank of the group must feed the same
    batch. Build the full model identically on every rank (same seed or a broadcast), then wrap it::

        tp = TPContext(mode="fused")                     # or "nccl": library collectives around plain GEMMs
        model = TensorParallelDense(UniversalDenseTransformer.from_config(cfg).to(dev, torch.bfloat16), tp)
        loss = model.forward_loss(ids[:, :-1], ids[:, 1:])   # this rank's share of the mean loss
        loss.backward(); model.allreduce_replicated_grads(); optimizer.step()
        total = model.reduce_loss(loss)                  # the mean loss over all tokens, for logging
    """

    def __init__(self, model: UniversalDenseTransformer, tp: TPContext):
        super().__init__()
        self.tp, self.cfg = tp, model.cfg
        self.embed_tokens, self.norm, self.lm_head = model.embed_tokens, model.norm, model.lm_head
        self.layers = nn.ModuleList([TPBlock(b, tp) for b in model.layers])
        self.vocab_size, self.hidden_dim, self.num_layers = model.vocab_size, model.hidden_dim, model.num_layers

    # ------------------------------------------------------------------ parameters by role
    def replicated_parameters(self) -> List[nn.Parameter]:
        seen, out = set(), []
        mods = [self.embed_tokens, self.norm, self.lm_head] + [m for b in self.layers for m in (b.input_norm, b.post_attn_norm)]
        for m in mods:
            for p in m.parameters():
                if id(p) not in seen:
                    seen.add(id(p))
                    out.append(p)
        for b in self.layers:
            if b.down_bias is not None:
                out.append(b.down_bias)
        return out

    def _rows(self, M: int):
        w, r = self.tp.world, self.tp.rank
        if M % w != 0:
            raise ValueError(f"{M} token rows cannot be split over {w} ranks")
        n = M // w
        return r * n, (r + 1) * n

    # ------------------------------------------------------------------ forward
    def hidden_rows(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Final-norm hidden states of this rank's token rows, ``[B*T / tp, d]``."""
        B, T = input_ids.shape
        lo, hi = self._rows(B * T)
        x_s = self.embed_tokens(input_ids.reshape(-1)[lo:hi])
        for blk in self.layers:
            x_s = blk(x_s, B, T)
        return self.norm(x_s)

    def forward_loss(self, input_ids, labels, force_depth: int = 2, ignore_index: int = -100, n_valid: Optional[int] = None):
        """This rank's share of the mean cross entropy: the shares of the group add up to the loss of the whole batch."""
        B, T = input_ids.shape
        lo, hi = self._rows(B * T)
        h_s = self.hidden_rows(input_ids)
        y_s = labels.reshape(-1)[lo:hi]
        if n_valid is None:
            n_valid = max(1, int((labels != ignore_index).sum().item()))
        w = self.lm_head.weight
        if _ext.use_kernels(h_s, w) and h_s.dtype == torch.bfloat16 and w.shape[0] % 8 == 0:
            return ops.linear_cross_entropy(h_s, w, y_s, ignore_index=ignore_index, n_valid=n_valid)
        logits = F.linear(h_s.float(), w.float())
        return F.cross_entropy(logits, y_s, ignore_index=ignore_index, reduction="sum") / n_valid

    def forward(self, input_ids, **_):
        """Logits of this rank's token rows, ``[B*T / tp, vocab]``."""
        return ops.linear(self.hidden_rows(input_ids), self.lm_head.weight)

    # ------------------------------------------------------------------ collectives around the step
    @torch.no_grad()
    def reduce_loss(self, loss: torch.Tensor) -> torch.Tensor:
        total = loss.detach().float().clone()
        if self.tp.world > 1:
            dist.all_reduce(total, group=self.tp.group)
        return total

    @torch.no_grad()
    def allreduce_replicated_grads(self) -> None:
        """Sum the partial gradients of the replicated parameters (each rank back-propagated its own rows)."""
        if self.tp.world == 1:
            return
        grads = []
        for p in self.replicated_parameters():
            g = getattr(p, "main_grad", None)
            g = g if g is not None else p.grad
            if g is not None:
                grads.append(g)
        if not grads:
            return
        flat = torch.cat([g.reshape(-1).float() for g in grads])
        dist.all_reduce(flat, group=self.tp.group)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off : off + n].view_as(g).to(g.dtype))
            off += n


def make_tp_dp_groups(tp_size: int):
    """Split the world into tensor-parallel groups of ``tp_size`` consecutive ranks and the data-parallel groups across
    them (ranks with the same position inside their tensor-parallel group). Every rank must call this. Returns
    ``(tp_group, dp_group)`` of the calling rank."""
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % tp_size != 0:
        raise ValueError(f"world size {world} is not a multiple of the tensor-parallel size {tp_size}")
    tp_group = dp_group = None
    for start in range(0, world, tp_size):
        ranks = list(range(start, start + tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            tp_group = g
    for pos in range(tp_size):
        ranks = list(range(pos, world, tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            dp_group = g
    return tp_group, dp_group


@torch.no_grad()
def average_grads_over_replicas(model: nn.Module, dp_group) -> None:
    """Data parallelism on top of tensor parallelism: average every gradient over the replicas that hold the same shard
    (one flat all-reduce). Call after ``allreduce_replicated_grads``."""
    n = dist.get_world_size(dp_group)
    if n == 1:
        return
    grads = []
    for p in model.parameters():
        g = getattr(p, "main_grad", None)
        g = g if g is not None else p.grad
        if g is not None:
            grads.append(g)
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=dp_group)
    flat.div_(n)
    off = 0
    for g in grads:
        k = g.numel()
        g.copy_(flat[off : off + k].view_as(g).to(g.dtype))
        off += k


def tensor_parallelize(model: UniversalDenseTransformer, tp: TPContext) -> TensorParallelDense:
    return TensorParallelDense(model, tp)
