"""Pipeline parallelism for both model families: contiguous layer ranges per rank, one-forward-one-backward schedule.

Rank ``s`` of the pipeline group keeps the blocks ``[lo_s, hi_s)`` of a :class:`UniversalDenseTransformer`
(:class:`PipelineStage`) or of the multi-exit MoE ``TriuneTransformer`` trained at full depth
(:class:`TriunePipelineStage`, whose tied embedding / head weight lives on both end stages with summed gradients); the
first stage also keeps the token embedding, the last one the final norm and the vocabulary head (fused with the cross
entropy). A step splits the batch into ``micro_batches`` equal micro-batches and runs the classic 1F1B order:

    stage s:  (S - s - 1) warm-up forwards | steady pairs of one forward and one backward | the same number of backwards

so at most ``S - s`` micro-batches of activations are alive on a stage, whatever the number of micro-batches. Only the
``[b, T, d]`` boundary activation (forward) and its gradient (backward) cross between neighbours. In the steady phase
the send of one direction and the receive of the other are issued as ONE batched point-to-point group, which is what
keeps a rendezvous transport (NCCL send / recv kernels on one stream) from deadlocking: neither neighbour ever waits in
a send while the other waits in a send.

The schedule itself (:func:`one_f_one_b`) is plain data, testable without any process group. The point-to-point
traffic goes through ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on CPU); nothing here reads a peer's memory
directly. The reference has no pipeline parallelism (its model runs on one device, ``triune/model/transformer.py``).
"""

from __future__ import annotations

from collections import deque
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops


def split_layers(num_layers: int, stages: int, weights: Optional[Sequence[float]] = None) -> List[Tuple[int, int]]:
    """Contiguous ``[lo, hi)`` layer ranges, one per stage, as even as possible (earlier stages take the remainder).

    ``weights`` (one cost per stage, default all 1) shifts layers away from a stage that carries extra work: the last
    stage also runs the vocabulary head, so ``weights=[1, 1, 1, 1.5]`` gives it fewer blocks.
    """
    if stages < 1 or num_layers < stages:
        raise ValueError(f"cannot split {num_layers} layers over {stages} stages")
    if weights is None:
        base, rem = divmod(num_layers, stages)
        sizes = [base + (1 if s < rem else 0) for s in range(stages)]
    else:
        if len(weights) != stages or min(weights) <= 0:
            raise ValueError("weights: one positive cost per stage")
        inv = [1.0 / w for w in weights]
        ideal = [num_layers * x / sum(inv) for x in inv]
        sizes = [max(1, int(x)) for x in ideal]
        # hand the layers lost to rounding to the stages that were rounded down the most
        order = sorted(range(stages), key=lambda s: ideal[s] - sizes[s], reverse=True)
        i = 0
        while sum(sizes) < num_layers:
            sizes[order[i % stages]] += 1
            i += 1
        while sum(sizes) > num_layers:
            j = max(range(stages), key=lambda s: sizes[s])
            sizes[j] -= 1
    out, lo = [], 0
    for n in sizes:
        out.append((lo, lo + n))
        lo += n
    return out


def one_f_one_b(stage: int, stages: int, micro_batches: int) -> List[Tuple[str, int]]:
    """The order of work of one stage: a list of ``("F", i)`` / ``("B", i)`` over micro-batch indices."""
    warm = min(stages - stage - 1, micro_batches)
    steps: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < micro_batches:
        steps.append(("F", f))
        steps.append(("B", b))
        f += 1
        b += 1
    while b < micro_batches:
        steps.append(("B", b))
        b += 1
    return steps


def peak_live_micro_batches(stage: int, stages: int, micro_batches: int) -> int:
    """How many micro-batches of activations a stage holds at most under :func:`one_f_one_b`."""
    live = peak = 0
    for kind, _ in one_f_one_b(stage, stages, micro_batches):
        live += 1 if kind == "F" else -1
        peak = max(peak, live)
    return peak


class PipelineStage(nn.Module):
    """The part of a :class:`UniversalDenseTransformer` that one pipeline rank keeps.

    Built from the full model (every rank constructs the same one with the same seed, or loads the same checkpoint) and
    keeps references to its own blocks only, so the rest can be freed by dropping the full model.
    """

    def __init__(self, full: nn.Module, stage: int, stages: int, bounds: Optional[List[Tuple[int, int]]] = None):
        super().__init__()
        if stages > 1 and getattr(full.cfg, "tie_embeddings", False):
            raise ValueError("pipeline parallelism needs untied embeddings: the table and the head live on different ranks")
        self.cfg = full.cfg
        self.hidden_dim = full.cfg.hidden_dim
        self.stage, self.stages = stage, stages
        self.bounds = bounds if bounds is not None else split_layers(len(full.layers), stages)
        lo, hi = self.bounds[stage]
        self.layer_range = (lo, hi)
        self.layers = nn.ModuleList([full.layers[i] for i in range(lo, hi)])
        self.is_first, self.is_last = stage == 0, stage == stages - 1
        self.embed_tokens = full.embed_tokens if self.is_first else None
        self.norm = full.norm if self.is_last else None
        self.lm_head = full.lm_head if self.is_last else None

    def full_names(self):
        """``(name in the full model, parameter)`` pairs of this stage, for checkpoints and comparisons."""
        lo, _ = self.layer_range
        for name, p in self.named_parameters():
            if name.startswith("layers."):
                _, idx, rest = name.split(".", 2)
                yield f"layers.{lo + int(idx)}.{rest}", p
            else:
                yield name, p

    def run_blocks(self, x: torch.Tensor) -> torch.Tensor:
        for layer in self.layers:
            x, _ = layer(x, cache=None)
        return x

    def forward(self, x: torch.Tensor, labels: Optional[torch.Tensor] = None, n_valid: Optional[int] = None):
        """``x``: token ids on the first stage, the previous stage's activation elsewhere. Returns the boundary
        activation, or on the last stage the mean cross entropy of this micro-batch."""
        if self.is_first:
            x = self.embed_tokens(x)
        x = self.run_blocks(x)
        if not self.is_last:
            return x
        return ops.linear_cross_entropy(self.norm(x), self.lm_head.weight, labels, n_valid=n_valid)


class TriunePipelineStage(nn.Module):
    """One pipeline rank's part of the multi-exit MoE :class:`TriuneTransformer`, trained at full depth.

    The stage keeps the model object (its layer-running helpers, routing statistics and exit bookkeeping stay in one
    place) but replaces every block outside ``[lo, hi)`` by an empty module, drops the token embedding on all but the
    first stage and the final norm / head on all but the last, so only this stage's weights stay allocated. The loss is
    the full-depth one (``force_depth=2``); early-exit heads that live on this stage's blocks keep their weights and
    receive no gradient from this loss, exactly as in single-device full-depth training. The tied embedding / head
    weight exists on the first and on the last stage; see ``tied_weight``.
    """

    def __init__(self, full: nn.Module, stage: int, stages: int, bounds: Optional[List[Tuple[int, int]]] = None,
                 update_stats: bool = True):
        super().__init__()
        self.stage, self.stages = stage, stages
        self.hidden_dim = full.hidden_dim
        self.bounds = bounds if bounds is not None else split_layers(len(full.layers), stages)
        lo, hi = self.bounds[stage]
        self.layer_range = (lo, hi)
        self.is_first, self.is_last = stage == 0, stage == stages - 1
        self.update_stats = update_stats
        tied = getattr(full, "final_head", None) is not None and full.final_head.weight is full.token_embed.weight
        for i in range(len(full.layers)):
            if not lo <= i < hi:
                full.layers[i] = nn.Identity()
        if not self.is_first and not (self.is_last and tied):
            full.token_embed = None  # (a tied last stage keeps the module: same tensor as the head, same parameter name)
        if not self.is_last:
            full.final_norm, full.final_head = None, None
        if not self.is_first and getattr(full, "router", None) is not None:
            full.router = None  # the depth router reads the prefix layers, which live on the first stage
        # The table and the head are one tensor in this family. On two different ranks they become two copies that
        # start equal and stay equal because the engine sums their gradients after every step (both then take the
        # same update, under the same parameter name and therefore the same optimizer tier).
        self.tied_weight = full.token_embed.weight if tied and stages > 1 and (self.is_first or self.is_last) else None
        self.model = full

    def full_names(self):
        for name, p in self.model.named_parameters():
            yield name, p

    def forward(self, x: torch.Tensor, labels: Optional[torch.Tensor] = None, n_valid: Optional[int] = None):
        m = self.model
        if self.is_first:
            x = m.token_embed(x)
        lo, hi = self.layer_range
        x, _ = m._run_layers(x, lo, hi, update_stats=self.update_stats)
        if not self.is_last:
            return x
        return ops.linear_cross_entropy(m.final_norm(x), m.final_head.weight, labels, bias=m.final_head.bias, n_valid=n_valid)


class PipelineEngine:
    """Runs training steps of a :class:`PipelineStage` under the 1F1B schedule.

    ``group``: the process group of the pipeline (its ranks in stage order; default: the whole world). Every rank of the
    group calls :meth:`train_step` with the same ``input_ids`` / ``labels`` (only the first and the last stage read
    them). Gradients accumulate in ``.grad`` over the micro-batches, scaled so that the total is the gradient of the
    mean loss over the whole batch.
    """

    def __init__(self, stage_module: nn.Module, micro_batches: int, group=None):
        self.m = stage_module
        self.group = group if group is not None else dist.group.WORLD
        self.stages = dist.get_world_size(self.group)
        self.stage = dist.get_rank(self.group)
        if (self.stage, self.stages) != (stage_module.stage, stage_module.stages):
            raise ValueError("the stage module was built for another position of the pipeline")
        self.micro_batches = int(micro_batches)
        ranks = dist.get_process_group_ranks(self.group)
        self.prev_rank = ranks[self.stage - 1] if self.stage > 0 else None
        self.next_rank = ranks[self.stage + 1] if self.stage + 1 < self.stages else None
        self.first_rank, self.last_rank = ranks[0], ranks[-1]
        self.peak_live = 0

    # ------------------------------------------------------------------ point-to-point
    def _exchange(self, send: Optional[torch.Tensor], send_to: Optional[int], recv_like: Optional[torch.Tensor],
                  recv_from: Optional[int]) -> Optional[torch.Tensor]:
        """One batched group with at most one send and one receive; returns the received tensor."""
        ops_ = []
        if send is not None and send_to is not None:
            ops_.append(dist.P2POp(dist.isend, send.contiguous(), send_to, self.group))
        if recv_like is not None and recv_from is not None:
            ops_.append(dist.P2POp(dist.irecv, recv_like, recv_from, self.group))
        if not ops_:
            return None
        for req in dist.batch_isend_irecv(ops_):
            req.wait()
        return recv_like if recv_from is not None else None

    def _buffer(self, shape, dtype, device):
        return torch.empty(shape, dtype=dtype, device=device)

    # ------------------------------------------------------------------ one step
    def train_step(self, input_ids: torch.Tensor, labels: torch.Tensor, n_valid: Optional[int] = None) -> torch.Tensor:
        """Forward and backward of one batch; returns the mean loss (broadcast from the last stage to every rank).

        ``n_valid``: the number of non-ignored labels of EACH micro-batch when the caller knows it (all of them for
        packed pre-training data); it saves the last stage one host synchronisation per micro-batch. Micro-batches
        are weighted equally, so with ignored labels the result is the mean of the micro-batch means."""
        M, m = self.micro_batches, self.m
        B, T = input_ids.shape
        if B % M != 0:
            raise ValueError(f"batch {B} is not a multiple of the number of micro-batches {M}")
        mb = B // M
        dev = next(m.parameters()).device
        dtype = next(m.parameters()).dtype
        act_shape = (mb, T, m.hidden_dim)
        ids = input_ids.to(dev).split(mb) if m.is_first else None
        tgt = labels.to(dev).split(mb) if m.is_last else None
        live = deque()  # (input activation or None, output) of forwards whose backward is still to come
        loss_sum = torch.zeros((), dtype=torch.float32, device=dev)
        self.peak_live = 0

        def forward(i, x_in):
            if x_in is not None:
                x_in.requires_grad_(True)  # a received buffer: a leaf whose .grad is what goes back
            out = m(ids[i] if m.is_first else x_in, labels=tgt[i] if m.is_last else None, n_valid=n_valid)
            live.append((x_in, out))
            self.peak_live = max(self.peak_live, len(live))
            return out

        def backward(grad_out):
            x_in, out = live.popleft()
            if m.is_last:
                loss_sum.add_(out.detach().float())
                (out / M).backward()
            else:
                torch.autograd.backward(out, grad_tensors=grad_out)
            return None if x_in is None else x_in.grad

        recv_act = lambda: self._exchange(None, None, self._buffer(act_shape, dtype, dev), self.prev_rank)  # noqa: E731
        warm = min(self.stages - self.stage - 1, M)
        steady = M - warm
        for i in range(warm):
            out = forward(i, None if m.is_first else recv_act())
            self._exchange(out.detach(), self.next_rank, None, None)
        x_in = None if (m.is_first or steady == 0) else recv_act()
        for j in range(steady):
            out = forward(warm + j, x_in)
            grad_out = None
            if not m.is_last:  # send the activation forward and receive the gradient of the oldest live micro-batch
                grad_out = self._exchange(out.detach(), self.next_rank, self._buffer(act_shape, dtype, dev), self.next_rank)
            grad_in = backward(grad_out)
            more = j + 1 < steady
            if m.is_first:
                x_in = None
            else:  # send the gradient back; in the same group receive the next activation if one is coming
                x_in = self._exchange(grad_in, self.prev_rank, self._buffer(act_shape, dtype, dev) if more else None,
                                      self.prev_rank if more else None)
        for _ in range(warm):
            grad_out = self._exchange(None, None, self._buffer(act_shape, dtype, dev), self.next_rank)
            grad_in = backward(grad_out)
            if not m.is_first:
                self._exchange(grad_in, self.prev_rank, None, None)
        self._sum_tied_gradients()
        loss = loss_sum / M
        if self.stages > 1:
            dist.broadcast(loss, src=self.last_rank, group=self.group)
        return loss

    @torch.no_grad()
    def eval_loss(self, input_ids: torch.Tensor, labels: torch.Tensor, n_valid: Optional[int] = None) -> torch.Tensor:
        """Forward only (validation): the micro-batches stream through the stages one after another; returns the mean
        loss on every rank. Nothing is kept between micro-batches, so memory is one micro-batch per stage."""
        M, m = self.micro_batches, self.m
        B, T = input_ids.shape
        if B % M != 0:
            raise ValueError(f"batch {B} is not a multiple of the number of micro-batches {M}")
        mb = B // M
        dev, dtype = next(m.parameters()).device, next(m.parameters()).dtype
        ids = input_ids.to(dev).split(mb) if m.is_first else None
        tgt = labels.to(dev).split(mb) if m.is_last else None
        total = torch.zeros((), dtype=torch.float32, device=dev)
        was = m.training
        m.eval()
        try:
            for i in range(M):
                x = ids[i] if m.is_first else self._exchange(None, None, self._buffer((mb, T, m.hidden_dim), dtype, dev), self.prev_rank)
                out = m(x, labels=tgt[i] if m.is_last else None, n_valid=n_valid)
                if m.is_last:
                    total += out.float()
                else:
                    self._exchange(out, self.next_rank, None, None)
        finally:
            m.train(was)
        total = total / M
        if self.stages > 1:
            dist.broadcast(total, src=self.last_rank, group=self.group)
        return total

    def _sum_tied_gradients(self) -> None:
        """First and last stage exchange the gradient of the tied embedding / head weight and add the other's."""
        w = getattr(self.m, "tied_weight", None)
        if w is None or self.stages == 1:
            return
        if w.grad is None:
            w.grad = torch.zeros_like(w)
        other = self.last_rank if self.stage == 0 else self.first_rank
        got = self._exchange(w.grad, other, torch.empty_like(w.grad), other)
        w.grad.add_(got)

    # ------------------------------------------------------------------ helpers around the optimizer
    @torch.no_grad()
    def clip_grad_norm(self, max_norm: float) -> torch.Tensor:
        """Clip by the norm of the WHOLE model's gradient (the squared norms of the stages are summed over the group).
        Returns that norm. Give the per-stage optimizers no clipping of their own when this is used."""
        grads = [p.grad for p in self.m.parameters() if p.grad is not None]
        dev = next(self.m.parameters()).device
        sq = torch.zeros((), dtype=torch.float32, device=dev)
        tied = getattr(self.m, "tied_weight", None)
        for p in self.m.parameters():
            if p.grad is None or (p is tied and self.stage != 0):  # the tied weight counts once, on the first stage
                continue
            sq += p.grad.float().pow(2).sum()
        if self.stages > 1:
            dist.all_reduce(sq, group=self.group)
        norm = sq.sqrt()
        scale = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        for g in grads:
            g.mul_(scale.to(g.dtype))
        return norm


def make_pp_dp_groups(pp_size: int):
    """Pipelines of ``pp_size`` consecutive ranks with data parallelism across them (ranks holding the same stage).
    Every rank must call this. Returns ``(pp_group, dp_group)`` of the calling rank."""
    from .tp_model import make_tp_dp_groups

    return make_tp_dp_groups(pp_size)  # the same partition of the world: blocks of consecutive ranks and their columns


def pipeline_parallelize(full: nn.Module, micro_batches: int, group=None, bounds=None) -> PipelineEngine:
    """Keep this rank's stage of ``full`` and wrap it in an engine. Drop ``full`` afterwards to free the other stages."""
    group = group if group is not None else dist.group.WORLD
    cls = TriunePipelineStage if hasattr(full, "exit_layers") else PipelineStage
    stage = cls(full, dist.get_rank(group), dist.get_world_size(group), bounds)
    return PipelineEngine(stage, micro_batches, group)
