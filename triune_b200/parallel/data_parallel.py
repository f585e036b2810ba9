"""Data parallelism over the flat gradient arena.

The reference only wraps the model in DDP (``triune/trainer/distributed.py:142-156``) and never reaches it from
its trainer. Here gradients live in ONE fp32 buffer (``ParamArena.flat_grad``), so data parallelism is a single
collective over that buffer followed by the tiered update:

* ``mode="nccl"``  baseline: NCCL all-reduce (average) of the flat buffer, every rank applies the full update;
* ``mode="fused"`` product path: one kernel per tier reads every peer's gradient shard over NVLink, averages,
  applies the AdamW / Muon update to the shard it owns and writes the new bf16 parameters into every peer's
  parameter buffer (reduce-scatter + update + all-gather in one launch; see ``parallel/fused_dp.py``).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class _GroupView:
    """rank / world_size of a process sub-group behind the attribute names of ``DistributedContext``."""

    def __init__(self, ctx, group):
        self.group = group
        self.rank, self.world_size = dist.get_rank(group), dist.get_world_size(group)
        self.device, self.local_rank = ctx.device, getattr(ctx, "local_rank", 0)


class ShardedDataParallel:
    def __init__(self, ctx, mode: str = "nccl", use_multimem=None, group=None):
        """``group``: the data-parallel process group when it is not the whole world (replicas of a tensor-parallel
        or pipeline-parallel model: the ranks that hold the same shard)."""
        self.group = group
        if group is not None:
            ctx = _GroupView(ctx, group)
        self.ctx = ctx
        self.mode = mode
        self.optimizer = None
        self.comm_bytes = 0
        self._fused = None
        self.storage_factory = None
        if mode == "fused" and ctx.world_size > 1:
            from .fused_dp import SymmetricArenaStorage

            # pass this to the optimizer (``storage_factory=dp.storage_factory``) so its arenas are peer-visible
            self.storage_factory = SymmetricArenaStorage(ctx, use_multimem=use_multimem, group=group)

    def attach(self, optimizer) -> None:
        self.optimizer = optimizer
        if not hasattr(optimizer, "arena"):
            raise ValueError("ShardedDataParallel needs an arena-based optimizer (CentroidSteerOptimizer)")
        if self.ctx.world_size > 1:
            # identical initial parameters on every rank
            src = 0 if self.group is None else dist.get_global_rank(self.group, 0)
            dist.broadcast(optimizer.arena.flat_param, src=src, group=self.group)
            optimizer.arena.sync_master_from_params()
            for b in optimizer.model.buffers():
                dist.broadcast(b, src=src, group=self.group)
        if self.mode == "fused" and self.ctx.world_size > 1:
            from .fused_dp import FusedDPUpdater

            self._fused = FusedDPUpdater(self.ctx, optimizer, self.storage_factory)
        inner = optimizer.step

        def step(closure=None):
            if self.ctx.world_size > 1:
                optimizer.arena.fold_autograd_grads()
                if self._fused is not None:
                    return self._fused.step()
                g = optimizer.arena.flat_grad
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
                g.mul_(1.0 / self.ctx.world_size)
                self.comm_bytes += g.numel() * 4
                self._sync_routing_statistics()
            return inner(closure)

        optimizer.step = step

    def _sync_routing_statistics(self) -> None:
        """Average the routing statistics that feed the update rule (expert centroids used by the steering tier, the
        pending selection-bias update, the load ratios) so every replica applies the identical step. They are derived
        from each rank's own tokens; without this the replicas' expert weights drift apart."""
        tensors = []
        for m in self.optimizer.model.modules():
            for name in ("last_centroids", "expert_load_ratio", "_pending_bias_update"):
                t = getattr(m, name, None)
                if torch.is_tensor(t) and t.is_floating_point() and hasattr(m, "expert_bias"):
                    tensors.append(t)
        if not tensors:
            return
        flat = torch.cat([t.detach().float().reshape(-1) for t in tensors])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
        flat.mul_(1.0 / self.ctx.world_size)
        off = 0
        for t in tensors:
            n = t.numel()
            t.copy_(flat[off : off + n].view(t.shape).to(t.dtype))
            off += n
        self.comm_bytes += flat.numel() * 4
