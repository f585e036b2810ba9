"""Fused data-parallel optimizer step over NVLink (no NCCL on the path).

Layout: the optimizer's parameter arena (bf16) and gradient arena (fp32) live in one symmetric buffer, so every
rank can read every peer's gradients and write every peer's parameters from inside a kernel.

One step =
  1. ``dp_reduce_scatter``   each rank pulls, for the element ranges it owns (its AdamW shard, its Muon matrices,
                             its experts), the gradients of all ranks (peer loads or one ``multimem.ld_reduce``),
                             scales by 1/world, accumulates the grad-norm partial and publishes it to all peers;
  2. ``dp_adamw_allgather``  waits for all partials, derives the global clip coefficient, applies AdamW to the
                             owned shard and stores the new bf16 weights straight into every peer's arena;
  3. Muon / CentroidSteer    run on the owned matrices only (Newton-Schulz on the tcgen05 GEMM), then
     ``dp_broadcast_ranges`` pushes the updated bf16 ranges to all peers;
  4. ``comm_barrier``        nobody starts the next forward before every owner's stores have landed.

Ownership is whole-matrix for the matrix tiers (Newton-Schulz and the subspace projections need entire matrices)
and flat for the AdamW tier. Reference baseline: DDP all-reduce + full update on every rank
(``triune/trainer/distributed.py:142-156``).
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist

from .. import _ext, ops
from ..profiling import nvtx_range
from .symm import SymmetricBuffer

CH_PARAMS_DONE = 2
CH_STATS = 7
STATS_MAX = 1 << 16  # floats of routing statistics the symmetric buffer has room for, per rank


class SymmetricArenaStorage:
    """``storage_factory`` for :class:`ParamArena` that places both arenas in a :class:`SymmetricBuffer`."""

    def __init__(self, ctx, use_multimem=None, group=None):
        """``use_multimem``: ``None`` (default) = plain peer loads and stores. With four loads in flight per thread they
        match the in-switch reduction at 8 ranks (0.57 against 0.58 ms for 96 M parameters) and beat it at 2 (0.34 against
        0.64 ms), and a rank that dies while bound to a multicast object can fault its peers' GPUs; ``True`` asks for
        ``multimem`` where the heap reports multicast support."""
        self.ctx = ctx
        self.group = group
        self.use_multimem = False if use_multimem is None else bool(use_multimem)
        self.buffer = None
        self.total = 0

    def __call__(self, total: int, dtype: torch.dtype, device: torch.device):
        assert dtype == torch.bfloat16, "the fused data-parallel step needs bf16 parameters"
        w = self.ctx.world_size
        self.total = total
        self.buffer = SymmetricBuffer(
            {"param": total * 2, "grad": total * 4, "norm": 2 * w * 4 + 64, "metric": 16 * w * 4,
             "stats": STATS_MAX * w * 4},
            device, group=self.group, use_multimem=self.use_multimem)
        return self.buffer.view("param", torch.bfloat16, total), self.buffer.view("grad", torch.float32, total)


class FusedDPUpdater:
    def __init__(self, ctx, optimizer, storage: SymmetricArenaStorage):
        # Every device-side wait of the step gives up after one second (``WAIT_LIMIT_NS`` in ``csrc/common/ptx.cuh``,
        # a compile-time constant) and records why in ``self.status``; read it with :meth:`check`.
        self.ctx, self.opt, self.buf = ctx, optimizer, storage.buffer
        if self.buf is None:
            raise RuntimeError("optimizer was not built with SymmetricArenaStorage as storage_factory")
        a = optimizer.arena
        if a.flat_master is None:
            raise RuntimeError("fused data parallelism expects bf16 parameters with fp32 masters")
        optimizer.shard = (ctx.rank, ctx.world_size)
        dev = a.device
        self.counter = torch.zeros(1, device=dev, dtype=torch.int32)
        self.status = torch.zeros(1, device=dev, dtype=torch.int32)
        self.norm_out = torch.zeros(1, device=dev, dtype=torch.float32)
        b, e = optimizer.owned_adamw_range()
        self.adamw_owned = (b, e)
        self.matrix_ranges: List[Tuple[int, int]] = optimizer.owned_matrix_ranges()
        flat: List[int] = [b, e] if e > b else []
        for r in self.matrix_ranges:
            flat += [r[0], r[1]]
        self.owned_flat = flat
        self.bcast_flat = [x for r in self.matrix_ranges for x in r]
        # The epoch of the three step channels lives on the device and is bumped by the step itself, so a captured
        # step can be replayed; every rank runs the same sequence of steps, so the counters stay equal.
        self.epoch_dev = torch.zeros(1, device=dev, dtype=torch.int32)
        owned = sum(flat[i + 1] - flat[i] for i in range(0, len(flat), 2))
        self.bytes_per_step = owned * 4 * (ctx.world_size - 1) + owned * 2 * (ctx.world_size - 1)
        self.steps = 0

    @property
    def comm_bytes(self) -> int:
        return self.bytes_per_step * self.opt.step_count

    def _sync_routing_statistics(self, e, rank, world, bufs, sigs) -> None:
        """Average the routing statistics that feed the update rule (expert centroids of the steering tier, pending
        selection-bias updates, load ratios) over the ranks with one small peer-store all-reduce, so every replica
        applies the step of the global batch. Same tensors as ``ShardedDataParallel._sync_routing_statistics``."""
        model = getattr(self.opt, "model", None)
        if model is None:
            return
        tensors = []
        for m in model.modules():
            if not hasattr(m, "expert_bias"):
                continue
            for name in ("last_centroids", "expert_load_ratio", "_pending_bias_update"):
                t = getattr(m, name, None)
                if torch.is_tensor(t) and t.is_floating_point() and t.is_cuda:
                    tensors.append(t)
        n = sum(t.numel() for t in tensors)
        if n == 0 or n > STATS_MAX:
            return
        flat = torch.cat([t.detach().float().reshape(-1) for t in tensors])
        red = torch.empty_like(flat)
        e.metric_allreduce(rank, world, bufs, sigs, self.buf.offset("stats"), flat, red, CH_STATS, 0, self.status,
                           self.epoch_dev)
        ops._tick()
        red.mul_(1.0 / world)
        off = 0
        for t in tensors:
            k = t.numel()
            t.copy_(red[off : off + k].view(t.shape).to(t.dtype))
            off += k

    def step(self, mark=None):
        """One data-parallel optimizer step. ``mark(name)`` (optional) is called after each phase, on the launching
        stream, so a benchmark can record CUDA events between the kernels."""
        mark = mark or (lambda name: None)
        opt, buf = self.opt, self.buf
        a = opt.arena
        e = _ext.ext()
        rank, world, bufs, sigs, mc = buf.table()
        ep = 0
        self.epoch_dev.add_(1)
        if world > 1:
            self._sync_routing_statistics(e, rank, world, bufs, sigs)
        hyper = opt.hyper if getattr(opt, "capturable", False) else None
        opt.step_count += 1
        goff, noff, poff = buf.offset("grad"), buf.offset("norm"), buf.offset("param")
        dp_range = nvtx_range("dp_reduce_scatter_update_allgather")
        dp_range.__enter__()
        e.dp_reduce_scatter(rank, world, bufs, sigs, mc, goff, noff, self.owned_flat, ep, buf.use_multimem, self.counter,
                            self.status, self.epoch_dev)
        mark("reduce_scatter")
        lo, hi = a.adamw_range
        b1, b2 = opt.betas
        clip = float(opt.grad_clip) if opt.grad_clip else 0.0
        ob, oe = self.adamw_owned
        e.dp_adamw_allgather(rank, world, bufs, sigs, mc, goff, noff, poff, ob, oe, lo, a.master()[lo:hi], opt.exp_avg,
                             opt.exp_avg_sq, opt.lr, b1, b2, opt.eps, opt.weight_decay, opt.step_count, clip,
                             opt._clip_coef, self.norm_out, ep, buf.use_multimem, self.status, self.epoch_dev, hyper)
        ops._tick(2)
        dp_range.__exit__(None, None, None)
        mark("adamw_allgather")
        opt.last_grad_norm = self.norm_out
        opt._step_muon()
        opt._step_steer()
        mark("matrix_tiers")
        if self.bcast_flat:
            e.dp_broadcast_ranges(rank, world, bufs, sigs, mc, poff, self.bcast_flat, buf.use_multimem)
            ops._tick()
        e.comm_barrier(rank, world, bufs, sigs, CH_PARAMS_DONE, ep, self.status, self.epoch_dev)
        ops._tick()
        mark("broadcast_barrier")
        self.steps += 1

    def audit(self) -> Dict[int, bool]:
        """Every step channel's flags from every peer stand at the device-resident epoch: no signal is outstanding and no
        rank is a step ahead or behind. Synchronises."""
        ep = int(self.epoch_dev.item())
        chans = {0: ep, 1: ep, CH_PARAMS_DONE: ep}
        return self.buf.audit_signals(chans)

    def check(self) -> int:
        """Status word of the bounded waits (0 = every wait completed). Synchronises."""
        return int(self.status.item())

    def raise_if_failed(self) -> None:
        """Raise :class:`~triune_b200.parallel.elastic.CollectiveTimeout` when a bounded device-side wait ran out
        (a peer did not arrive); the CUDA context stays usable. Synchronises."""
        from .elastic import raise_on_status

        raise_on_status(self.check(), "fused data-parallel reduction")
