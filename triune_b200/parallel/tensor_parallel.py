"""Tensor parallelism with sequence-parallel activations: the two collectives live inside the GEMM kernels.

The reference has no tensor parallelism (its only distributed code is a DDP wrapper,
``triune/trainer/distributed.py:142-156``). Layout (Megatron style): between blocks every rank holds ``M / tp`` rows
of the activations (sequence parallel); a column-parallel linear needs all rows (all-gather), a row-parallel linear
produces partial sums of all rows and each rank keeps its own ``M / tp`` rows of the sum (reduce-scatter).

  * ``allgather_gemm``       Y[M, N/tp] = gather(X)[M, K] @ W[N/tp, K]^T; four copy warps per CTA pull the remote row
                             shards over NVLink into the local gathered buffer while tensor-core tiles of the local
                             shard are already running; a tile of a remote chunk waits on that chunk's flag.
  * ``gemm_reduce_scatter``  Y[M/tp, N] = sum_ranks (X[M, K/tp] @ W[N, K/tp]^T)[own rows]; every output tile is TMA
                             reduce-added from the GEMM epilogue into the buffer of the rank that owns its rows.

Backward passes are the duals (the data gradient of an all-gather GEMM is a GEMM + reduce-scatter and vice versa), and
weight gradients are local GEMMs over the gathered operand that the forward or backward already produced.
``mode="nccl"`` runs the same math with NCCL all-gather / reduce-scatter + the plain GEMM: the measured baseline.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _ext, ops
from .symm import SymmetricBuffer

CH_AG, CH_RS_ZERO, CH_RS_DONE = 3, 4, 5


class TPContext:
    """Per tensor-parallel group: symmetric workspaces (allocated once per shape), epochs, cached tensor-map tables."""

    def __init__(self, group=None, device=None, mode: str = "fused", rs_fp32: bool = False):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.mode = mode if self.world > 1 else "local"
        self.rs_fp32 = rs_fp32
        self._bufs: Dict[Tuple, SymmetricBuffer] = {}
        self._cmaps: Dict[Tuple, torch.Tensor] = {}
        self._flags: Dict[int, torch.Tensor] = {}
        self._epochs: Dict[Tuple, int] = {}
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.comm_bytes = 0

    # ------------------------------------------------------------------ workspaces
    def workspace(self, kind: str, rows: int, cols: int, elem: int) -> SymmetricBuffer:
        key = (kind, rows, cols, elem)
        if key not in self._bufs:  # collective: every rank reaches this with the same key in the same order
            self._bufs[key] = SymmetricBuffer({"a": rows * cols * elem, "b": rows * cols * elem}, self.device, self.group,
                                              use_multimem=False)
        return self._bufs[key]

    def _epoch(self, key) -> int:
        self._epochs[key] = self._epochs.get(key, 0) + 1
        return self._epochs[key]

    def barrier(self, buf: SymmetricBuffer, channel: int) -> None:
        e = _ext.ext()
        e.comm_barrier(buf.rank, buf.world, buf.bufs_dev, buf.signals_dev, channel, self._epoch((id(buf), channel)), self.status)
        ops._tick()

    def check(self) -> int:
        return int(self.status.item())

    def raise_if_failed(self) -> None:
        """Raise :class:`~triune_b200.parallel.elastic.CollectiveTimeout` when a bounded device-side wait ran out
        (a peer did not arrive); the CUDA context stays usable. Synchronises."""
        from .elastic import raise_on_status

        raise_on_status(self.check(), "fused tensor-parallel GEMM")


# ---------------------------------------------------------------------------------------------------- primitives
def _ag_gemm_fused(ctx: TPContext, x_shard: torch.Tensor, w: torch.Tensor, b_mn: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (y [M, N], gathered x [M, K] living in the symmetric workspace; valid until the call after next)."""
    rows, K = x_shard.shape
    M = rows * ctx.world
    N = w.shape[1] if b_mn else w.shape[0]
    buf = ctx.workspace("ag", M, K, 2)
    n = ctx._epoch(("ag", id(buf)))
    region = "a" if n % 2 else "b"  # double-buffered: peers may still read the previous call's slot
    gathered = buf.view(region, torch.bfloat16, M * K).view(M, K)
    gathered[ctx.rank * rows : (ctx.rank + 1) * rows].copy_(x_shard)
    ctx.barrier(buf, CH_AG)  # every rank's own slot is written (and, transitively, call n-1 finished everywhere)
    flags = ctx._flags.setdefault(id(buf), torch.zeros(max(4, M // 32), dtype=torch.int32, device=ctx.device))
    y = torch.empty(M, N, dtype=torch.bfloat16, device=ctx.device)
    _ext.ext().allgather_gemm(gathered, w, b_mn, y, buf.rank, buf.world, buf.bufs_dev, buf.offset(region), rows, flags, n, ctx.status)
    ops._tick()
    ctx.comm_bytes += (ctx.world - 1) * rows * K * 2
    return y, gathered


def _gemm_rs_fused(ctx: TPContext, x: torch.Tensor, w: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """x [M, Kp] (this rank's slice of the reduction), w [N, Kp] (or [Kp, N] when b_mn) -> y [M/tp, N] summed over ranks."""
    M = x.shape[0]
    N = w.shape[1] if b_mn else w.shape[0]
    rows = M // ctx.world
    f32 = ctx.rs_fp32
    elem = 4 if f32 else 2
    buf = ctx.workspace("rs", rows, N, elem)
    out = buf.view("a", torch.float32 if f32 else torch.bfloat16, rows * N).view(rows, N)
    key = (id(buf), rows, N, f32)
    if key not in ctx._cmaps:
        ptrs = [int(p) for p in buf.handle.buffer_ptrs]
        ctx._cmaps[key] = _ext.ext().peer_c_maps(ptrs, buf.offset("a"), rows, N, N, f32, out)
    out.zero_()
    ctx.barrier(buf, CH_RS_ZERO)  # every owner's buffer is zero before anyone adds into it
    _ext.ext().gemm_reduce_scatter(x, w, b_mn, buf.rank, buf.world, buf.bufs_dev, ctx._cmaps[key], rows, f32, ctx.status)
    ops._tick()
    ctx.barrier(buf, CH_RS_DONE)  # every rank's tiles have been added
    ctx.comm_bytes += (ctx.world - 1) * rows * N * elem
    return out.to(torch.bfloat16) if f32 else out.clone()


def _ag_gemm_nccl(ctx, x_shard, w, b_mn):
    rows, K = x_shard.shape
    gathered = torch.empty(rows * ctx.world, K, dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather_into_tensor(gathered, x_shard.contiguous(), group=ctx.group)
    return ops.gemm(gathered, w, b_mn=b_mn) if _ext.use_kernels(gathered, w) else gathered @ (w if b_mn else w.t()), gathered


def _gemm_rs_nccl(ctx, x, w, b_mn):
    y = ops.gemm(x, w, b_mn=b_mn) if _ext.use_kernels(x, w) else x @ (w if b_mn else w.t())
    out = torch.empty(y.shape[0] // ctx.world, y.shape[1], dtype=y.dtype, device=y.device)
    dist.reduce_scatter_tensor(out, y.contiguous(), group=ctx.group)
    return out


def _fusable(ctx: TPContext, *ts, rows: int) -> bool:
    return (ctx.mode == "fused" and all(t.is_cuda and t.dtype == torch.bfloat16 for t in ts) and rows % 128 == 0
            and all(t.shape[-1] % 8 == 0 for t in ts))


def ag_gemm(ctx: TPContext, x_shard, w, b_mn: bool = False):
    if ctx.world == 1:
        return (ops.gemm(x_shard, w, b_mn=b_mn) if _ext.use_kernels(x_shard, w) else x_shard @ (w if b_mn else w.t())), x_shard
    if _fusable(ctx, x_shard, w, rows=x_shard.shape[0]):
        return _ag_gemm_fused(ctx, x_shard.contiguous(), w, b_mn)
    return _ag_gemm_nccl(ctx, x_shard, w, b_mn)


def gemm_rs(ctx: TPContext, x, w, b_mn: bool = False):
    if ctx.world == 1:
        return ops.gemm(x, w, b_mn=b_mn) if _ext.use_kernels(x, w) else x @ (w if b_mn else w.t())
    if _fusable(ctx, x, w, rows=x.shape[0] // ctx.world):
        return _gemm_rs_fused(ctx, x.contiguous(), w, b_mn)
    return _gemm_rs_nccl(ctx, x, w, b_mn)


def _wgrad(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor):
    """dW[N, K] = dy[M, N]^T x[M, K], accumulated into ``w.main_grad`` when the optimizer arena provides it."""
    if _ext.use_kernels(dy, x):
        return ops._accumulate_weight_grad(w, dy.contiguous(), x.contiguous())
    return dy.t() @ x


# ---------------------------------------------------------------------------------------------------- autograd
class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx_, x_shard, w, tp: TPContext):
        y, gathered = ag_gemm(tp, x_shard, w)
        ctx_.tp = tp
        # the gathered activations live in a recycled workspace: keep an own copy for the weight gradient
        ctx_.save_for_backward(gathered.clone() if tp.world > 1 and tp.mode == "fused" else gathered, w)
        return y

    @staticmethod
    def backward(ctx_, dy):
        gathered, w = ctx_.saved_tensors
        dy = dy.contiguous()
        dx = gemm_rs(ctx_.tp, dy, w, b_mn=True) if ctx_.needs_input_grad[0] else None  # [M, N/tp] @ [N/tp, K] -> rows of dX
        dw = _wgrad(dy, gathered, w) if ctx_.needs_input_grad[1] else None
        return dx, dw, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx_, x, w, tp: TPContext):
        ctx_.tp = tp
        ctx_.save_for_backward(x, w)
        return gemm_rs(tp, x, w)

    @staticmethod
    def backward(ctx_, dy_shard):
        x, w = ctx_.saved_tensors
        dx, dy_full = ag_gemm(ctx_.tp, dy_shard.contiguous(), w, b_mn=True)  # gather(dY)[M, N] @ W[N, K/tp]
        dw = _wgrad(dy_full, x, w) if ctx_.needs_input_grad[1] else None
        return (dx if ctx_.needs_input_grad[0] else None), dw, None


class ColumnParallelLinear(nn.Module):
    """Weight rows (output features) are split over the group; input is the sequence-parallel row shard."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = False, dtype=torch.bfloat16):
        super().__init__()
        assert out_features % tp.world == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features // tp.world, in_features, dtype=dtype, device=tp.device))
        self.bias = nn.Parameter(torch.zeros(out_features // tp.world, dtype=dtype, device=tp.device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x_shard: torch.Tensor) -> torch.Tensor:
        y = _ColumnParallelFn.apply(x_shard, self.weight, self.tp)
        return y + self.bias if self.bias is not None else y


class RowParallelLinear(nn.Module):
    """Weight columns (input features) are split over the group; output is the sequence-parallel row shard of the sum."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = False, dtype=torch.bfloat16):
        super().__init__()
        assert in_features % tp.world == 0
        self.tp, self.in_features, self.out_features = tp, in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp.world, dtype=dtype, device=tp.device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=tp.device)) if bias else None
        nn.init.normal_(self.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = _RowParallelFn.apply(x, self.weight, self.tp)
        return y + self.bias if self.bias is not None else y  # bias added once, on the reduced rows


def shard_linear_weight(weight: torch.Tensor, tp_rank: int, tp_world: int, column: bool) -> torch.Tensor:
    """Slice of a full ``[out, in]`` weight for this rank (column parallel: rows; row parallel: columns)."""
    n = weight.shape[0 if column else 1] // tp_world
    return weight[tp_rank * n : (tp_rank + 1) * n].contiguous() if column else weight[:, tp_rank * n : (tp_rank + 1) * n].contiguous()
