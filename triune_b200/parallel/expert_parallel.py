"""Expert parallelism: experts are split over the group; tokens travel to their experts and back over NVLink.

The reference keeps every expert on one device (``MoE_FFN``, ``triune/model/moe.py:64-73``) and has no all-to-all. Here
``E`` experts are partitioned ``E / ep`` per rank and the two all-to-alls are done by kernels through peer memory:

  dispatch   ``ep_dispatch``: every (token, choice) row is stored straight into the owner's expert-major input buffer
             (segment = (local expert, source rank), fixed capacity per segment so no size exchange is needed for
             addressing), together with the slot its result must return to and the per-expert counts;
  experts    grouped GEMM-1 (+bias, GELU) over the valid 128-row tiles of the received segments;
  combine    ``gemm_scatter_rows``: grouped GEMM-2 whose epilogue adds the bias and stores every output row into the
             token owner's receive buffer; the owner then sums its k rows with the routing weights.

The backward pass is the same machinery run in reverse (gradient rows are dispatched to the experts, the data-gradient
GEMM scatters rows back), with expert weight gradients as local grouped-by-reduction GEMMs.
``mode="nccl"`` does the two all-to-alls with ``all_to_all_single`` around the single-GPU expert kernels: the baseline.
"""

from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _ext, ops
from ..ops import GEMM_GROUPED_K, GEMM_GROUPED_M, gemm
from .symm import SymmetricBuffer

CH_DISPATCH, CH_COMBINE = 3, 4


class EPContext:
    def __init__(self, num_experts: int, group=None, device=None, capacity_factor: float = 1.5, mode: str = "fused"):
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert num_experts % self.world == 0, "experts must divide evenly over the expert-parallel group"
        self.num_experts, self.experts_per_rank = num_experts, num_experts // self.world
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.capacity_factor, self.mode = capacity_factor, mode
        self._bufs: Dict[Tuple, SymmetricBuffer] = {}
        self._epochs: Dict[Tuple, int] = {}
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.comm_bytes = 0
        # The weight- and bias-gradient GEMMs reduce only over the 64-row blocks of each (expert, source rank) segment
        # that hold tokens (a run list built from the received counts on the device) instead of whole capacity ranges.
        self.bounded_wgrad = True

    def reduction_runs(self, cnt_all: torch.Tensor, cap: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(k_runs [El * W, 2] int32, run offsets [El + 1] int32) for ``ops.gemm(mode=GEMM_GROUPED_K, k_runs=...)``.

        ``cnt_all`` [W, El] holds the rows each source rank sent to each local expert; segment ``el * W + src`` of the
        expert-major buffer starts at row ``(el * W + src) * cap`` and holds ``min(count, cap)`` rows. No host read."""
        El, W = self.experts_per_rank, self.world
        cnt = cnt_all.view(W, El).t().reshape(-1).clamp(min=0, max=cap)
        blocks = torch.div(cnt + 63, 64, rounding_mode="floor").to(torch.int32)
        starts = torch.arange(El * W, device=cnt.device, dtype=torch.int32) * cap
        runs = torch.stack((starts, blocks), dim=1).contiguous()
        offs = (torch.arange(El + 1, device=cnt.device, dtype=torch.int32) * W).contiguous()
        return runs, offs

    def capacity(self, n_assign: int) -> int:
        """Rows reserved per (expert, source rank) segment: capacity_factor x the mean load, rounded up to 128."""
        return max(128, int(math.ceil(self.capacity_factor * n_assign / self.num_experts / 128.0)) * 128)

    def workspace(self, n_assign: int, d: int) -> Tuple[SymmetricBuffer, int]:
        cap = self.capacity(n_assign)
        key = (n_assign, d, cap)
        if key not in self._bufs:  # collective allocation: same sequence of shapes on every rank
            rows = self.experts_per_rank * self.world * cap
            self._bufs[key] = SymmetricBuffer({"xin": rows * d * 2, "dst": rows * 4, "cnt": self.world * self.experts_per_rank * 4,
                                               "recv": n_assign * d * 2}, self.device, self.group, use_multimem=False)
        return self._bufs[key], cap

    def barrier(self, buf: SymmetricBuffer, channel: int) -> None:
        k = (id(buf), channel)
        self._epochs[k] = self._epochs.get(k, 0) + 1
        _ext.ext().comm_barrier(buf.rank, buf.world, buf.bufs_dev, buf.signals_dev, channel, self._epochs[k], self.status)
        ops._tick()

    def check(self) -> int:
        return int(self.status.item())

    def raise_if_failed(self) -> None:
        """Raise :class:`~triune_b200.parallel.elastic.CollectiveTimeout` when a bounded device-side wait ran out
        (a peer did not arrive); the CUDA context stays usable. Synchronises."""
        from .elastic import raise_on_status

        raise_on_status(self.check(), "expert-parallel dispatch / combine")


def _positions(idx_flat: torch.Tensor, num_experts: int):
    """Position of every assignment among this rank's assignments to the same expert (in assignment order), and the
    per-expert counts. No host synchronisation.

    One stable sort by expert groups the assignments without disturbing their order inside a group; the position is
    then the distance to the start of the group. (A one-hot cumulative sum over [assignments, experts] computes the
    same thing but costs milliseconds per layer at 64 experts.)"""
    E = num_experts
    A = idx_flat.numel()
    dev = idx_flat.device
    key = torch.where(idx_flat >= 0, idx_flat, torch.full_like(idx_flat, E)).long()  # dropped assignments sort last
    e_sorted, order = torch.sort(key, stable=True)
    counts_all = torch.zeros(E + 1, device=dev, dtype=torch.int64).scatter_add_(0, key, torch.ones_like(key))
    starts = torch.cumsum(counts_all, 0) - counts_all
    rank_sorted = torch.arange(A, device=dev) - starts[e_sorted]
    pos = torch.empty(A, device=dev, dtype=torch.int64)
    pos[order] = torch.where(e_sorted < E, rank_sorted, torch.full_like(rank_sorted, -1))
    return pos.to(torch.int32).contiguous(), counts_all[:E].to(torch.int32).contiguous()


class _EPExpertsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, idx, wts, w1, b1, w2, b2, ep: EPContext):
        e = _ext.ext()
        T, d = x.shape
        K = idx.shape[1]
        A = T * K
        El, W = ep.experts_per_rank, ep.world
        buf, cap = ep.workspace(A, d)
        rows = El * W * cap
        idx_flat = idx.reshape(-1).to(torch.int32).contiguous()
        pos, counts = _positions(idx_flat, ep.num_experts)
        xin = buf.view("xin", torch.bfloat16, rows * d).view(rows, d)
        row_dst = buf.view("dst", torch.int32, rows)
        cnt_all = buf.view("cnt", torch.int32, W * El)
        recv = buf.view("recv", torch.bfloat16, A * d).view(A, d)
        e.ep_dispatch(x.contiguous(), idx_flat, pos, K, El, cap, buf.rank, W, buf.bufs_dev, buf.offset("xin"), buf.offset("dst"),
                      buf.offset("cnt"), counts, A)
        ep.barrier(buf, CH_DISPATCH)
        tile_group = torch.empty(rows // 128, dtype=torch.int32, device=x.device)
        e.ep_build_tiles(cnt_all, El, W, cap, tile_group, row_dst)
        e.ep_zero_invalid_rows(xin, cnt_all, El, W, cap)
        H = w1.shape[1]
        # Rows without a token must hold finite values (they meet zero rows in the weight-gradient GEMMs, and 0 * NaN
        # would poison them). The grouped GEMM writes every row of a tile it runs; only the rows past each segment's count
        # are zeroed afterwards (about a third of the buffer at capacity factor 1.5) instead of filling all of it first.
        dact = torch.empty(rows, H, dtype=x.dtype, device=x.device)
        h = torch.empty(rows, H, dtype=x.dtype, device=x.device)
        gemm(xin, w1, h, bias=b1, gelu=True, aux_out=dact, mode=GEMM_GROUPED_M, tile_group=tile_group)
        e.ep_zero_invalid_rows(h, cnt_all, El, W, cap)
        e.ep_zero_invalid_rows(dact, cnt_all, El, W, cap)
        # Copies for the backward pass are taken BEFORE this rank signals the combine barrier: once a peer has passed
        # that barrier it may start its next dispatch and overwrite these regions.
        xin_saved, dst_saved, cnt_saved = xin.clone(), row_dst.clone(), cnt_all.clone()
        e.gemm_scatter_rows(h, w2, False, b2, None, tile_group, row_dst, A, buf.rank, W, buf.bufs_dev, buf.offset("recv"), d, ep.status)
        ops._tick(5)
        ep.barrier(buf, CH_COMBINE)
        keep = (pos >= 0) & (pos < cap)
        slot = torch.where(keep, torch.arange(A, device=x.device, dtype=torch.int32), torch.full_like(pos, -1)).view(T, K).contiguous()
        wk = wts.float().contiguous()
        out = e.combine_rows(recv, slot, wk, None, 0.0)
        ops._tick()
        ctx.ep, ctx.cap, ctx.buf = ep, cap, buf
        ctx.save_for_backward(xin_saved, dact, h, tile_group, dst_saved, cnt_saved, idx_flat, pos, counts, slot, wk,
                              recv.clone(), w1, b1, w2, b2)
        ep.comm_bytes += 2 * A * d * 2
        return out

    @staticmethod
    def backward(ctx, dout):
        (xin, dact, h, tile_group, row_dst, cnt_all, idx_flat, pos, counts, slot, wk, recv, w1, b1, w2, b2) = ctx.saved_tensors
        ep, cap, buf = ctx.ep, ctx.cap, ctx.buf
        e = _ext.ext()
        dout = dout.contiguous()
        T, d = dout.shape
        K = slot.shape[1]
        A = T * K
        El, W = ep.experts_per_rank, ep.world
        rows = El * W * cap
        dw = e.row_dots(dout, recv, slot)  # d loss / d routing weight
        src_tok = (torch.arange(A, device=dout.device, dtype=torch.int32) // K).contiguous()
        drows = e.gather_rows(dout, src_tok, (wk.view(-1) * (slot.view(-1) >= 0)).contiguous())  # w[a] * dout[t(a)]
        dyin = buf.view("xin", torch.bfloat16, rows * d).view(rows, d)  # the forward copy of this region was saved
        live_dst = buf.view("dst", torch.int32, rows)
        e.ep_dispatch(drows, idx_flat, pos, 1, El, cap, buf.rank, W, buf.bufs_dev, buf.offset("xin"), buf.offset("dst"),
                      buf.offset("cnt"), counts, A)
        ep.barrier(buf, CH_DISPATCH)
        e.ep_zero_invalid_rows(dyin, cnt_all, El, W, cap)
        live_dst.copy_(row_dst)  # same routing as the forward, including the rows invalidated there
        H = w1.shape[1]
        dpre = torch.empty(rows, H, dtype=dout.dtype, device=dout.device)
        gemm(dyin, w2, dpre, b_mn=True, dgelu_aux=dact, mode=GEMM_GROUPED_M, tile_group=tile_group)
        e.ep_zero_invalid_rows(dpre, cnt_all, El, W, cap)  # rows of skipped tiles (the others are 0 * finite already)
        if ep.bounded_wgrad:
            # rows past a segment's count are zero in every operand below, so whole 64-row blocks are safe to include
            runs, offs = ep.reduction_runs(cnt_all, cap)
        else:
            runs, offs = None, (torch.arange(El + 1, device=dout.device, dtype=torch.int32) * (W * cap)).contiguous()
        ones = torch.ones(rows, 8, device=dout.device, dtype=dout.dtype)

        def wgrad(w, a, b):
            mg = getattr(w, "main_grad", None)
            if mg is not None:
                gemm(a, b, mg, a_mn=True, b_mn=True, accumulate=True, mode=GEMM_GROUPED_K, group_offsets=offs, num_groups=El,
                     k_runs=runs)
                return None
            return gemm(a, b, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_offsets=offs, num_groups=El, k_runs=runs)

        def bgrad(bp, a):
            s = gemm(ones, a, a_mn=True, b_mn=True, mode=GEMM_GROUPED_K, group_offsets=offs, num_groups=El, out_dtype=torch.float32,
                     k_runs=runs)[:, 0, :]
            mg = getattr(bp, "main_grad", None)
            if mg is not None:
                mg.add_(s)
                return None
            return s.to(bp.dtype)

        dyin_c = dyin.clone()  # the region is reused below by nobody, but the wgrad reads must not race a later layer
        dw2, db2 = wgrad(w2, dyin_c, h), bgrad(b2, dyin_c)
        dw1, db1 = wgrad(w1, dpre, xin), bgrad(b1, dpre)
        e.gemm_scatter_rows(dpre, w1, True, None, None, tile_group, live_dst, A, buf.rank, W, buf.bufs_dev, buf.offset("recv"), d, ep.status)
        ops._tick(8)
        ep.barrier(buf, CH_COMBINE)
        recv2 = buf.view("recv", torch.bfloat16, A * d).view(A, d)
        dx = e.combine_rows(recv2, slot, torch.ones_like(wk), None, 0.0)
        ep.comm_bytes += 2 * A * d * 2
        return dx, None, dw.to(wk.dtype), dw1, db1, dw2, db2, None


def _experts_nccl(x, idx, wts, w1, b1, w2, b2, ep: EPContext):
    """Baseline: tokens sorted by destination rank, ``all_to_all_single`` there and back, local expert kernels."""
    T, d = x.shape
    K = idx.shape[1]
    El, W = ep.experts_per_rank, ep.world
    flat = idx.reshape(-1)
    dest = (flat // El).clamp(0, W - 1)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=W)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=ep.group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()  # host sync: part of what the fused path avoids
    xs = x[(order // K)]
    es = (flat[order] % El).to(torch.int64)
    xr = torch.empty(sum(rc), d, dtype=x.dtype, device=x.device)
    er = torch.empty(sum(rc), dtype=torch.int64, device=x.device)
    dist.all_to_all_single(xr, xs.contiguous(), rc, sc, group=ep.group)
    dist.all_to_all_single(er, es.contiguous(), rc, sc, group=ep.group)
    yr = ops.moe_experts(xr, er.view(-1, 1), torch.ones(er.numel(), 1, device=x.device), None, w1, b1, w2, b2)
    ys = torch.empty(A := T * K, d, dtype=x.dtype, device=x.device)
    dist.all_to_all_single(ys, yr.contiguous(), sc, rc, group=ep.group)
    y = torch.empty_like(ys)
    y[order] = ys
    return (y.view(T, K, d).float() * wts.float().unsqueeze(-1)).sum(1).to(x.dtype)


def ep_experts(x, idx, wts, w1, b1, w2, b2, ep: EPContext):
    """x [T, d] local tokens; idx / wts [T, k] global expert ids and routing weights; w1 [E/ep, H, d] ... local experts."""
    if ep.world == 1:
        return ops.moe_experts(x, idx, wts, None, w1, b1, w2, b2)
    if ep.mode == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
        return _EPExpertsFn.apply(x, idx, wts, w1, b1, w2, b2, ep)
    return _experts_nccl(x, idx, wts, w1, b1, w2, b2, ep)


class ExpertParallelMoE(nn.Module):
    """MoE FFN whose routed experts are partitioned over the expert-parallel group; the router is replicated."""

    def __init__(self, dim: int, hidden: int, num_experts: int, top_k: int, ep: EPContext, dtype=torch.bfloat16):
        super().__init__()
        self.dim, self.hidden, self.num_experts, self.top_k, self.ep = dim, hidden, num_experts, top_k, ep
        El = ep.experts_per_rank
        dev = ep.device
        self.router = nn.Linear(dim, num_experts, device=dev, dtype=dtype)
        self.register_buffer("expert_bias", torch.zeros(num_experts, device=dev, dtype=torch.float32))
        self.w1 = nn.Parameter(torch.empty(El, hidden, dim, device=dev, dtype=dtype))
        self.b1 = nn.Parameter(torch.zeros(El, hidden, device=dev, dtype=dtype))
        self.w2 = nn.Parameter(torch.empty(El, dim, hidden, device=dev, dtype=dtype))
        self.b2 = nn.Parameter(torch.zeros(El, dim, device=dev, dtype=dtype))
        nn.init.normal_(self.w1, std=0.02)
        nn.init.normal_(self.w2, std=0.02)
        nn.init.normal_(self.router.weight, std=0.02)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, self.dim)
        logits = self.router(x2).float()
        idx, w, _ = ops.ref.moe_route(logits, self.expert_bias, self.top_k)
        return ep_experts(x2, idx, w.to(torch.float32), self.w1, self.b1, self.w2, self.b2, self.ep).view(shape)


class EPMoE_FFN(nn.Module):
    """Drop-in replacement for :class:`triune_b200.models.moe.MoE_FFN` holding only this rank's experts.

    The router, the selection bias and the shared expert are replicated; routed experts ``[rank * E/ep, (rank+1) * E/ep)``
    live here. Capacity is the per-(expert, source rank) segment size of the dispatch buffers
    (``EPContext.capacity_factor``), which plays the role of the reference's ``ceil(N / E * 1.5)`` admission limit.
    """

    def __init__(self, moe: nn.Module, ep: EPContext):
        super().__init__()
        self.ep, self.dim, self.num_experts, self.top_k = ep, moe.dim, moe.num_experts, moe.top_k
        self.shared_scale = moe.shared_scale
        lo, hi = ep.rank * ep.experts_per_rank, (ep.rank + 1) * ep.experts_per_rank
        self.router, self.shared = moe.router, moe.shared
        self.register_buffer("expert_bias", moe.expert_bias.detach().clone())
        # statistics of the full layer, carried only so that a merged checkpoint has every key of the unsharded layer;
        # kept under other attribute names because the optimizer's steering tier reads `last_centroids` of the module
        # that owns the experts, and these are neither sliced to the local experts nor updated here
        self._carried = {name: getattr(moe, name).detach().clone() for name in ("expert_load_ratio", "last_centroids", "_global_step")
                         if hasattr(moe, name)}
        for name in ("w1", "b1", "w2", "b2"):
            setattr(self, name, nn.Parameter(getattr(moe, name).detach()[lo:hi].clone()))
        self._pending_bias_update = None

    def forward(self, x: torch.Tensor, update_stats: bool = True) -> torch.Tensor:
        B, T, D = x.shape
        x2 = x.reshape(B * T, D)
        logits = ops.linear(x2, self.router.weight, self.router.bias).float()
        if ops.route_plan_supported(logits, self.top_k):
            idx, w, _keep, _plan = ops.moe_route_plan(logits, self.expert_bias, self.top_k, 1.0, None)
        else:
            idx, w, _ = ops.moe_route(logits, self.expert_bias, self.top_k, 1.0)
        out = ep_experts(x2, idx, w.float(), self.w1, self.b1, self.w2, self.b2, self.ep)
        if self.shared is not None:
            out = out + self.shared_scale * self.shared(x2)
        return out.reshape(B, T, D)

    # ------------------------------------------------------------------ rank-local checkpoints
    def checkpoint_pieces(self, prefix: str):
        """This rank's experts under the unsharded layer's per-expert keys (``experts.{e}.{0,2}.{weight,bias}``), as
        views of the live parameters (``trainer/sharded_checkpoint.py``)."""
        lo = self.ep.rank * self.ep.experts_per_rank
        for e in range(self.ep.experts_per_rank):
            yield (f"{prefix}experts.{lo + e}.0.weight", None, 0, 0, 0, self.w1[e])
            yield (f"{prefix}experts.{lo + e}.0.bias", None, 0, 0, 0, self.b1[e])
            yield (f"{prefix}experts.{lo + e}.2.weight", None, 0, 0, 0, self.w2[e])
            yield (f"{prefix}experts.{lo + e}.2.bias", None, 0, 0, 0, self.b2[e])

    def checkpoint_replicated(self, prefix: str):
        out = {f"{prefix}expert_bias": self.expert_bias}
        for n, t in self._carried.items():
            if t.device != self.expert_bias.device:
                t = self._carried[n] = t.to(self.expert_bias.device)
            out[f"{prefix}{n}"] = t
        for k, v in self.router.state_dict().items():
            out[f"{prefix}router.{k}"] = v
        if self.shared is not None:
            for k, v in self.shared.state_dict().items():
                out[f"{prefix}shared.{k}"] = v
        return out

    def step_bias(self) -> None:  # selection-bias updates need global counts; kept fixed under expert parallelism
        self._pending_bias_update = None


def shard_experts(model: nn.Module, ep: EPContext) -> int:
    """Replace every ``MoE_FFN`` of ``model`` by an :class:`EPMoE_FFN` with this rank's slice of its experts. Every rank
    must hold the same full model when this is called (e.g. same seed or a broadcast). Returns the number of layers."""
    from ..models.moe import MoE_FFN

    n = 0
    for parent in model.modules():
        for name, child in list(parent.named_children()):
            if isinstance(child, MoE_FFN):
                setattr(parent, name, EPMoE_FFN(child, ep))
                n += 1
    return n


def allreduce_replicated_grads(model: nn.Module, group=None) -> None:
    """Average the gradients of parameters that every rank holds (everything except the local experts): with expert
    parallelism each rank sees different tokens, so replicated weights need data-parallel averaging while expert
    gradients are already complete on their owner."""
    group = group if group is not None else dist.group.WORLD
    world = dist.get_world_size(group)
    expert_ids = {id(p) for m in model.modules() if isinstance(m, EPMoE_FFN) for p in (m.w1, m.b1, m.w2, m.b2)}
    grads = [p.grad for p in model.parameters() if p.grad is not None and id(p) not in expert_ids]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    flat.div_(world)
    off = 0
    for g in grads:
        n = g.numel()
        g.copy_(flat[off : off + n].view_as(g).to(g.dtype))
        off += n
